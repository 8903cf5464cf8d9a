"""Benchmark of the fused-layer step (data-parallel over token rows).

    python bench.py --gpus N --steps K --warmup W          # this backend, one rank per GPU
    python bench.py --impl reference ...                   # the CPU path on the host cores

Workload (N=1 and per GPU at N>1): the full fused-layer step of a random-init depth-20 GPT
(n_embd 1280, 10 heads x 128, seq 2048, vocab 32768, 16 sequences per GPU, LayerNorm + GELU
MLP + RoPE + tied embedding + fused linear+CE), synthetic seeded data.  One "step" = every fused
layer kernel of a training step, forward and backward, plus the gradient allreduce at N>1.

Prints ONE JSON line on rank 0.  `value` is tokens/s of the whole job with inputs resident in
HBM; `e2e` is the same metric with the step's token ids and targets copied from pinned host
memory and the loss read back inside the timed region.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fused_layer_tokens_per_s"
UNIT = "tokens/s"
CONFIG_IDLE_S = 4.0   # idle between the timed steps and the per-config kernel timings of the default run


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--ce-precision", default="3xtf32", choices=["fp32", "3xtf32", "bf16", "bf16x3"])
    ap.add_argument("--no-bf16-mode", action="store_true", help="skip the extra timing of the bf16 CE mode")
    ap.add_argument("--grad-wire", default="fp32", choices=["fp32", "bf16"],
                    help="N>1: form in which the tied table gradient crosses the links (bf16 = half the bytes)")
    # reduced shapes for profiler captures and tests; the defaults are the benchmark workload
    ap.add_argument("--layers", type=int, default=20)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--vocab", type=int, default=32768)
    ap.add_argument("--n-embd", type=int, default=1280)
    ap.add_argument("--workload", default="step", choices=["step", "kernels"],
                    help="step: the fused-layer step (the benchmark); kernels: one JSON line per fused layer "
                         "kernel at the shapes of BASELINE configs 1-4, each against its own roofline")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-config-kernels", action="store_true",
                    help="step workload: skip the per-kernel timings at the shapes of configs 1-4 (`configs` key)")
    ap.add_argument("--only", default="", help="--workload kernels: comma-separated sections (cfg1,gelu,cfg3,cfg4,cfg2,next,rmsce)")
    ap.add_argument("--cpu-sample-tokens", type=int, default=0,
                    help="token rows of the CPU sample (0: sized so that the CPU run stays within a few minutes)")
    ap.add_argument("--cpu-sample-layers", type=int, default=2, help="numpy-port fallback only")
    return ap.parse_args()


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def workload_name(a):
    return (f"gpt_fused_layer_step depth{a.layers} n_embd{a.n_embd} heads{a.n_embd // 128}x128 seq{a.seq_len} "
            f"vocab{a.vocab} batch{a.batch}/gpu")


def bench_config(a, world):
    """The `config` object of the JSON line; both arms (this backend and the CPU reference) print the same one."""
    return {"workload": workload_name(a), "tokens_per_gpu": a.batch * a.seq_len, "ce_precision": a.ce_precision,
            "vocab_chunk": 4096, "parallelism": f"dp{world} token-row sharded",
            "l2": "every streamed buffer is larger than the L2 cache; no flush needed"}


# --------------------------------------------------------------------------------------
# CPU path: the numpy restatement of the reference's CPU backend, on a bounded sample
# --------------------------------------------------------------------------------------
def cpu_sample_step(a, tokens, layers, seed=1238):
    """One fused-layer step on the host for `tokens` token rows and `layers` of the a.layers
    layers; the per-layer time is scaled to the full depth.  Returns (seconds_full_depth,
    description)."""
    from oracle import fused_layers as O
    C, V, I, H, D = a.n_embd, a.vocab, 4 * a.n_embd, a.n_embd // 128, 128
    T = min(a.seq_len, tokens)
    B = max(tokens // T, 1)
    n = B * T
    rng = np.random.default_rng(seed)
    f = np.float32
    ids = rng.integers(0, V, size=(B, T)).astype(np.int32)
    tg = rng.integers(0, V, size=n).astype(np.int32)
    table = (0.02 * rng.standard_normal((V, C), dtype=f)).astype(f)
    gam = (1 + 0.02 * rng.standard_normal(C)).astype(f)
    bet = (0.02 * rng.standard_normal(C)).astype(f)
    r = rng.standard_normal((n, C), dtype=f)
    u = rng.standard_normal((n, I), dtype=f)
    q = rng.standard_normal((B, T, H, D), dtype=f)
    kk = rng.standard_normal((B, T, H, D), dtype=f)
    dy = rng.standard_normal((n, C), dtype=f)
    dg = rng.standard_normal((n, I), dtype=f)
    cos, sin = O.rope_tables(T, D, 1e5)
    zc = np.zeros(C, f)

    t0 = time.perf_counter()
    x = O.gather_forward(ids, table).reshape(n, C)
    t_head = time.perf_counter() - t0
    t0 = time.perf_counter()
    hs = []
    for _ in range(layers):
        h1, y1, _, _ = O.add_layernorm_forward(x, r, gam, bet, 1e-5)
        O.rope_apply(q, cos, sin, -1); O.rope_apply(kk, cos, sin, -1)
        h2, y2, _, _ = O.add_layernorm_forward(h1, r, gam, bet, 1e-5)
        O.gelu_forward(u)
        hs.append((h1, h2))
        x = h2
    t_layers = time.perf_counter() - t0
    t0 = time.perf_counter()
    hf, yf, _, _ = O.add_layernorm_forward(x, r, gam, bet, 1e-5)
    res = O.flce_masked(yf, table, tg)                      # forward and backward of the head
    dh, _, _ = O.layernorm_backward(hf, gam, res["dX"], 1e-5, np.zeros_like(hf), zc, zc)
    t_head += time.perf_counter() - t0
    t0 = time.perf_counter()
    for h1, h2 in reversed(hs):
        O.gelu_backward(u, dg, np.zeros_like(u))
        dh, _, _ = O.layernorm_backward(h2, gam, dy, 1e-5, dh, zc, zc)
        O.rope_apply(q, cos, sin, +1); O.rope_apply(kk, cos, sin, +1)
        dh, _, _ = O.layernorm_backward(h1, gam, dy, 1e-5, dh, zc, zc)
    t_layers += time.perf_counter() - t0
    t0 = time.perf_counter()
    O.gather_backward(ids, dh.reshape(B, T, C), res["dW"])
    t_head += time.perf_counter() - t0
    total = t_head + t_layers * (a.layers / layers)
    desc = (f"{n} token rows, {layers} of {a.layers} layers timed and scaled x{a.layers / layers:g}, head "
            f"(gather, final LN, fused linear+CE fwd+bwd, scatter-add) at full vocab {V}")
    return n, total, desc


def cpu_reference_sample(a, tokens, warmup, steps):
    """The fused-layer step on the host with the reference's own CPU backend (`oracle/_ref`, through
    oracle/ref_timing.py) on a sample of `tokens` token rows at full depth and vocabulary.  Returns
    (tokens, mean seconds per step, cpu_baseline dict without "value") or None when oracle/_ref is absent."""
    from oracle import ref_loader
    if not ref_loader.available():
        return None
    from oracle import ref_timing as RT
    S = RT.FusedLayerStepSample(a.layers, a.n_embd, a.n_embd // 128, 128, a.seq_len, a.vocab, tokens)
    for _ in range(warmup):
        S.step()
    t = [S.step() for _ in range(max(steps, 1))]
    return S.tokens, sum(t) / len(t), {"unit": UNIT, "cores": S.threads, "kind": "reference", "sample": S.description}


def cpu_port_sample(a, tokens):
    """Fallback when oracle/_ref does not exist: the numpy restatement (oracle/fused_layers.py)."""
    n, t, desc = cpu_sample_step(a, tokens, a.cpu_sample_layers)
    return n, t, {"unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                  "sample": desc + f"; numpy restatement of the reference CPU backend (oracle/fused_layers.py), numpy {np.__version__}"}


def run_reference(a):
    """`--impl reference`: the reference's CPU implementation of the path on this host's cores.  Each
    step is a bounded sample of the workload (fewer token rows; full depth, full vocabulary); `value`
    is tokens/s of that sample, `ms_per_step` its measured wall time - nothing is extrapolated."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(a.gpus)))
    tokens = a.cpu_sample_tokens
    if tokens <= 0:
        # about 3.3 ms per token row and step on 8-16 cores: keep (warmup + steps) steps near two minutes
        tokens = int(36000 / max(a.steps + a.warmup, 1)) // 256 * 256
        tokens = min(max(tokens, 256), 2048)
    res = cpu_reference_sample(a, tokens, a.warmup, a.steps)
    if res is None:
        for _ in range(a.warmup):
            cpu_port_sample(a, tokens)
        runs = [cpu_port_sample(a, tokens) for _ in range(a.steps)]
        res = (runs[0][0], sum(r[1] for r in runs) / len(runs), runs[0][2])
    n, sec, cpu = res
    value = n / sec
    cpu["value"] = value
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": 1e3 * sec, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": bench_config(a, world),
        "cpu_baseline": cpu,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,utilization.gpu")

    def __init__(self, gpu_index):
        self.proc = None
        self.gpu_index = gpu_index      # an index in nvidia-smi's order, or a "GPU-<uuid>" string
        self.path = f"/tmp/ag_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.out,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()      # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, mx, util, reasons = [], [], [], set()
        try:
            with open(self.path) as f:
                for ln in f:
                    p = [x.strip() for x in ln.split(",")]
                    if len(p) < 9:
                        continue
                    try:
                        sm.append(float(p[1])); mx.append(float(p[2]))
                    except ValueError:
                        continue
                    try:
                        util.append(float(p[9]))
                    except (ValueError, IndexError):
                        util.append(-1.0)
                    for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                       p[5:9]):
                        if v.lower().startswith("active"):
                            reasons.add(name)
            os.remove(self.path)
        except Exception:
            pass
        # "under load" = the samples at which the GPU reported at least half utilisation (the sampler also runs
        # through set-up and through the CPU baseline); without such a reading, all samples
        load = [c for c, u in zip(sm, util) if u >= 50.0]
        if len(load) < 3:
            load = sm
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_under_load": len(load)}


# --------------------------------------------------------------------------------------
def run_b200(a):
    import torch
    import torch.distributed as dist

    import autograd_b200 as ag
    from autograd_b200 import dp
    from autograd_b200.step import FusedLayerStep, StepConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx, alloc, be = ag.create(local, stream.cuda_stream)
    peaks = load_peaks()

    prec = {"fp32": ag.AG_CE_FP32, "3xtf32": ag.AG_CE_3XTF32, "bf16": ag.AG_CE_BF16,
            "bf16x3": ag.AG_CE_BF16X3}[a.ce_precision]
    cfg = StepConfig(n_layer=a.layers, n_embd=a.n_embd, n_head=a.n_embd // 128, head_dim=128, seq_len=a.seq_len,
                     vocab=a.vocab, batch=a.batch, ce_precision=prec)

    def fill_normal(addr, n, seed, std):
        g = torch.Generator(device=f"cuda:{local}")
        g.manual_seed(seed * 1000 + rank)
        dp.as_torch(addr, n, local).normal_(0.0, std, generator=g)

    step = FusedLayerStep(ctx, alloc, be, cfg, seed=1238 + rank, fill_normal=fill_normal)
    Nn = cfg.tokens
    buckets = [dp.as_torch(addr, n, local) for addr, n in step.grad_buckets()]
    wires = None
    if world > 1 and a.grad_wire == "bf16":  # the small dgamma/dbeta bucket stays fp32
        wires = [None, dp.Bf16Wire.for_device(ctx, alloc, *step.grad_buckets()[1], local)]
    # two allreduces per step: [all dgamma/dbeta | loss scalar] and the tied table gradient
    reducer = dp.GradAllReducer(buckets, wires=wires) if world > 1 else None
    comm_timer = [None]
    if reducer is not None:
        ctx.fill_f32(step.dloss, reducer.grad_scale, 1)

    # pinned host batches (distinct per step so that nothing is cached across steps)
    n_batches = max(a.steps, 1)
    host = ctx.alloc_host(n_batches * 2 * Nn * 4)
    host_np = np.ctypeslib.as_array(ctypes.cast(host, ctypes.POINTER(ctypes.c_int32)), shape=(n_batches, 2, Nn))
    rng = np.random.default_rng(4242 + rank)
    host_np[:] = rng.integers(0, cfg.vocab, size=host_np.shape, dtype=np.int32)

    def load(i):
        b = i % n_batches
        step.load_batch(host + (b * 2) * Nn * 4, host + (b * 2 + 1) * Nn * 4)

    def one_step(i, e2e):
        if e2e:
            load(i)
        step.step()
        if reducer is not None:
            reducer.reduce(comm_timer[0])
        if e2e:
            return step.read_loss(world)
        return None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # The clock sampler starts before the warm-up steps: nvidia-smi takes the driver's lock while it
    # initialises, which would otherwise stall this process's launches inside the timed region.  The
    # warm-up steps run the same kernels, so its samples are under load as well.
    gpu_id = local
    try:   # nvidia-smi's order need not be CUDA's: name the device by its UUID where torch exposes it
        u = str(torch.cuda.get_device_properties(local).uuid)
        u = u if u.startswith("GPU-") else "GPU-" + u
        ok = subprocess.run(["nvidia-smi", "-i", u, "--query-gpu=index", "--format=csv,noheader"],
                            capture_output=True, text=True, timeout=20)
        if ok.returncode == 0 and ok.stdout.strip():
            gpu_id = u
    except Exception:
        pass
    sampler = ClockSampler(gpu_id)
    sampler.start()
    load(0)
    for i in range(a.warmup):
        one_step(i, e2e=True)
    ctx.check_status()

    # Event indices: 0, 1 bracket the timed regions, the family timer uses [16, TC_BASE), the per-launch
    # events of the tensor-core GEMM [TC_BASE, ...).  The pool is grown to its final size here: growing
    # it at the first use inside a pass would delay the ranks by different amounts, and the early ranks
    # would then wait for the late ones inside their timed region (at the allreduce).
    EV0, EV1 = 0, 1
    TC_BASE = 1 << 14
    step.timer.base = 16
    ctx.event_record(TC_BASE + 4 * 64 * (a.steps + 1))

    # ---- device-resident timing: exactly `steps` steps between two events, nothing else in the stream
    barrier()
    launches0 = ctx.launch_count
    ctx.event_record(EV0)
    for i in range(a.steps):
        one_step(i, e2e=False)
    ctx.event_record(EV1)
    barrier()
    ms_dev = ctx.event_elapsed_ms(EV0, EV1)
    launches = ctx.launch_count - launches0

    # ---- the same steps once more with an event pair around every kernel family and around every
    # tensor-core GEMM launch: the breakdown (`kernels`, `roofline`).  The extra events keep consecutive
    # kernels from overlapping their launch, so this pass is a little slower than the one above.
    step.timer.reset()
    step.timer.enabled = True
    if reducer is not None:
        comm_timer[0] = dp.CommTimer()      # an event pair around each allreduce of this pass
    barrier()
    ctx.tc_timing(True, TC_BASE)
    ctx.event_record(EV0)
    for i in range(a.steps):
        one_step(i, e2e=False)
    ctx.event_record(EV1)
    barrier()
    ctx.tc_timing(False)
    ms_breakdown = ctx.event_elapsed_ms(EV0, EV1)
    step.timer.enabled = False
    comm_ms = comm_timer[0].totals_ms() if comm_timer[0] is not None else {}
    comm_timer[0] = None
    fam = step.timer.totals_ms()
    tc_n = ctx.tc_timing_count()
    tc_ms = [ctx.event_elapsed_ms(TC_BASE + 2 * i, TC_BASE + 2 * i + 1) for i in range(tc_n)]

    # ---- end-to-end timing: h2d of ids/targets and d2h of the loss every step
    barrier()
    ctx.event_record(EV0)
    t_wall = time.perf_counter()
    last_loss = None
    for i in range(a.steps):
        last_loss = one_step(i, e2e=True)
    ctx.event_record(EV1)
    barrier()
    t_wall = time.perf_counter() - t_wall
    ms_e2e = max(ctx.event_elapsed_ms(EV0, EV1), 1e3 * t_wall)
    clocks = sampler.stop()
    ctx.check_status()

    # ---- the stated faster modes of the CE head, same step otherwise; reported beside the headline,
    # never as it: bf16 operands (2e-2), and bf16 (hi, lo) pairs with three MMAs (loss 1e-5, dX and dW 1e-4)
    alt_ms = {}
    if a.ce_precision == "3xtf32" and not a.no_bf16_mode:
        for name, prec_alt in (("bf16", ag.AG_CE_BF16), ("bf16x3", ag.AG_CE_BF16X3)):
            step.desc = ctx.flce_desc(Nn, cfg.n_embd, cfg.vocab, vocab_chunk=cfg.ce_vocab_chunk, precision=prec_alt)
            assert ctx.flce_scratch_bytes(step.desc) <= step.flce_bytes
            for i in range(max(a.warmup, 3)):
                one_step(i, e2e=False)
            barrier()
            ctx.event_record(EV0)
            for i in range(a.steps):
                one_step(i, e2e=False)
            ctx.event_record(EV1)
            barrier()
            alt_ms[name] = ctx.event_elapsed_ms(EV0, EV1)
            ctx.check_status()
    ms_bf16 = alt_ms.get("bf16")
    ms_x3 = alt_ms.get("bf16x3")

    comm = None
    if world > 1:
        # per-rank figures: device time of the timed steps, time inside the collectives, time of the
        # step's own kernels in the breakdown pass
        fam_ms = sum(v[1] for v in fam.values())
        mine = torch.tensor([ms_dev, comm_ms.get("bucket0", 0.0), comm_ms.get("bucket1", 0.0), fam_ms],
                            device=f"cuda:{local}", dtype=torch.float64)
        allr = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        per = torch.stack(allr).cpu().numpy() / a.steps
        comm = {"small_bucket_and_loss_ms": round(float(per[:, 1].max()), 4),
                "table_gradient_bucket_ms": round(float(per[:, 2].max()), 4),
                # the first collective of a step is where a rank waits for the slowest one: its shortest time
                # over the ranks is what the exchange itself costs, the rest is waiting
                "small_bucket_and_loss_ms_min_over_ranks": round(float(per[:, 1].min()), 4),
                "table_gradient_bucket_ms_min_over_ranks": round(float(per[:, 2].min()), 4),
                "kernel_skew_ms": round(float(per[:, 3].max() - per[:, 3].min()), 4),
                "rank_skew_ms": round(float(per[:, 0].max() - per[:, 0].min()), 4),
                "per_rank_step_ms": [round(float(v), 3) for v in per[:, 0]],
                "per_rank_kernel_ms": [round(float(v), 3) for v in per[:, 3]],
                "per_rank_small_bucket_ms": [round(float(v), 3) for v in per[:, 1]],
                "per_rank_table_bucket_ms": [round(float(v), 3) for v in per[:, 2]],
                "note": "CUDA-event pairs around each allreduce in the breakdown pass, per step; max over ranks unless "
                        "named otherwise.  The time inside a collective includes waiting for the slowest rank to arrive: "
                        "the ranks' steps run at the power cap and differ (per_rank_kernel_ms = sum of the step's own "
                        "kernel families, kernel_skew_ms its spread).  rank_skew_ms = max - min over ranks of the device "
                        "time of the timed steps (small, since every step ends in a collective)"}
        t = torch.tensor([ms_dev, ms_e2e, ms_bf16 or 0.0, ms_x3 or 0.0], device=f"cuda:{local}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_dev, ms_e2e = float(t[0]), float(t[1])
        ms_bf16 = float(t[2]) if ms_bf16 is not None else None
        ms_x3 = float(t[3]) if ms_x3 is not None else None

    # ---- the kernels of BASELINE configs 1-4, each alone at its stated shape (rank 0 of a 1-GPU run):
    # compact per-kernel figures in the same line, so that they come from the same run as the headline
    device_bytes = step.device_bytes
    alg = step.algorithmic_bytes()
    useful, executed = step.flce_flops()
    step.close()
    config_lines = None
    if world == 1 and not a.no_config_kernels:
        config_lines = []
        # these kernels are stated (and parity-tested) alone, so they are timed on a GPU that has left the
        # power-capped state of the step: a few seconds idle, bandwidth kernels first, the CE head last
        torch.cuda.synchronize()
        time.sleep(CONFIG_IDLE_S)
        a_k = argparse.Namespace(**vars(a))
        a_k.only = "cfg1,cfg3,cfg4,cfg2"
        run_kernels(a_k, env=(ctx, alloc, be), dev_index=local, collect=config_lines, steps=30, warmup=10,
                    cfg2_modes=("3xtf32",))

    if rank == 0:
        tokens = Nn * world
        ms_step = ms_dev / a.steps
        value = tokens / (ms_step / 1e3)
        e2e_value = tokens / (ms_e2e / a.steps / 1e3)
        kernels = {}
        for name, (count, total_ms) in sorted(fam.items()):
            per_step_ms = total_ms / a.steps
            ent = {"launch_groups_per_step": count // a.steps, "ms_per_step": round(per_step_ms, 4)}
            if name in alg:
                gbs = alg[name] / (per_step_ms / 1e3) / 1e9
                ent.update({"bound": "hbm", "achieved_gbs": round(gbs, 1), "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 4)})
            elif name in ("flce_fwd", "flce_bwd"):
                share = 1.0 if name == "flce_fwd" else 3.0
                u = useful * (share / 4.0) if name == "flce_bwd" else useful / 3.0
                tf = u / (per_step_ms / 1e3) / 1e12
                ent.update({"bound": "tensor", "useful_tflops": round(tf, 2)})
            kernels[name] = ent
        # dominant kernel family by time
        dom = max(fam.items(), key=lambda kv: kv[1][1])[0] if fam else None
        if dom in ("flce_fwd", "flce_bwd") and tc_ms:
            # the dominant kernel is the tcgen05 panel GEMM of the CE head: every launch does the
            # same useful work, 2 * rows_tile * vocab_chunk * C (logits, dX and dW panels alike)
            t_flce = (fam.get("flce_fwd", (0, 0))[1] + fam.get("flce_bwd", (0, 0))[1]) / a.steps / 1e3
            n_row_tiles = -(-Nn // 18944)          # the head takes token rows in tiles of 148 x 128
            rows_tile = Nn / n_row_tiles           # mean rows per launch
            vc = min(cfg.ce_vocab_chunk, cfg.vocab)
            fl_launch = 2.0 * rows_tile * vc * cfg.n_embd
            avg_ms = sum(tc_ms) / len(tc_ms)
            ach = fl_launch / (avg_ms / 1e3) / 1e12
            mma_per_kstep = 1 if a.ce_precision == "bf16" else 3
            peak = peaks["bf16_tflops_sustained"]
            nominal = 2250.0 if "bf16" in a.ce_precision else 1125.0
            roofline = {"bound": "tensor", "kernel": "tc_gemm_kernel",
                        "what": "tcgen05 panel GEMM of the fused linear+CE (logits+stats, logits+dlogits, dX, dW)",
                        "achieved": round(ach, 2), "peak": peak, "unit": "TFLOP/s", "frac": round(ach / peak, 4),
                        "traffic": None, "launches_per_step": len(tc_ms) // a.steps,
                        "avg_launch_ms": round(avg_ms, 4), "useful_flops_per_launch": fl_launch,
                        "issued_mma_tflops": round(ach * mma_per_kstep, 2),
                        # the issued MMA rate over the nominal dense rate of the part (2250 TFLOP/s bf16, 1125 TF32
                        # at the maximum SM clock), and over that rate scaled to the SM clock sampled during the
                        # step (the step runs below the maximum clock, at the power cap): a true ceiling, <= 1
                        "issued_frac_of_nominal": round(ach * mma_per_kstep / nominal, 4),
                        "issued_frac_of_nominal_at_sampled_clock": (
                            round(ach * mma_per_kstep / (nominal * clocks["sm_mhz"] / clocks["sm_max_mhz"]), 4)
                            if clocks.get("sm_mhz") and clocks.get("sm_max_mhz") else None),
                        "peak_source": peaks["source"] + " cuBLAS bf16, sustained; TF32 MMAs issue at half that "
                                       "rate and 3xTF32 issues three per k-step",
                        "flce_useful_tflops_whole_op": round(useful / t_flce / 1e12, 2),
                        "flce_executed_tflops_whole_op": round(executed / t_flce / 1e12, 2),
                        "precision": a.ce_precision}
        elif dom is not None and dom in alg:
            per = fam[dom][1] / a.steps / 1e3
            ach = alg[dom] / per / 1e9
            roofline = {"bound": "hbm", "kernel": dom, "achieved": round(ach, 1), "peak": peaks["hbm_gbs"],
                        "unit": "GB/s", "frac": round(ach / peaks["hbm_gbs"], 4), "traffic": None,
                        "peak_source": peaks["source"]}
        else:
            roofline = None
        traffic_path = os.path.join(ROOT, "bench_traffic.json")   # per-launch DRAM bytes read off the ncu summaries in profiles/
        if roofline is not None and os.path.exists(traffic_path):
            with open(traffic_path) as f:
                tr = json.load(f).get(roofline["kernel"])
            if isinstance(tr, dict):   # measured on a smaller capture: bytes per launch and what it scales with
                roofline["traffic"] = tr.get("bytes_per_launch")
                roofline["traffic_note"] = tr.get("note")
                if tr.get("tensor_pipe_note"):
                    roofline["tensor_pipe_note"] = tr.get("tensor_pipe_note")
            else:
                roofline["traffic"] = tr

        cpu = None
        if world == 1 and not a.no_cpu_baseline:
            # the reference's own CPU backend on a bounded sample: one warm-up step, one timed step
            res = cpu_reference_sample(a, a.cpu_sample_tokens or 1024, 1, 1) or cpu_port_sample(a, a.cpu_sample_tokens or 1024)
            n, sec, cpu = res
            cpu["value"] = n / sec
        configs = None
        if config_lines:
            configs = [{"config": ln["config"], "kernel": ln["kernel"], "dtype": ln["dtype"], "ms": ln["ms"],
                        "achieved": ln["roofline"]["achieved"], "unit": ln["roofline"]["unit"], "frac": ln["roofline"]["frac"],
                        **({"unique_rows": ln["unique_rows"]} if "unique_rows" in ln else {})} for ln in config_lines]
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32" if a.ce_precision in ("fp32", "3xtf32") else f"f32 ({a.ce_precision} tensor-core operands in the CE GEMMs)",
            "data": "synthetic",
            "config": bench_config(a, world),
            "setup": {"device_bytes": device_bytes, "allreduce_bytes_per_step": reducer.bytes_per_step if reducer else 0,
                      "allreduces_per_step": 2 if reducer else 0, "grad_wire": a.grad_wire if reducer else None},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 2 * Nn * 4, "d2h_bytes_per_step": 4,
                    "ms_per_step": ms_e2e / a.steps},
            "gpu_launches": int(launches),
            "ms_per_step_with_breakdown_events": ms_breakdown / a.steps,
            "clocks": clocks,
            "roofline": roofline,
            "kernels": kernels,
            "cpu_baseline": cpu,
            "loss": last_loss,
        }
        if comm is not None:
            line["comm"] = comm
        if configs is not None:
            # frac = achieved / peak of MEASURED_PEAKS.json (HBM copy rate; bf16 burst rate for the CE head); gather
            # bytes are the unique-row bound
            line["configs"] = configs
            line["configs_note"] = (f"every kernel of configs 1-4 alone at its stated shape, {CONFIG_IDLE_S:g} s after the timed "
                                    "steps (GPU idle in between), 30 back-to-back launches after 10 warm-up launches, "
                                    "operands rotated through more copies than fit in L2")
        if ms_bf16 is not None:
            line["ce_bf16_mode"] = {"ms_per_step": ms_bf16 / a.steps, "value": tokens / (ms_bf16 / a.steps / 1e3),
                                    "unit": UNIT, "note": "same step with the CE head's GEMM operands rounded to bf16 "
                                                          "(fp32 accumulation, 2e-2 tolerance); not the headline"}
        if ms_x3 is not None:
            line["ce_bf16x3_mode"] = {"ms_per_step": ms_x3 / a.steps, "value": tokens / (ms_x3 / a.steps / 1e3),
                                      "unit": UNIT, "note": "same step with the CE head's GEMM operands as bf16 (hi, lo) "
                                                            "pairs, three MMAs per k-step at the bf16 rate (measured inside the fp32 bounds "
                                                            "of the path: loss 1e-5, dX and dW 1e-4); not the headline"}
        print(json.dumps(line), flush=True)
    ctx.free_host(host)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------
# per-kernel measurements at the shapes of BASELINE configs 1-4
# --------------------------------------------------------------------------------------
def run_kernels(a, env=None, dev_index=0, collect=None, steps=None, warmup=None, cfg2_modes=None, with_cpu=False):
    """Each kernel alone, CUDA events around `steps` launches after `warmup`, operands rotated
    through enough copies that consecutive launches never find their inputs in L2.

    Stand-alone (`--workload kernels`) it creates its own context and prints one JSON line per
    kernel; from the step benchmark it runs on that benchmark's context (`env`) and appends the lines
    to `collect`.  `with_cpu`: each line also carries the reference's CPU time for the same shape
    (`cpu_baseline`; a bounded sample where the full shape would take minutes)."""
    import torch

    import autograd_b200 as ag
    from autograd_b200 import dp

    steps = steps or a.steps
    warmup = warmup or a.warmup
    if env is None:
        torch.cuda.set_device(dev_index)
        stream = torch.cuda.Stream()
        torch.cuda.set_stream(stream)
        ctx, alloc, be = ag.create(dev_index, stream.cuda_stream)
    else:
        ctx, alloc, be = env
    peaks = load_peaks()
    L2 = ctx.l2_bytes
    bufs = []
    cpu_ref = None
    if with_cpu:
        from oracle import ref_loader
        if ref_loader.available():
            from oracle import ref_timing as RT
            cpu_ref = (ref_loader.load(), RT, RT.use_all_cores())

    def cpu_entry(seconds, tokens, sample, kind="reference"):
        """`cpu_baseline` of one kernel line: the same operation on the host."""
        return {"cpu_baseline": {"value": tokens / seconds, "unit": UNIT, "ms": round(1e3 * seconds, 3),
                                 "cores": cpu_ref[2][0], "kind": kind, "sample": sample + "; " + cpu_ref[2][1]}}

    def dev(n_elems, dtype=np.float32, std=1.0, ints=None):
        st = alloc.alloc((int(n_elems),), dtype)
        bufs.append(st)
        addr = st.ptr.address
        if ints is not None:
            ctx.copy_from_host(addr, ints.astype(np.int32))
        elif np.dtype(dtype) == np.dtype(np.float32):
            dp.as_torch(addr, n_elems, dev_index).normal_(0.0, std)
        else:  # bf16 bit patterns of N(0, std), written through an int16 alias of the buffer
            t = torch.empty(int(n_elems), device=f"cuda:{dev_index}", dtype=torch.bfloat16).normal_(0.0, std)
            dst = torch.as_tensor(dp.DeviceArrayView(addr, n_elems, "<i2"), device=f"cuda:{dev_index}")
            dst.copy_(t.view(torch.int16))
        return addr

    def free_all():
        ctx.synchronize()
        for st in bufs:
            alloc.free(st)
        bufs.clear()

    def sets_for(bytes_per_set):
        return max(2, int(2.5 * L2 // max(bytes_per_set, 1)) + 1)

    def time_it(fn, n_sets):
        for i in range(warmup):
            fn(i % n_sets)
        ctx.synchronize()
        E0, E1 = 2, 3
        ctx.event_record(E0)
        for i in range(steps):
            fn(i % n_sets)
        ctx.event_record(E1)
        return ctx.event_elapsed_ms(E0, E1) / steps

    def emit(cfg, kernel, ms, tokens, alg_bytes=None, useful_flops=None, dtype="f32", extra=None):
        line = {"workload": "kernels", "config": cfg, "kernel": kernel, "dtype": dtype, "ms": round(ms, 5),
                "tokens_per_s": tokens / (ms / 1e3), "steps": steps, "warmup": warmup}
        if alg_bytes is not None:
            gbs = alg_bytes / (ms / 1e3) / 1e9
            line["roofline"] = {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                "frac": round(gbs / peaks["hbm_gbs"], 4), "algorithmic_bytes": int(alg_bytes),
                                "frac_of_nominal_8TBs": round(gbs / 8000.0, 4), "peak_source": peaks["source"]}
        if useful_flops is not None:
            tf = useful_flops / (ms / 1e3) / 1e12
            line["roofline"] = {"bound": "tensor", "achieved": round(tf, 2), "peak": peaks["bf16_tflops"],
                                "unit": "TFLOP/s", "frac": round(tf / peaks["bf16_tflops"], 4),
                                "useful_flops": useful_flops, "peak_source": peaks["source"] + " bf16 burst"}
        if extra:
            line.update(extra)
        if collect is not None:
            collect.append(line)
        else:
            print(json.dumps(line), flush=True)

    f4 = 4
    def sec_cfg1():
        # ---- config 1: fused add + LayerNorm, 16384 x 384 (and the config-5 width 32768 x 1280)
        for (N, C) in ((16384, 384), (32768, 1280)):
            nb = N * C * f4
            n_sets = sets_for(4 * nb)
            x = [dev(N * C) for _ in range(n_sets)]; r = [dev(N * C) for _ in range(n_sets)]
            h = [dev(N * C) for _ in range(n_sets)]; y = [dev(N * C) for _ in range(n_sets)]
            gam, bet, dg, db = dev(C), dev(C), dev(C), dev(C)
            pb = ctx.norm_partials_bytes(C); part = alloc.alloc((pb,), np.uint8); bufs.append(part)
            cf = cb = None
            if cpu_ref is not None:       # the reference's Add + LayerNorm graph at the same shape
                tf, tb = cpu_ref[1].OpGraph(cpu_ref[0], cpu_ref[1].add_layernorm(N // 512, 512, C)).time_pair(1, 2)
                what = f"AddOp + LayerNormOp graph, {N} x {C}, Runtime(device='cpu')"
                cf, cb = cpu_entry(tf, N, what + " forward()"), cpu_entry(tb, N, what + " backward_graph()")
            ms = time_it(lambda i: ctx.add_layernorm_forward(x[i], r[i], gam, bet, h[i], y[i], 0, 0, N, C, 1e-5), n_sets)
            emit("cfg1" if C == 384 else "cfg5-width", f"add_layernorm_forward {N}x{C}", ms, N, alg_bytes=4 * nb, extra=cf)
            # backward: dy = y[i], saved input = h[i], residual gradient accumulated in place in x[i]
            ms = time_it(lambda i: ctx.layernorm_backward(y[i], h[i], gam, x[i], x[i], dg, db, part.ptr.address, pb, N, C,
                                                          1e-5), n_sets)
            emit("cfg1" if C == 384 else "cfg5-width", f"layernorm_backward(+residual grad) {N}x{C}", ms, N, alg_bytes=4 * nb,
                 extra=cb)
            free_all()

    def sec_gelu():
        # ---- GELU 16384 x 1536
        n = 16384 * 1536
        n_sets = sets_for(3 * n * f4)
        x = [dev(n) for _ in range(n_sets)]; y = [dev(n) for _ in range(n_sets)]; g = [dev(n) for _ in range(n_sets)]
        cf = cb = None
        if cpu_ref is not None:
            tf, tb = cpu_ref[1].OpGraph(cpu_ref[0], cpu_ref[1].gelu(16384, 1536)).time_pair(1, 2)
            cf = cpu_entry(tf, 16384, "GELUOp graph, 16384 x 1536, Runtime(device='cpu') forward()")
            cb = cpu_entry(tb, 16384, "GELUOp graph, 16384 x 1536, Runtime(device='cpu') backward_graph()")
        ms = time_it(lambda i: ctx.gelu_forward(x[i], y[i], n), n_sets)
        emit("gelu", "gelu_forward 16384x1536", ms, 16384, alg_bytes=2 * n * f4, extra=cf)
        ms = time_it(lambda i: ctx.gelu_backward(x[i], y[i], 0, g[i], n), n_sets)
        emit("gelu", "gelu_backward 16384x1536", ms, 16384, alg_bytes=3 * n * f4, extra=cb)
        free_all()

    def sec_cfg3():
        # ---- config 3: RMSNorm, RoPE, SwiGLU at the Qwen shapes, fp32 and bf16 storage
        N, C, H, HKV, D, I, B, T = 8192, 1536, 12, 2, 128, 8960, 4, 2048
        # RoPE tables, positions 0..T-1 (module.py:247-250)
        freqs = np.arange(T, dtype=np.float32)[:, None] * (np.float32(1e6) ** (-np.arange(0, D, 2, dtype=np.float32)[None, :]
                                                                              / np.float32(D)))
        cos_, sin_ = np.cos(freqs).astype(np.float32), np.sin(freqs).astype(np.float32)
        cpu = {}
        if cpu_ref is not None:
            # The reference has no standalone op for these stages.  Two CPU figures per stage: the carrier op
            # end to end (FusedRMSNormMLPOp: RMSNorm + two GEMMs + SwiGLU, mostly GEMM time), and the stage alone
            # = the numpy statements of that stage (backend.py:1097-1108, :1113-1126, :1202-1251, restated in
            # oracle/fused_layers.py; RoPE: the reference's own apply_rope_np / apply_rope_backward_np).
            ref, RT, _ = cpu_ref
            from oracle import fused_layers as O
            rng = np.random.default_rng(1236)
            cx = rng.standard_normal((N, C), dtype=np.float32); cg = np.ones(C, np.float32)
            t0 = time.perf_counter(); O.rmsnorm_forward(cx, cg, 1e-6); t1 = time.perf_counter()
            O.rmsnorm_backward(cx, cg, cx, 1e-6, cx, cg); t2 = time.perf_counter()
            cgu = rng.standard_normal((N, 2 * I), dtype=np.float32); chd = rng.standard_normal((N, I), dtype=np.float32)
            t3 = time.perf_counter(); O.swiglu_forward(cgu); t4 = time.perf_counter()
            O.swiglu_backward(cgu, chd); t5 = time.perf_counter()
            rp = RT.RopeBuffers(ref, B, T, H, HKV, D, 1e6)
            rf, rb = rp.time_pair(1)
            ctf, ctb = RT.OpGraph(ref, RT.rmsnorm_mlp(B, T, C, I)).time_pair(0, 1)
            carrier = {"cpu_carrier_op": {"op": "FusedRMSNormMLPOp 4x2048x1536, I 8960, Runtime(device='cpu')",
                                          "forward_ms": round(1e3 * ctf, 1), "backward_ms": round(1e3 * ctb, 1)}}
            stage = "stage alone, numpy statements of the reference's CPU kernel"
            cpu = {"rms_f": {**cpu_entry(t1 - t0, N, stage, "port"), **carrier},
                   "rms_b": {**cpu_entry(t2 - t1, N, stage, "port"), **carrier},
                   "rope": cpu_entry(rf, N, "apply_rope_np on q (12 heads) and k (2 heads), 4 x 2048 x 128"),
                   "swi_f": {**cpu_entry(t4 - t3, N, stage, "port"), **carrier},
                   "swi_b": {**cpu_entry(t5 - t4, N, stage, "port"), **carrier}}
            del cx, cgu, chd, rp
        for dt_name, dt, es in (("f32", np.float32, 4), ("bf16", np.uint16, 2)):
            agdt = ag.AG_F32 if es == 4 else ag.AG_BF16
            n_sets = sets_for(3 * N * C * es)
            x = [dev(N * C, dt) for _ in range(n_sets)]; y = [dev(N * C, dt) for _ in range(n_sets)]
            d = [dev(N * C, dt) for _ in range(n_sets)]
            gam, dg = dev(C), dev(C)
            pb = ctx.norm_partials_bytes(C); part = alloc.alloc((pb,), np.uint8); bufs.append(part)
            ms = time_it(lambda i: ctx.rmsnorm_forward(x[i], gam, y[i], 0, N, C, 1e-6, agdt), n_sets)
            emit("cfg3", "rmsnorm_forward 8192x1536", ms, N, alg_bytes=2 * N * C * es, dtype=dt_name, extra=cpu.get("rms_f"))
            ms = time_it(lambda i: ctx.rmsnorm_backward(y[i], x[i], gam, d[i], d[i], dg, part.ptr.address, pb, N, C, 1e-6,
                                                        agdt), n_sets)
            emit("cfg3", "rmsnorm_backward(+residual grad) 8192x1536", ms, N, alg_bytes=4 * N * C * es, dtype=dt_name,
                 extra=cpu.get("rms_b"))
            free_all()
            nq, nk = N * H * D, N * HKV * D
            n_sets = sets_for((nq + nk) * es)
            q = [dev(nq, dt) for _ in range(n_sets)]; k = [dev(nk, dt) for _ in range(n_sets)]
            cos = dev(cos_.size); sin = dev(sin_.size)
            ctx.copy_from_host(cos, cos_); ctx.copy_from_host(sin, sin_)
            ms = time_it(lambda i: ctx.rope_qk(q[i], k[i], cos, sin, B, T, H, HKV, D, sin_sign=1, dtype=agdt), n_sets)
            emit("cfg3", "rope_qk 4x2048 q12 k2 d128", ms, N, alg_bytes=2 * (nq + nk) * es, dtype=dt_name, extra=cpu.get("rope"))
            free_all()
            n_sets = sets_for(4 * N * I * es)
            gu = [dev(N * 2 * I, dt) for _ in range(n_sets)]; hid = [dev(N * I, dt) for _ in range(n_sets)]
            ms = time_it(lambda i: ctx.swiglu_forward(gu[i], hid[i], N, I, agdt), n_sets)
            emit("cfg3", "swiglu_forward 8192x8960", ms, N, alg_bytes=3 * N * I * es, dtype=dt_name, extra=cpu.get("swi_f"))
            ms = time_it(lambda i: ctx.swiglu_backward(gu[i], hid[i], N, I, agdt), n_sets)
            emit("cfg3", "swiglu_backward_inplace 8192x8960", ms, N, alg_bytes=5 * N * I * es, dtype=dt_name,
                 extra=cpu.get("swi_b"))
            free_all()

    def sec_cfg4():
        # ---- config 4: gather / deterministic scatter-add, Zipf(1.1) ids
        V, C, n = 151936, 1536, 65536
        rng = np.random.default_rng(1237)
        p = 1.0 / np.arange(1, V + 1) ** 1.1
        p /= p.sum()
        ids_ = rng.choice(V, size=n, p=p).astype(np.int32)
        uniq = int(np.unique(ids_).size)
        ids = dev(n, np.int32, ints=ids_)
        table = dev(V * C, std=0.02); dtable = dev(V * C)
        n_sets = 2
        out = [dev(n * C) for _ in range(n_sets)]
        sb = ctx.scatter_add_scratch_bytes(n, C, V); sc = alloc.alloc((sb,), np.uint8); bufs.append(sc)
        cf, cb = {}, {}
        if cpu_ref is not None:
            tf, tb = cpu_ref[1].OpGraph(cpu_ref[0], cpu_ref[1].gather(32, 2048, V, C, ids=ids_)).time_pair(0, 1)
            what = "GatherOp graph, 65536 Zipf ids, table 151936 x 1536, Runtime(device='cpu')"
            cf = cpu_entry(tf, n, what + " forward()")
            cb = cpu_entry(tb, n, what + " backward_graph() (np.add.at, plus the zero-fill of the output gradient)")
        ms = time_it(lambda i: ctx.gather_forward(ids, table, out[i], n, C, V), n_sets)
        # DRAM sees every distinct table row once (the hot Zipf rows stay in L2) plus the output: the
        # roofline numerator is that bound, not 2 x n x C
        emit("cfg4", "gather_forward 65536 ids x 1536", ms, n, alg_bytes=(n + uniq) * C * f4,
             extra={"unique_rows": uniq, "bytes_if_every_row_were_distinct": 2 * n * C * f4, **cf})
        ctx.fill_f32(dtable, 0.0, V * C)
        ms = time_it(lambda i: ctx.gather_backward(ids, out[i], dtable, sc.ptr.address, sb, n, C, V), n_sets)
        emit("cfg4", "scatter_add (sort + segmented sum) 65536 ids x 1536", ms, n, alg_bytes=(n + 2 * uniq) * C * f4,
             extra={"unique_rows": uniq, "note": "without the dense zero-fill of dTable", **cb})
        ms0 = time_it(lambda i: ctx.fill_f32(dtable, 0.0, V * C), 1)
        emit("cfg4", "zero-fill of dTable 151936x1536", ms0, n, alg_bytes=V * C * f4)
        free_all()

    def sec_cfg2():
        # ---- config 2: fused linear + CE, N 16384, V 32768, C 384 and 1280
        N, V = 16384, 32768
        rng = np.random.default_rng(1238)
        tg_ = rng.integers(0, V, size=N).astype(np.int32)
        tg_[rng.random(N) < 0.05] = -1
        modes = {"3xtf32": ag.AG_CE_3XTF32, "bf16": ag.AG_CE_BF16, "bf16x3": ag.AG_CE_BF16X3}
        for C in (384, 1280):
            cf = cb = None
            if cpu_ref is not None:     # a 2048-row sample of the 16384 rows: the cost is linear in the rows
                tf, tb = cpu_ref[1].OpGraph(cpu_ref[0], cpu_ref[1].fused_linear_ce(1, 2048, C, V)).time_pair(0, 1)
                what = f"FusedLinearCrossEntropyOp graph, 2048 of 16384 rows, C {C}, V 32768, Runtime(device='cpu')"
                cf, cb = cpu_entry(tf, 2048, what + " forward()"), cpu_entry(tb, 2048, what + " backward_graph()")
            for pname in (cfg2_modes or modes):
                prec = modes[pname]
                X = dev(N * C, std=1.0 / np.sqrt(C)); W = dev(V * C, std=0.02)
                dX, dW = dev(N * C), dev(V * C)
                tg = dev(N, np.int32, ints=tg_)
                loss, dloss, lse = dev(1), dev(1), dev(N)
                ctx.fill_f32(dloss, 1.0, 1)
                desc = ctx.flce_desc(N, C, V, vocab_chunk=4096, precision=prec)
                sbytes = ctx.flce_scratch_bytes(desc); scr = alloc.alloc((sbytes,), np.uint8); bufs.append(scr)
                ms_f = time_it(lambda i: ctx.flce_forward(desc, X, W, tg, 0, loss, lse, scr.ptr.address, sbytes), 1)
                ms_b = time_it(lambda i: ctx.flce_backward(desc, X, W, tg, 0, dloss, lse, dX, dW, scr.ptr.address, sbytes), 1)
                fl = 2.0 * N * C * V
                emit("cfg2", f"fused_linear_ce forward N16384 C{C} V32768", ms_f, N, useful_flops=fl, dtype=pname, extra=cf)
                emit("cfg2", f"fused_linear_ce backward N16384 C{C} V32768", ms_b, N, useful_flops=2 * fl, dtype=pname,
                     extra={"executed_flops": 3 * fl, **(cb or {})})
                emit("cfg2", f"fused_linear_ce fwd+bwd N16384 C{C} V32768", ms_f + ms_b, N, useful_flops=3 * fl, dtype=pname,
                     extra={"scratch_bytes": sbytes})
                free_all()

    def sec_next():
        # ---- the rows after the core path: linear + bias + residual projection, AdamW
        N = 16384
        for (K, C, what) in ((1280, 1280, "attention out-projection"), (5120, 1280, "MLP down-projection")):
            for pname, prec in (("3xtf32", ag.AG_CE_3XTF32), ("bf16", ag.AG_CE_BF16)):
                x, act, w, b, out = dev(N * C), dev(N * K, std=1.0), dev(K * C, std=0.02), dev(C), dev(N * C)
                dout, dx, dact, dw, db = dev(N * C), dev(N * C), dev(N * K), dev(K * C), dev(C)
                sbytes = ctx.linear_add_scratch_bytes(N, K, C, prec)
                scr = alloc.alloc((sbytes,), np.uint8); bufs.append(scr)
                ms_f = time_it(lambda i: ctx.linear_add_forward(x, act, w, b, out, N, K, C, prec, scr.ptr.address, sbytes), 1)
                ms_b = time_it(lambda i: ctx.linear_add_backward(dout, act, w, dx, dact, dw, db, N, K, C, prec,
                                                                 scr.ptr.address, sbytes), 1)
                fl = 2.0 * N * K * C
                emit("next", f"linear_add forward N16384 K{K} C{C} ({what})", ms_f, N, useful_flops=fl, dtype=pname)
                emit("next", f"linear_add backward N16384 K{K} C{C}", ms_b, N, useful_flops=2 * fl, dtype=pname)
                free_all()
        n = 32768 * 1280
        n_sets = sets_for(4 * n * f4)
        ps = [dev(n, std=0.02) for _ in range(n_sets)]; gs = [dev(n, std=0.01) for _ in range(n_sets)]
        ms_ = [dev(n, std=0.0) for _ in range(n_sets)]; vs = [dev(n, std=0.0) for _ in range(n_sets)]
        ms = time_it(lambda i: ctx.adamw_step(ps[i], gs[i], ms_[i], vs[i], n, 1e-3, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1.0), n_sets)
        emit("next", "adamw_step 32768x1280 parameters (read p,g,m,v; write p,m,v)", ms, n, alg_bytes=7 * n * f4)
        free_all()
        # ---- parameter gradients stored as bf16: conversion (with accumulate), AdamW on bf16 gradients,
        # scatter-add into a bf16 table gradient
        n_sets = sets_for(3 * n * f4)
        src = [dev(n, std=0.01) for _ in range(n_sets)]; bits = [dev(n, np.uint16, std=0.01) for _ in range(n_sets)]
        ms = time_it(lambda i: ctx.f32_to_bf16(src[i], bits[i], n, accumulate=False), n_sets)
        emit("next", "f32_to_bf16 32768x1280 (read fp32, write bf16)", ms, n, alg_bytes=6 * n)
        ms = time_it(lambda i: ctx.f32_to_bf16(src[i], bits[i], n, accumulate=True), n_sets)
        emit("next", "f32_to_bf16 accumulate 32768x1280 (read fp32 + bf16, write bf16)", ms, n, alg_bytes=8 * n)
        ms = time_it(lambda i: ctx.bf16_to_f32(bits[i], src[i], n), n_sets)
        emit("next", "bf16_to_f32 32768x1280", ms, n, alg_bytes=6 * n)
        free_all()
        n_sets = sets_for(4 * n * f4)
        ps = [dev(n, std=0.02) for _ in range(n_sets)]; gb = [dev(n, np.uint16, std=0.01) for _ in range(n_sets)]
        ms_ = [dev(n, std=0.0) for _ in range(n_sets)]; vs = [dev(n, std=0.0) for _ in range(n_sets)]
        ms = time_it(lambda i: ctx.adamw_step(ps[i], gb[i], ms_[i], vs[i], n, 1e-3, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1.0,
                                              grad_bf16=True), n_sets)
        emit("next", "adamw_step, bf16 gradients, 32768x1280 parameters", ms, n, alg_bytes=26 * n)
        free_all()
        V, C, nid = 151936, 1536, 65536
        rng = np.random.default_rng(1237)
        p = 1.0 / np.arange(1, V + 1) ** 1.1
        p /= p.sum()
        ids_ = rng.choice(V, size=nid, p=p).astype(np.int32)
        uniq = int(np.unique(ids_).size)
        ids = dev(nid, np.int32, ints=ids_)
        dtb = dev(V * C, np.uint16, std=0.0)
        out = [dev(nid * C) for _ in range(2)]
        sb = ctx.scatter_add_scratch_bytes(nid, C, V); sc = alloc.alloc((sb,), np.uint8); bufs.append(sc)
        ms = time_it(lambda i: ctx.gather_backward_bf16(ids, out[i], dtb, sc.ptr.address, sb, nid, C, V), 2)
        emit("next", "scatter_add into a bf16 table gradient, 65536 Zipf ids x 1536", ms, nid,
             alg_bytes=nid * C * f4 + 2 * uniq * C * 2, extra={"unique_rows": uniq})
        free_all()

    def sec_rmsce():
        # ---- FusedRMSNormLinearCrossEntropy with row_scale at the Qwen head shape (hidden 1536, vocabulary
        # 151936, 8192 token rows): the launch sequence of the backend's callables - RMSNorm, the CE head on its
        # output with per-row weights; backward: RMSNorm again, dz zero-fill, CE backward into dz and dW,
        # RMSNorm backward with the residual-gradient add and dgamma
        N, C, V = 8192, 1536, 151936
        rng = np.random.default_rng(1241)
        tg_ = rng.integers(0, V, size=N).astype(np.int32)
        tg_[rng.random(N) < 0.05] = -1
        tg_[rng.random(N) < 0.01] = V          # out of range: ignored like -1
        X = dev(N * C, std=1.0); W = dev(V * C, std=0.02); gam = dev(C, std=0.02)
        ctx.fill_f32(gam, 1.0, C)
        rs = dev(N, std=0.0); ctx.fill_f32(rs, 1.0 / N, N)
        dX, dW, dgam = dev(N * C), dev(V * C), dev(C)
        z, dz = dev(N * C), dev(N * C)
        tg = dev(N, np.int32, ints=tg_)
        loss, dloss, lse = dev(1), dev(1), dev(N)
        ctx.fill_f32(dloss, 1.0, 1)
        pb = ctx.norm_partials_bytes(C); part = alloc.alloc((pb,), np.uint8); bufs.append(part)
        cf = cb = None
        if cpu_ref is not None:     # a 512-row sample of the 8192 rows: the cost is linear in the rows
            tf, tb = cpu_ref[1].OpGraph(cpu_ref[0], cpu_ref[1].rmsnorm_fused_linear_ce(1, 512, C, V)).time_pair(0, 1)
            what = f"FusedRMSNormLinearCrossEntropyOp graph with row_scale, 512 of {N} rows, C {C}, V {V}, Runtime(device='cpu')"
            cf, cb = cpu_entry(tf, 512, what + " forward()"), cpu_entry(tb, 512, what + " backward_graph()")
        for pname, prec in (("3xtf32", ag.AG_CE_3XTF32), ("bf16x3", ag.AG_CE_BF16X3)):
            desc = ctx.flce_desc(N, C, V, vocab_chunk=4096, precision=prec)
            sbytes = ctx.flce_scratch_bytes(desc); scr = alloc.alloc((sbytes,), np.uint8); bufs.append(scr)

            def fwd(i):
                ctx.rmsnorm_forward(X, gam, z, 0, N, C, 1e-6)
                ctx.flce_forward(desc, z, W, tg, rs, loss, lse, scr.ptr.address, sbytes)

            def bwd(i):
                ctx.rmsnorm_forward(X, gam, z, 0, N, C, 1e-6)
                ctx.fill_f32(dz, 0.0, N * C)
                ctx.flce_backward(desc, z, W, tg, rs, dloss, lse, dz, dW, scr.ptr.address, sbytes)
                ctx.rmsnorm_backward(dz, X, gam, dX, dX, dgam, part.ptr.address, pb, N, C, 1e-6)

            ms_f = time_it(fwd, 1)
            ms_b = time_it(bwd, 1)
            fl = 2.0 * N * C * V
            emit("rmsce", f"rmsnorm + fused_linear_ce(row_scale) forward N{N} C{C} V{V}", ms_f, N, useful_flops=fl, dtype=pname,
                 extra=cf)
            emit("rmsce", f"rmsnorm + fused_linear_ce(row_scale) backward N{N} C{C} V{V}", ms_b, N, useful_flops=2 * fl,
                 dtype=pname, extra={"executed_flops": 3 * fl, "scratch_bytes": sbytes, **(cb or {})})
        free_all()

    sections = {"cfg1": sec_cfg1, "gelu": sec_gelu, "cfg3": sec_cfg3, "cfg4": sec_cfg4, "cfg2": sec_cfg2,
                "next": sec_next, "rmsce": sec_rmsce}
    wanted = [s for s in (a.only.split(",") if a.only else sections) if s]
    for name in wanted:
        if name not in sections:
            raise SystemExit(f"--only: unknown section {name!r}; choose from {sorted(sections)}")
        sections[name]()
    ctx.check_status()
    return collect


def main():
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    elif a.workload == "kernels":
        run_kernels(a, with_cpu=not a.no_cpu_baseline)
    else:
        run_b200(a)


if __name__ == "__main__":
    main()
