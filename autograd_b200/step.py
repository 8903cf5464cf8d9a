"""The fused-layer step of a GPT-shaped model: every fused layer kernel of one training step,
in model order, forward then backward, inside buffers allocated once.

Per layer the model is   h1 = x + r ; y1 = LN1(h1) ; [qkv GEMM] ; RoPE(q,k) ; [attention,
out-proj] ; h2 = h1 + a ; y2 = LN2(h2) ; [fc GEMM] ; g = GELU(u) ; [proj GEMM]   and the head is
LN_f + fused linear+CE on the tied embedding.  The bracketed GEMM / attention nodes are not part
of this backend: their outputs (r, a, q, k, u) and, in backward, their input gradients are
stand-in buffers of the right shape holding seeded N(0,1) data.  What a real backward needs from
forward is kept per layer exactly as a real model would keep it (h1, h2 for the LayerNorm
backward; u for the GELU backward); everything else rotates through a few transient buffers.
All transient buffers are larger than the L2 cache, so every pass streams from HBM.

The step covers: 1 gather, 2L+1 fused (add+)LayerNorm forward and backward, L RoPE(q,k)
forward and backward, L GELU forward and backward, 1 fused linear+CE forward and backward, 1
deterministic scatter-add into the tied table, plus the zero-fills of the gradient buffers.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import _native as N


@dataclass
class StepConfig:
    n_layer: int = 20
    n_embd: int = 1280
    n_head: int = 10
    head_dim: int = 128
    seq_len: int = 2048
    vocab: int = 32768
    batch: int = 16            # sequences per GPU
    mlp_ratio: int = 4
    eps: float = 1e-5
    rope_theta: float = 1e5    # module.py:146 (GPT2 uses 100000.0)
    ce_precision: int = N.AG_CE_3XTF32
    ce_vocab_chunk: int = 4096

    @property
    def tokens(self):
        return self.batch * self.seq_len


class FamilyTimer:
    """Collects (start, end) event index pairs per kernel family for one or more steps."""

    def __init__(self, ctx, base=0):
        self.ctx = ctx
        self.pairs = {}
        self.base = base          # first event index this timer may use
        self.next = base
        self.enabled = False

    def reset(self):
        self.pairs = {}
        self.next = self.base

    def begin(self, family):
        if not self.enabled:
            return None
        i = self.next
        self.next += 2
        self.ctx.event_record(i)
        self.pairs.setdefault(family, []).append(i)
        return i

    def end(self, token):
        if token is not None:
            self.ctx.event_record(token + 1)

    def totals_ms(self):
        out = {}
        for fam, starts in self.pairs.items():
            ms = [self.ctx.event_elapsed_ms(i, i + 1) for i in starts]
            out[fam] = (len(ms), float(sum(ms)))
        return out


class FusedLayerStep:
    def __init__(self, ctx, allocator, backend, cfg: StepConfig, seed: int = 1238, fill_normal=None):
        """`fill_normal(address, n_floats, seed)` fills a device buffer with N(0,1) values; when
        None, buffers are filled from host-generated numpy data (slow for the full size)."""
        self.ctx, self.alloc, self.be, self.cfg = ctx, allocator, backend, cfg
        c = cfg
        self.N, self.C, self.V, self.L = c.tokens, c.n_embd, c.vocab, c.n_layer
        self.I = c.mlp_ratio * c.n_embd
        self.timer = FamilyTimer(ctx)
        self._seed = seed
        self._fill_normal = fill_normal
        self._bufs = []
        Nn, C, V, L, I = self.N, self.C, self.V, self.L, self.I
        f32 = np.float32
        # inputs
        self.ids = self._dev((Nn,), np.int32)
        self.targets = self._dev((Nn,), np.int32)
        # parameters: tied embedding / lm head, LayerNorm affine pairs
        self.table = self._dev((V, C), f32, normal=0.02)
        self.n_norms = 2 * L + 1
        gam = (1 + 0.02 * np.random.default_rng(seed + 1).standard_normal((self.n_norms, C))).astype(f32)
        bet = (0.02 * np.random.default_rng(seed + 2).standard_normal((self.n_norms, C))).astype(f32)
        self.gamma = self._dev((self.n_norms, C), f32, host=gam)
        self.beta = self._dev((self.n_norms, C), f32, host=bet)
        # gradient buckets (contiguous, so that one allreduce covers each)
        # [dgamma | dbeta] per norm, then the loss scalar: one small allreduce carries all of them
        self.n_small = self.n_norms * 2 * C
        self.small_bucket = self._dev((self.n_small + 4,), f32)
        self.loss = self.small_bucket + self.n_small * 4
        self.dtable = self._dev((V, C), f32)                           # dW_vocab == embedding grad (tied)
        self.dloss = self._dev((1,), f32)
        # RoPE tables (module.py:146-156)
        pos = np.arange(c.seq_len, dtype=f32)[:, None]
        ch = np.arange(0, c.head_dim, 2, dtype=f32)[None, :]
        freqs = pos * (f32(c.rope_theta) ** (-ch / f32(c.head_dim)))
        self.cos = self._dev(freqs.shape, f32, host=np.cos(freqs).astype(f32))
        self.sin = self._dev(freqs.shape, f32, host=np.sin(freqs).astype(f32))
        # saved activations, per layer
        self.h1 = [self._dev((Nn, C), f32) for _ in range(L)]
        self.h2 = [self._dev((Nn, C), f32) for _ in range(L)]
        self.u = [self._dev((Nn, I), f32, normal=1.0) for _ in range(L)]
        self.h_final = self._dev((Nn, C), f32)
        # transient buffers
        self.x0 = self._dev((Nn, C), f32)                              # gather output
        self.branch = [self._dev((Nn, C), f32, normal=1.0) for _ in range(4)]   # r / a stand-ins
        self.y = [self._dev((Nn, C), f32) for _ in range(2)]           # LayerNorm outputs
        self.q = self._dev((Nn, c.n_head * c.head_dim), f32, normal=1.0)
        self.k = self._dev((Nn, c.n_head * c.head_dim), f32, normal=1.0)
        self.g = self._dev((Nn, I), f32)                               # GELU output
        self.dy = [self._dev((Nn, C), f32, normal=1.0) for _ in range(2)]       # upstream grads of the norms
        self.dg = self._dev((Nn, I), f32, normal=1.0)                  # upstream grad of GELU
        self.du = self._dev((Nn, I), f32)                              # GELU input grad
        self.dh = self._dev((Nn, C), f32)                              # residual-stream gradient
        self.lse = self._dev((Nn,), f32)
        self.partials_bytes = ctx.norm_partials_bytes(C)
        self.partials = self._raw(self.partials_bytes)
        self.scatter_bytes = ctx.scatter_add_scratch_bytes(Nn, C, V)
        self.scatter = self._raw(self.scatter_bytes)
        self.desc = ctx.flce_desc(Nn, C, V, vocab_chunk=c.ce_vocab_chunk, precision=c.ce_precision)
        self.flce_bytes = ctx.flce_scratch_bytes(self.desc)
        self.flce_scratch = self._raw(self.flce_bytes)
        ctx.fill_f32(self.dloss, 1.0, 1)
        ctx.synchronize()

    # ------------------------------------------------------------------ buffers
    def _raw(self, nbytes):
        st = self.alloc.alloc((max(int(nbytes), 256),), np.uint8)
        self._bufs.append(st)
        return st.ptr.address

    def _dev(self, shape, dtype, normal=None, host=None):
        n = int(np.prod(shape))
        addr = self._raw(n * np.dtype(dtype).itemsize)
        if host is not None:
            self.ctx.copy_from_host(addr, np.ascontiguousarray(host, dtype=dtype))
        elif normal is not None:
            self._seed += 1
            if self._fill_normal is not None:
                self._fill_normal(addr, n, self._seed, float(normal))
            else:
                rng = np.random.default_rng(self._seed)
                self.ctx.copy_from_host(addr, (normal * rng.standard_normal(n, dtype=np.float32)).astype(np.float32))
        else:
            self.ctx.fill_pattern(addr, 0, 1, n * np.dtype(dtype).itemsize)
        return addr

    def close(self):
        self.ctx.synchronize()
        for st in self._bufs:
            self.alloc.free(st)
        self._bufs = []

    @property
    def device_bytes(self):
        return sum(st.nbytes for st in self._bufs)

    # ------------------------------------------------------------------ the step
    def load_batch(self, ids_host_addr, targets_host_addr):
        """Host -> device copy of this step's token ids and targets (int32, N each)."""
        self.ctx.copy_h2d_raw(self.ids, ids_host_addr, self.N * 4)
        self.ctx.copy_h2d_raw(self.targets, targets_host_addr, self.N * 4)

    def _norm_params(self, i):
        C = self.C
        return (self.gamma + i * C * 4, self.beta + i * C * 4,
                self.small_bucket + (2 * i) * C * 4, self.small_bucket + (2 * i + 1) * C * 4)

    def forward(self):
        ctx, t, c = self.ctx, self.timer, self.cfg
        Nn, C, V, L, I = self.N, self.C, self.V, self.L, self.I
        k = t.begin("gather_fwd"); ctx.gather_forward(self.ids, self.table, self.x0, Nn, C, V); t.end(k)
        x = self.x0
        for l in range(L):
            g1, b1, _, _ = self._norm_params(2 * l)
            k = t.begin("ln_fwd")
            ctx.add_layernorm_forward(x, self.branch[(2 * l) % 4], g1, b1, self.h1[l], self.y[0], 0, 0, Nn, C, c.eps)
            t.end(k)
            k = t.begin("rope")
            ctx.rope_qk(self.q, self.k, self.cos, self.sin, c.batch, c.seq_len, c.n_head, c.n_head, c.head_dim,
                        sin_sign=-1)
            t.end(k)
            g2, b2, _, _ = self._norm_params(2 * l + 1)
            k = t.begin("ln_fwd")
            ctx.add_layernorm_forward(self.h1[l], self.branch[(2 * l + 1) % 4], g2, b2, self.h2[l], self.y[1], 0, 0,
                                      Nn, C, c.eps)
            t.end(k)
            k = t.begin("gelu_fwd"); ctx.gelu_forward(self.u[l], self.g, Nn * I); t.end(k)
            x = self.h2[l]
        gf, bf, _, _ = self._norm_params(2 * L)
        k = t.begin("ln_fwd")
        ctx.add_layernorm_forward(x, self.branch[0], gf, bf, self.h_final, self.y[0], 0, 0, Nn, C, c.eps)
        t.end(k)
        k = t.begin("flce_fwd")
        ctx.flce_forward(self.desc, self.y[0], self.table, self.targets, 0, self.loss, self.lse, self.flce_scratch,
                         self.flce_bytes)
        t.end(k)

    def backward(self):
        ctx, t, c = self.ctx, self.timer, self.cfg
        Nn, C, V, L, I = self.N, self.C, self.V, self.L, self.I
        k = t.begin("zero_grads")
        ctx.fill_f32(self.small_bucket, 0.0, self.n_small)       # not the loss word behind the gradients
        ctx.fill_f32(self.dtable, 0.0, V * C)
        ctx.fill_f32(self.dy[0], 0.0, Nn * C)      # gradient of the final norm's output: written by the head
        t.end(k)
        k = t.begin("flce_bwd")
        ctx.flce_backward(self.desc, self.y[0], self.table, self.targets, 0, self.dloss, self.lse, self.dy[0],
                          self.dtable, self.flce_scratch, self.flce_bytes)
        t.end(k)
        gf, _, dgf, dbf = self._norm_params(2 * L)
        k = t.begin("ln_bwd")   # first writer of the residual gradient: dres = NULL
        ctx.layernorm_backward(self.dy[0], self.h_final, gf, 0, self.dh, dgf, dbf, self.partials,
                               self.partials_bytes, Nn, C, c.eps)
        t.end(k)
        for l in reversed(range(L)):
            k = t.begin("gelu_bwd"); ctx.gelu_backward(self.u[l], self.dg, 0, self.du, Nn * I); t.end(k)
            g2, _, dg2, db2 = self._norm_params(2 * l + 1)
            k = t.begin("ln_bwd")   # fused residual-gradient add: dh += local
            ctx.layernorm_backward(self.dy[1], self.h2[l], g2, self.dh, self.dh, dg2, db2, self.partials,
                                   self.partials_bytes, Nn, C, c.eps)
            t.end(k)
            k = t.begin("rope")     # backward of RoPE = the transposed rotation on dq, dk
            ctx.rope_qk(self.q, self.k, self.cos, self.sin, c.batch, c.seq_len, c.n_head, c.n_head, c.head_dim,
                        sin_sign=+1)
            t.end(k)
            g1, _, dg1, db1 = self._norm_params(2 * l)
            k = t.begin("ln_bwd")
            ctx.layernorm_backward(self.dy[l % 2], self.h1[l], g1, self.dh, self.dh, dg1, db1, self.partials,
                                   self.partials_bytes, Nn, C, c.eps)
            t.end(k)
        k = t.begin("scatter_add")
        ctx.gather_backward(self.ids, self.dh, self.dtable, self.scatter, self.scatter_bytes, Nn, C, V)
        t.end(k)

    def step(self):
        self.forward()
        self.backward()

    def read_loss(self, world: int = 1) -> float:
        """Device -> host read of the loss; after a data-parallel reduce the word holds the sum of the
        ranks' mean losses, `world` turns it into the global mean."""
        return float(self.ctx.copy_to_host(self.loss, (1,), np.float32)[0]) / world

    def grad_buckets(self):
        """(address, n_floats) of the two contiguous buckets a data-parallel allreduce covers: all
        dgamma/dbeta followed by the loss scalar (the sum of the ranks' mean losses; divide by the
        world size), and the tied dW_vocab / embedding gradient."""
        return [(self.small_bucket, self.n_small + 1), (self.dtable, self.V * self.C)]

    # ------------------------------------------------------------------ accounting
    def algorithmic_bytes(self):
        """HBM bytes each kernel family must move per step (reads + writes of its operands)."""
        Nn, C, V, L, I = self.N, self.C, self.V, self.L, self.I
        qk = 2 * Nn * self.cfg.n_head * self.cfg.head_dim
        return {
            "gather_fwd": 8 * Nn * C,                              # read rows + write out
            "ln_fwd": self.n_norms * 16 * Nn * C,                  # read x, r; write h, y
            "ln_bwd": (self.n_norms * 16 - 4) * Nn * C,            # read dy, h, dres; write dx (first has no dres)
            "rope": 2 * L * 8 * qk,                                # fwd + bwd: read + write q, k
            "gelu_fwd": L * 8 * Nn * I,
            "gelu_bwd": L * 12 * Nn * I,
            "scatter_add": 4 * Nn * C + 8 * min(Nn, V) * C,        # read dOut; read-modify-write touched rows
            "zero_grads": 4 * (V * C + Nn * C),
        }

    def flce_flops(self):
        """(useful, executed) FLOPs of the fused linear+CE per step: 6NCV useful, 8NCV
        executed because the logits panels are recomputed in backward."""
        n = 2.0 * self.N * self.C * self.V
        return 3 * n, 4 * n
