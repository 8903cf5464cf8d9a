// pybind11 module `cuda_ext`: the C ABI of include/autograd_b200.h, one Python function per entry
// point, in the place the reference gives its own native binding (a pybind11 module built by
// setup.py: metal_ext.mm:770-796, setup.py:13-36).
//
// The module is a binding and nothing else: it contains no CUDA code and no logic of its own, it
// links against libautograd_b200.so next to it.  Every pointer parameter of the C function (device
// pointers, host pointers, the context handle, out-parameters, the CE descriptor) is an integer
// address on the Python side; scalars pass through; the C function's return value is returned
// unchanged, so status codes are checked by the caller exactly as with the ctypes binding
// (autograd_b200/_native.py), which stays the default.  AG_B200_BINDING=pybind11 selects this one.
#include <pybind11/pybind11.h>

#include <cstdint>
#include <string>

#include "autograd_b200.h"

namespace py = pybind11;

namespace {

// C parameter type -> Python-side type and the conversion back
template <typename T>
struct Arg {
  using py_t = T;
  static T to_c(T v) { return v; }
};
template <typename T>
struct Arg<T*> {
  using py_t = std::uintptr_t;
  static T* to_c(std::uintptr_t v) { return reinterpret_cast<T*>(v); }
};

template <typename R, typename... A>
auto wrap(R (*fn)(A...)) {
  return [fn](typename Arg<A>::py_t... a) -> R { return fn(Arg<A>::to_c(a)...); };
}

}  // namespace

#define AG_DEF(name) m.def(#name, wrap(&name))

PYBIND11_MODULE(cuda_ext, m) {
  m.doc() = "C ABI of libautograd_b200.so; pointers are integer addresses, return values are the C function's own";

  AG_DEF(ag_ctx_create);
  AG_DEF(ag_ctx_destroy);
  AG_DEF(ag_set_stream);
  m.def("ag_last_error", [](std::uintptr_t ctx) {
    const char* msg = ag_last_error(reinterpret_cast<const ag_ctx*>(ctx));
    return py::bytes(msg ? std::string(msg) : std::string());
  });
  AG_DEF(ag_device_info);
  AG_DEF(ag_alloc);
  AG_DEF(ag_free);
  AG_DEF(ag_copy_h2d);
  AG_DEF(ag_copy_d2h);
  AG_DEF(ag_synchronize);
  AG_DEF(ag_status);
  AG_DEF(ag_launch_count);
  AG_DEF(ag_pass_begin_profiled);
  AG_DEF(ag_pass_end_profiled);
  AG_DEF(ag_event_record);
  AG_DEF(ag_event_elapsed);
  AG_DEF(ag_tc_timing);
  AG_DEF(ag_tc_timing_count);
  AG_DEF(ag_alloc_host);
  AG_DEF(ag_free_host);
  AG_DEF(ag_fill_f32);
  AG_DEF(ag_fill_pattern);
  AG_DEF(ag_add_forward);
  AG_DEF(ag_add_backward);
  AG_DEF(ag_add_layernorm_forward);
  AG_DEF(ag_norm_partials_bytes);
  AG_DEF(ag_layernorm_backward);
  AG_DEF(ag_layernorm_backward_noalloc);
  AG_DEF(ag_debug_expire_staging);
  AG_DEF(ag_rmsnorm_forward);
  AG_DEF(ag_rmsnorm_backward);
  AG_DEF(ag_gelu_forward);
  AG_DEF(ag_gelu_backward);
  AG_DEF(ag_swiglu_forward);
  AG_DEF(ag_swiglu_backward);
  AG_DEF(ag_rope_qk);
  AG_DEF(ag_gather_forward);
  AG_DEF(ag_scatter_add_scratch_bytes);
  AG_DEF(ag_gather_backward);
  AG_DEF(ag_flce_scratch_bytes);
  AG_DEF(ag_flce_forward);
  AG_DEF(ag_flce_backward);
  AG_DEF(ag_linear_add_scratch_bytes);
  AG_DEF(ag_linear_add_forward);
  AG_DEF(ag_linear_add_backward);
  AG_DEF(ag_adamw_step);
  AG_DEF(ag_f32_to_bf16);
  AG_DEF(ag_bf16_to_f32);
  AG_DEF(ag_gather_backward_bf16);
  AG_DEF(ag_adamw_step_bf16grad);
}
