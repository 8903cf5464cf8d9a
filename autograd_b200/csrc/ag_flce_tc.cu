// tcgen05 tensor-core panels of the fused linear + cross-entropy head (placeholder: the
// tensor-core path is reported as unavailable, the exact-fp32 panels are used).
#include "ag_flce.cuh"

bool ag_flce_tc_supported(const ag_flce_desc*) { return false; }
size_t ag_flce_tc_scratch_bytes(const ag_flce_desc*) { return 0; }
int ag_flce_tc_prepare(ag_ctx* ctx, const ag_flce_desc*, const float*, const float*, void*) {
  AG_FAIL(ctx, AG_ERR_INVALID, "tensor-core FLCE path not available");
}
int ag_flce_tc_logits(ag_ctx* ctx, const ag_flce_desc*, void*, int64_t, int, int, int, float*, int64_t) {
  AG_FAIL(ctx, AG_ERR_INVALID, "tensor-core FLCE path not available");
}
