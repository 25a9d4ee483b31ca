// extern "C" surface of libxattn_b200 (declared in include/xattn_b200.h).
#include "common.cuh"

namespace xb {
const char* last_error();
int fwd_entry(const XattnFwdArgs* a, cudaStream_t stream);
int fwd_split_entry(const XattnFwdArgs* a, int64_t splits, void* workspace, size_t workspace_bytes, cudaStream_t stream);
size_t fwd_split_workspace_bytes(int64_t batch, int64_t q_len, int64_t q_heads, int64_t v_dim, int64_t splits);
int64_t fwd_split_suggest(int64_t batch, int64_t q_len, int64_t k_len, int64_t q_heads, int64_t kv_heads, int64_t sm_count);
int bwd_entry(const XattnBwdArgs* a, cudaStream_t stream);
int gate_fwd_entry(const XattnGateArgs* a, cudaStream_t stream);
int gate_bwd_entry(const XattnGateArgs* a, cudaStream_t stream);
int zero_constant_entry(const XattnConstantKeyArgs* a, cudaStream_t stream);
int merge_gradients_entry(const XattnMergeArgs* a, cudaStream_t stream);
int build_plan_entry(const XattnPlanArgs* a, cudaStream_t stream);
int build_varlen_plan_entry(const XattnVarlenPlanArgs* a, cudaStream_t stream);
int wait_timeout_probe_entry(int32_t* status, int64_t budget_us, cudaStream_t stream);
int merge_outputs_entry(const XattnMergeOutputsArgs* a, cudaStream_t stream);
}  // namespace xb

extern "C" {

int xattn_b200_abi_version(void) { return XATTN_B200_ABI_VERSION; }

const char* xattn_b200_last_error(void) { return xb::last_error(); }

size_t xattn_b200_plan_bytes(int64_t batch, int64_t q_len, int64_t k_len) {
  if (batch <= 0 || q_len <= 0 || k_len <= 0) return 0;
  return (size_t)xb::PlanLayout(batch, q_len, k_len).words * sizeof(int32_t);
}

int xattn_b200_build_plan(const XattnPlanArgs* args, xattn_stream_t stream) {
  return xb::build_plan_entry(args, static_cast<cudaStream_t>(stream));
}

int xattn_b200_build_varlen_plan(const XattnVarlenPlanArgs* args, xattn_stream_t stream) {
  return xb::build_varlen_plan_entry(args, static_cast<cudaStream_t>(stream));
}

int xattn_b200_fwd(const XattnFwdArgs* args, xattn_stream_t stream) {
  return xb::fwd_entry(args, static_cast<cudaStream_t>(stream));
}

int64_t xattn_b200_fwd_split_suggest(int64_t batch, int64_t q_len, int64_t k_len, int64_t q_heads,
                                     int64_t kv_heads, int64_t sm_count) {
  return xb::fwd_split_suggest(batch, q_len, k_len, q_heads, kv_heads, sm_count);
}

size_t xattn_b200_fwd_split_workspace_bytes(int64_t batch, int64_t q_len, int64_t q_heads, int64_t v_dim,
                                            int64_t splits) {
  return xb::fwd_split_workspace_bytes(batch, q_len, q_heads, v_dim, splits);
}

int xattn_b200_fwd_split(const XattnFwdArgs* args, int64_t splits, void* workspace, size_t workspace_bytes,
                         xattn_stream_t stream) {
  return xb::fwd_split_entry(args, splits, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

size_t xattn_b200_bwd_workspace_bytes(int64_t batch, int64_t q_heads, int64_t q_len) {
  if (batch <= 0 || q_heads <= 0 || q_len <= 0) return 0;
  // per (batch row, query head, query row), rows padded to whole 128-row tiles: two FP32 words
  // (-delta, -lse * log2e) and one 32-byte row of extra GEMM columns carrying the same numbers
  const size_t padded = ((size_t)q_len + 127) / 128 * 128;
  return (size_t)batch * q_heads * padded * (2 * sizeof(float) + 32);
}

size_t xattn_b200_bwd_workspace_bytes_hp(int64_t batch, int64_t q_heads, int64_t q_len) {
  if (batch <= 0 || q_heads <= 0 || q_len <= 0) return 0;
  // the low-precision layout plus one FP32 word per row: -dP at the anchor key
  const size_t padded = ((size_t)q_len + 127) / 128 * 128;
  return (size_t)batch * q_heads * padded * (3 * sizeof(float) + 32);
}

int xattn_b200_bwd(const XattnBwdArgs* args, xattn_stream_t stream) {
  return xb::bwd_entry(args, static_cast<cudaStream_t>(stream));
}

int xattn_b200_softdelta_gate_fwd(const XattnGateArgs* args, xattn_stream_t stream) {
  return xb::gate_fwd_entry(args, static_cast<cudaStream_t>(stream));
}

int xattn_b200_softdelta_gate_bwd(const XattnGateArgs* args, xattn_stream_t stream) {
  return xb::gate_bwd_entry(args, static_cast<cudaStream_t>(stream));
}

int xattn_b200_zero_constant_key_rows(const XattnConstantKeyArgs* args, xattn_stream_t stream) {
  return xb::zero_constant_entry(args, static_cast<cudaStream_t>(stream));
}

int xattn_b200_softdelta_merge_gradients(const XattnMergeArgs* args, xattn_stream_t stream) {
  return xb::merge_gradients_entry(args, static_cast<cudaStream_t>(stream));
}

int xattn_b200_profile_enable(int enable) { return xb::profile_enable(enable); }

int xattn_b200_profile_read(int* kinds, float* ms, int capacity) {
  if (!kinds || !ms || capacity < 0) return XATTN_E_INVALID;
  return xb::profile_read(kinds, ms, capacity);
}

int xattn_b200_merge_partial_outputs(const XattnMergeOutputsArgs* args, xattn_stream_t stream) {
  return xb::merge_outputs_entry(args, static_cast<cudaStream_t>(stream));
}

int xattn_b200_selftest_wait_timeout(int32_t* status, int64_t budget_us, xattn_stream_t stream) {
  return xb::wait_timeout_probe_entry(status, budget_us, static_cast<cudaStream_t>(stream));
}

int xattn_b200_check_status(const int32_t* status, xattn_stream_t stream) {
  int32_t host = 0;
  cudaError_t e = cudaMemcpyAsync(&host, status, sizeof(host), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) { xb::set_error("status read: %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  if (host != 0) {
    xb::set_error("kernel reported status %d (wait site %d)", host & 0xff, host >> 8);
    return XATTN_E_DEVICE;
  }
  return XATTN_OK;
}

}  // extern "C"
