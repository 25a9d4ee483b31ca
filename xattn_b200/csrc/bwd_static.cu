// Backward pass for callers that must not allocate device memory.
//
// The regular backward entry takes a caller-provided workspace (two FP32 words per batch row, query
// head and query position, positions padded to whole 128-row tiles: -rowsum(dy*y) and -lse*log2e,
// plus a 32-byte row that carries the same two numbers into the tensor products).  Some callers cannot provide one: a plugin
// host that owns the whole device arena and hands an op nothing but its input and output buffers,
// or a serving loop where a cudaMalloc would stall every stream of the device at an unpredictable
// moment.  For them the same kernels run here with the workspace in a fixed array that lives in the
// library image: no cudaMalloc, cudaFree or allocating library call is made on any path of this file.
//
// Costs and rules:
//  * the array is part of the module, so every GPU that loads the library holds its
//    kStaticRows * 40 bytes (40 MiB) until the process exits, used or not;
//  * batch * q_heads * q_len may not exceed kStaticRows; larger problems are refused with
//    XATTN_E_INVALID before anything is launched;
//  * every call on a device shares the one array.  The preprocess kernel rewrites all entries it
//    later reads, so nothing has to be cleared between calls and a previous call's contents are
//    never observed; but two calls whose kernels overlap on the GPU (different streams, or threads
//    without ordering) would overwrite each other's rows — callers serialise them;
//  * the high-precision backward (high_precision = 1) needs 44 bytes per row instead of 40, so its
//    limit is 10/11 of kStaticRows;
//  * the first call on a device resolves the array's device address (cudaGetSymbolAddress, with
//    that device current).  Where the CUDA runtime loads modules lazily that call is also the one
//    that loads this module and reserves the array on the device: it can take milliseconds, and it
//    fails with an out-of-memory error if another owner already holds all device memory.  Make that
//    first call at start-up, before the arena owner takes the rest of the device and outside any
//    stream capture.
#include <mutex>
#include "common.cuh"

namespace xb {
int bwd_entry(const XattnBwdArgs* a, cudaStream_t stream);

namespace {

constexpr long long kStaticRows = 1ll << 20;   // batch * q_heads * (q_len rounded up to 128), at most
constexpr int kMaxDevices = 64;

// bwd_entry lays its two arrays out back to back from the start of whatever workspace it is given
static __device__ __align__(256) float g_static_workspace[10 * kStaticRows];   // 40 bytes per row

std::mutex g_static_mutex;
float* g_static_ptr[kMaxDevices] = {};

// Device address of the array on the current device; resolved once per device.
int static_workspace(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { set_error("cudaGetDevice: %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  if (dev < 0 || dev >= kMaxDevices) { set_error("device index %d out of range", dev); return XATTN_E_UNSUPPORTED; }
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_ptr[dev]) {
    // In host code the array's name is only a handle for the runtime, not an address a kernel can use.
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_workspace);
    if (e != cudaSuccess || !p) {
      set_error("cudaGetSymbolAddress(static workspace): %s", cudaGetErrorString(e));
      return XATTN_E_CUDA;
    }
    g_static_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_static_ptr[dev];
  return XATTN_OK;
}

}  // namespace

int bwd_static_entry(const XattnBwdArgs* a, cudaStream_t stream) {
  if (!a) { set_error("null arguments"); return XATTN_E_INVALID; }
  if (a->batch <= 0 || a->q_heads <= 0 || a->q_len <= 0) { set_error("bad batch / head / length"); return XATTN_E_INVALID; }
  // each factor is bounded before anything is multiplied, so the products below cannot overflow
  if (a->batch > kStaticRows || a->q_heads > kStaticRows || a->q_len > kStaticRows) {
    set_error("batch, q_heads or q_len alone exceeds the static workspace of %lld rows; "
              "use xattn_b200_bwd with a caller-provided workspace", kStaticRows);
    return XATTN_E_INVALID;
  }
  const long long padded = (a->q_len + 127) / 128 * 128;      // the kernels keep whole 128-row tiles
  const long long bh = (long long)a->batch * a->q_heads;       // <= 2^40
  const long long floats_per_row = a->high_precision ? 11 : 10;
  const long long max_rows = 10 * kStaticRows / floats_per_row;
  if (bh > max_rows || bh * padded > max_rows) {
    set_error("batch * q_heads * q_len (rounded up to 128) exceeds the static workspace of %lld rows; "
              "use xattn_b200_bwd with a caller-provided workspace", max_rows);
    return XATTN_E_INVALID;
  }
  float* ws = nullptr;
  if (int rc = static_workspace(&ws)) return rc;
  XattnBwdArgs with_ws = *a;
  with_ws.workspace = ws;            // whatever the caller put there is ignored
  return bwd_entry(&with_ws, stream);
}

long long bwd_static_max_rows() { return kStaticRows; }

}  // namespace xb

extern "C" int xattn_b200_bwd_static_scratch(const XattnBwdArgs* args, xattn_stream_t stream) {
  return xb::bwd_static_entry(args, static_cast<cudaStream_t>(stream));
}
