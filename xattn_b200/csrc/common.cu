// Host utilities shared by the entry points: error text, tensor-map creation.
#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <vector>
#include "common.cuh"

namespace xb {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

const char* last_error() { return g_error; }

TensorMapEncodeFn tensor_map_encoder() {
  static TensorMapEncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<TensorMapEncodeFn>(p);
    }
  });
  return fn;
}

int make_tile_map(CUtensorMap* out, const void* base, int dtype, int64_t B, int64_t L, int64_t H, int64_t D,
                  int64_t sb, int64_t sl, int64_t sh, int box_rows, int box_heads) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (!enc) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return -1; }
  if (reinterpret_cast<uintptr_t>(base) & 15) { set_error("tensor base must be 16-byte aligned"); return -1; }
  // A dimension of extent 1 may carry any stride; give it a legal one.
  if (H == 1) sh = D;
  if (L == 1) sl = H * D > sh ? H * D : sh;
  if (B == 1) sb = L * sl;
  if (sb <= 0 || sl <= 0 || sh <= 0 || ((sb * 2) & 15) || ((sl * 2) & 15) || ((sh * 2) & 15)) {
    set_error("tensor strides must be positive multiples of 16 bytes (got %lld, %lld, %lld elements)",
              (long long)sb, (long long)sl, (long long)sh);
    return -1;
  }
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)L, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)sl * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_heads, (cuuint32_t)box_rows, 1};
  cuuint32_t elem[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == XATTN_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(out, dt, 4, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with code %d", (int)r); return -1; }
  return 0;
}

int make_row_map(CUtensorMap* out, const void* base, int64_t B, int64_t H, int64_t L, int box_rows) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (!enc) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return -1; }
  if (reinterpret_cast<uintptr_t>(base) & 15) { set_error("tensor base must be 16-byte aligned"); return -1; }
  cuuint64_t dims[4] = {16, (cuuint64_t)L, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {32, (cuuint64_t)L * 32, (cuuint64_t)H * L * 32};
  cuuint32_t box[4] = {16, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (row map) failed with code %d", (int)r); return -1; }
  return 0;
}

// ---- optional per-kernel timing -------------------------------------------------
namespace {
struct ProfRecord { int kind; cudaEvent_t start, stop; };
std::mutex g_prof_mutex;
std::vector<ProfRecord> g_prof_records;
std::vector<cudaEvent_t> g_prof_pool;
bool g_prof_on = false;
cudaEvent_t prof_event() {
  if (!g_prof_pool.empty()) { cudaEvent_t e = g_prof_pool.back(); g_prof_pool.pop_back(); return e; }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}
}  // namespace

ProfileScope::ProfileScope(int kind, cudaStream_t st) : slot(-1), stream(st) {
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  if (!g_prof_on) return;
  ProfRecord r{kind, prof_event(), prof_event()};
  if (!r.start || !r.stop) return;
  cudaEventRecord(r.start, stream);
  g_prof_records.push_back(r);
  slot = (int)g_prof_records.size() - 1;
}

ProfileScope::~ProfileScope() {
  if (slot < 0) return;
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  if (slot < (int)g_prof_records.size()) cudaEventRecord(g_prof_records[slot].stop, stream);
}

int profile_enable(int enable) {
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  g_prof_on = enable != 0;
  return 0;
}

int profile_read(int* kinds, float* ms, int capacity) {
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  int n = 0;
  for (const ProfRecord& r : g_prof_records) {
    float t = 0.f;
    if (cudaEventSynchronize(r.stop) == cudaSuccess && cudaEventElapsedTime(&t, r.start, r.stop) == cudaSuccess &&
        n < capacity) {
      kinds[n] = r.kind;
      ms[n] = t;
      ++n;
    }
    g_prof_pool.push_back(r.start);
    g_prof_pool.push_back(r.stop);
  }
  g_prof_records.clear();
  return n;
}

}  // namespace xb
