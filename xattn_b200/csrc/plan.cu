// Mask plan: the visible keys of every query row as one interval [lo, hi),
// plus per-tile summaries.  HBM-bound integer work: a few bytes per row.
//
// Visibility rule restated from the reference's oracle (tests/_reference.py:35-131)
// and its device twins (csrc/attention/hopper/mask.h:197-442, hopper/block.h:17-179,
// csrc/flash_sca/hopper/sliding_chunk_attention.cu:1953-1963):
//   query i sits at position q_pos = i + Lk - Lq; key j is visible iff it has the
//   query's segment id, j <= q_pos (j < q_pos when strict), and
//     window: j >= q_pos - span      chunk: j >= floor(q_pos / span) * span - span.
//   With per-segment reset, positions count from the start of the segment run:
//     q_pos = (i - q_run_start) + (k_run_len - q_run_len),  key position = j - k_run_start.
// Key segment ids are nondecreasing along a row (csrc/attention/partition/segment_index.h:362-363),
// so the keys of one id form one run, found by binary search.
#include <cub/block/block_scan.cuh>
#include "common.cuh"

namespace xb {

__device__ __forceinline__ long long floor_div(long long a, long long b) {
  long long q = a / b;
  if ((a % b != 0) && ((a < 0) != (b < 0))) --q;
  return q;
}

// left edge (inclusive) of visible key positions for a query at position qp
__device__ __forceinline__ long long left_edge(int visibility, long long span, long long qp) {
  if (visibility == XATTN_VIS_WINDOW) return qp - span;
  if (visibility == XATTN_VIS_CHUNK) return floor_div(qp, span) * span - span;
  return LLONG_MIN / 4;
}

__device__ __forceinline__ int lower_bound_i64(const int64_t* a, int n, int64_t key) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (a[mid] < key) lo = mid + 1; else hi = mid;
  }
  return lo;
}
__device__ __forceinline__ int upper_bound_i64(const int64_t* a, int n, int64_t key) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (a[mid] <= key) lo = mid + 1; else hi = mid;
  }
  return lo;
}

struct MaxOp { __device__ int operator()(int a, int b) const { return a > b ? a : b; } };
struct MinOp { __device__ int operator()(int a, int b) const { return a < b ? a : b; } };

// Start and end of the run of equal ids around every position of a row.
// One block per batch row; forward max-scan for starts, backward min-scan for ends.
__global__ void __launch_bounds__(256) run_bounds_kernel(const int64_t* ids, int64_t row_stride, int L,
                                                         int* run_start, int* run_end) {
  typedef cub::BlockScan<int, 256> Scan;
  __shared__ typename Scan::TempStorage tmp;
  __shared__ int carry;
  const int64_t* row = ids + (size_t)blockIdx.x * row_stride;
  int* rs = run_start + (size_t)blockIdx.x * L;
  int* re = run_end + (size_t)blockIdx.x * L;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < L; base += 256) {
    const int i = base + threadIdx.x;
    int v = 0;
    if (i < L) v = (i == 0 || row[i] != row[i - 1]) ? i : 0;
    int out;
    Scan(tmp).InclusiveScan(v, out, MaxOp());
    const int c = carry;
    out = out > c ? out : c;
    if (i < L) rs[i] = out;
    __syncthreads();
    if (threadIdx.x == 255) carry = out;
    __syncthreads();
  }
  if (threadIdx.x == 0) carry = L;
  __syncthreads();
  const int nchunks = (L + 255) / 256;
  for (int ch = nchunks - 1; ch >= 0; --ch) {
    // thread t handles position base + 255 - t so that an inclusive scan runs right to left
    const int i = ch * 256 + 255 - threadIdx.x;
    int v = L;
    if (i < L) v = (i == L - 1 || row[i] != row[i + 1]) ? i + 1 : L;
    int out;
    Scan(tmp).InclusiveScan(v, out, MinOp());
    const int c = carry;
    out = out < c ? out : c;
    if (i < L) re[i] = out;
    __syncthreads();
    if (threadIdx.x == 255) carry = out;
    __syncthreads();
  }
}

struct RowArgs {
  int B, Lq, Lk;
  int visibility;
  long long span;
  int strict, reset;
  const int64_t* q_seg; const int64_t* k_seg;
  int64_t q_seg_stride, k_seg_stride;
  const int* q_run_start; const int* q_run_end;   // reset only
  int* row_lo; int* row_hi;
  int* status;                                    // optional: where a broken id contract is reported
};

// The binary searches above are only right when the key ids of a row never decrease (the reference's
// kernels assume the same, csrc/attention/partition/segment_index.h:362-363, and say nothing when it
// does not hold).  Each thread compares a share of the neighbouring key ids; a decrease stores
// (batch row << 8) | kStatusUnsortedSegments in the caller's status word.
__device__ __forceinline__ void check_key_ids(const RowArgs& a, long long first, long long stride) {
  if (!a.k_seg || !a.status) return;
  const long long total = (long long)a.B * a.Lk;
  for (long long j = first; j < total; j += stride) {
    const int b = (int)(j / a.Lk);
    const int jj = (int)(j - (long long)b * a.Lk);
    const int64_t* ks = a.k_seg + (size_t)b * a.k_seg_stride;
    if (jj > 0 && ks[jj] < ks[jj - 1]) atomicCAS(a.status, 0, ((b & 0x7fffff) << 8) | kStatusUnsortedSegments);
  }
}

// visible-key interval of query row i of batch row b (idx = b * Lq + i)
__device__ __forceinline__ void row_interval(const RowArgs& a, int b, int i, long long idx, int& out_lo, int& out_hi) {
  long long k_start = 0, k_end = a.Lk;
  if (a.q_seg) {
    const int64_t id = a.q_seg[(size_t)b * a.q_seg_stride + i];
    const int64_t* ks = a.k_seg + (size_t)b * a.k_seg_stride;
    k_start = lower_bound_i64(ks, a.Lk, id);
    k_end = upper_bound_i64(ks, a.Lk, id);
  }
  long long qp, origin;
  if (a.reset && a.q_seg) {
    const long long qs = a.q_run_start[idx], qe = a.q_run_end[idx];
    qp = (i - qs) + (k_end - k_start) - (qe - qs);
    origin = k_start;
  } else {
    qp = (long long)i + a.Lk - a.Lq;
    origin = 0;
  }
  long long lo = origin + left_edge(a.visibility, a.span, qp);
  long long hi = origin + qp + 1 - (a.strict ? 1 : 0);
  if (a.visibility == XATTN_VIS_ALL) hi = k_end;
  if (lo < k_start) lo = k_start;
  if (hi > k_end) hi = k_end;
  if (hi <= lo) { lo = 0; hi = 0; }
  out_lo = (int)lo;
  out_hi = (int)hi;
}

__global__ void __launch_bounds__(256) plan_rows_kernel(const RowArgs a) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  check_key_ids(a, idx, (long long)gridDim.x * blockDim.x);
  if (idx >= (long long)a.B * a.Lq) return;
  const int b = (int)(idx / a.Lq);
  const int i = (int)(idx - (long long)b * a.Lq);
  int lo, hi;
  row_interval(a, b, i, idx, lo, hi);
  a.row_lo[idx] = lo;
  a.row_hi[idx] = hi;
}

// The whole plan of a batch row in one block when the queries fit one tile (decode shapes, where the
// four launches of the general path cost as much as the attention itself): row intervals, the one
// query-tile summary, the key tiles it touches, and the identity as key-tile order (every key tile is
// seen by at most one query tile, so there is nothing to sort).  128 threads; blockIdx.x = batch row.
__global__ void __launch_bounds__(128) plan_one_tile_kernel(const RowArgs a, int nKT, TileInfo* q_tiles,
                                                            KeyTileInfo* k_tiles, int* k_order) {
  __shared__ int red[4][4];
  __shared__ int any_empty_s[4];
  const int b = blockIdx.x, i = threadIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  check_key_ids(a, (long long)blockIdx.x * blockDim.x + threadIdx.x, (long long)gridDim.x * blockDim.x);
  int min_lo = INT_MAX, max_hi = 0, max_lo = 0, min_hi = INT_MAX;
  bool any_empty = false;
  if (i < a.Lq) {
    const long long idx = (long long)b * a.Lq + i;
    int lo, hi;
    row_interval(a, b, i, idx, lo, hi);
    a.row_lo[idx] = lo;
    a.row_hi[idx] = hi;
    if (hi > lo) { min_lo = lo; max_hi = hi; max_lo = lo; min_hi = hi; } else { any_empty = true; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    min_lo = min(min_lo, __shfl_xor_sync(0xffffffffu, min_lo, o));
    max_hi = max(max_hi, __shfl_xor_sync(0xffffffffu, max_hi, o));
    max_lo = max(max_lo, __shfl_xor_sync(0xffffffffu, max_lo, o));
    min_hi = min(min_hi, __shfl_xor_sync(0xffffffffu, min_hi, o));
  }
  any_empty = __any_sync(0xffffffffu, any_empty);
  if (lane == 0) {
    red[warp][0] = min_lo; red[warp][1] = max_hi; red[warp][2] = max_lo; red[warp][3] = min_hi;
    any_empty_s[warp] = any_empty ? 1 : 0;
  }
  __syncthreads();
  min_lo = min(min(red[0][0], red[1][0]), min(red[2][0], red[3][0]));
  max_hi = max(max(red[0][1], red[1][1]), max(red[2][1], red[3][1]));
  max_lo = max(max(red[0][2], red[1][2]), max(red[2][2], red[3][2]));
  min_hi = min(min(red[0][3], red[1][3]), min(red[2][3], red[3][3]));
  any_empty = (any_empty_s[0] | any_empty_s[1] | any_empty_s[2] | any_empty_s[3]) != 0;
  TileInfo t;
  if (max_hi == 0) { t.min_lo = 0; t.max_hi = 0; t.max_lo = INT_MAX; t.min_hi = 0; }
  else { t.min_lo = min_lo; t.max_hi = max_hi; t.max_lo = any_empty ? INT_MAX : max_lo; t.min_hi = min_hi; }
  if (threadIdx.x == 0) q_tiles[b] = t;
  for (int kt = threadIdx.x; kt < nKT; kt += blockDim.x) {
    const int k0 = kt * kBlockN, k1 = k0 + kBlockN;
    const bool seen = t.max_hi > t.min_lo && t.min_lo < k1 && t.max_hi > k0;
    KeyTileInfo k;
    k.m_first = 0;
    k.m_end = seen ? 1 : 0;
    k_tiles[(size_t)b * nKT + kt] = k;
    k_order[(size_t)b * nKT + kt] = b * nKT + kt;
  }
}

struct VarlenRowArgs {
  int total_q, total_k, nq, nk;
  const int* cu_q; const int* cu_k;
  int visibility; long long span; int strict;
  int* row_lo; int* row_hi;
};

__global__ void __launch_bounds__(256) plan_varlen_rows_kernel(const VarlenRowArgs a) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= a.total_q) return;
  // sequence r with cu_q[r] <= i < cu_q[r+1] (zero-length sequences are skipped by the search)
  int lo_s = 0, hi_s = a.nq;
  while (lo_s < hi_s) {
    const int mid = (lo_s + hi_s) >> 1;
    if (a.cu_q[mid + 1] <= i) lo_s = mid + 1; else hi_s = mid;
  }
  const int r = lo_s;
  long long lo = 0, hi = 0;
  if (r < a.nq) {
    const int rk = r + (a.nk - a.nq);
    const long long q0 = a.cu_q[r], q1 = a.cu_q[r + 1];
    const long long k_start = a.cu_k[rk], k_end = a.cu_k[rk + 1];
    const long long qp = (i - q0) + (k_end - k_start) - (q1 - q0);
    lo = k_start + left_edge(a.visibility, a.span, qp);
    hi = k_start + qp + 1 - (a.strict ? 1 : 0);
    if (lo < k_start) lo = k_start;
    if (hi > k_end) hi = k_end;
    if (hi > a.total_k) hi = a.total_k;
    if (hi <= lo) { lo = 0; hi = 0; }
  }
  a.row_lo[i] = (int)lo;
  a.row_hi[i] = (int)hi;
}

// One warp per (batch, query tile).
__global__ void __launch_bounds__(128) plan_qtiles_kernel(const int* row_lo, const int* row_hi, int B, int Lq,
                                                          int nQT, TileInfo* out) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= B * nQT) return;
  const int b = w / nQT, qt = w - b * nQT;
  int min_lo = INT_MAX, max_hi = 0, max_lo = 0, min_hi = INT_MAX;
  bool any_empty = false;
  for (int r = lane; r < kBlockM; r += 32) {
    const int row = qt * kBlockM + r;
    if (row >= Lq) break;
    const int lo = row_lo[(size_t)b * Lq + row], hi = row_hi[(size_t)b * Lq + row];
    if (hi > lo) {
      min_lo = min(min_lo, lo); max_hi = max(max_hi, hi);
      max_lo = max(max_lo, lo); min_hi = min(min_hi, hi);
    } else {
      any_empty = true;
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    min_lo = min(min_lo, __shfl_xor_sync(0xffffffffu, min_lo, o));
    max_hi = max(max_hi, __shfl_xor_sync(0xffffffffu, max_hi, o));
    max_lo = max(max_lo, __shfl_xor_sync(0xffffffffu, max_lo, o));
    min_hi = min(min_hi, __shfl_xor_sync(0xffffffffu, min_hi, o));
  }
  any_empty = __any_sync(0xffffffffu, any_empty);
  if (lane == 0) {
    TileInfo t;
    if (max_hi == 0) { t.min_lo = 0; t.max_hi = 0; t.max_lo = INT_MAX; t.min_hi = 0; }
    else { t.min_lo = min_lo; t.max_hi = max_hi; t.max_lo = any_empty ? INT_MAX : max_lo; t.min_hi = min_hi; }
    out[w] = t;
  }
}

// One warp per (batch, key tile): which query tiles can see it.
__global__ void __launch_bounds__(128) plan_ktiles_kernel(const TileInfo* qt_info, int B, int nQT, int nKT,
                                                          KeyTileInfo* out) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= B * nKT) return;
  const int b = w / nKT, kt = w - b * nKT;
  const int k0 = kt * kBlockN, k1 = k0 + kBlockN;
  int first = INT_MAX, end = 0;
  for (int m = lane; m < nQT; m += 32) {
    const TileInfo t = qt_info[(size_t)b * nQT + m];
    if (t.max_hi > t.min_lo && t.min_lo < k1 && t.max_hi > k0) { first = min(first, m); end = max(end, m + 1); }
  }
  for (int o = 16; o > 0; o >>= 1) {
    first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
    end = max(end, __shfl_xor_sync(0xffffffffu, end, o));
  }
  if (lane == 0) { KeyTileInfo k; k.m_first = end > 0 ? first : 0; k.m_end = end; out[w] = k; }
}

// Key tiles of all batch rows ordered by the number of query tiles that see them, most first: the
// dK / dV kernel's CTAs differ a lot in length under packed segments, and the hardware hands CTAs
// to SMs in index order, so the long ones have to come first for the SMs to finish together.
// One block; a counting sort (the order among equals is whatever the atomics give: it only
// affects scheduling).  More bins than fit shared memory: identity order.
constexpr int kOrderMaxBins = 8192;
__global__ void __launch_bounds__(1024) plan_korder_kernel(const KeyTileInfo* kt, int items, int nQT, int* order) {
  __shared__ int hist[kOrderMaxBins + 1];
  typedef cub::BlockScan<int, 1024> Scan;
  __shared__ typename Scan::TempStorage scan_tmp;
  const int bins = nQT + 1, tid = threadIdx.x;
  if (bins > kOrderMaxBins) {
    for (int i = tid; i < items; i += 1024) order[i] = i;
    return;
  }
  for (int i = tid; i < bins; i += 1024) hist[i] = 0;
  __syncthreads();
  for (int i = tid; i < items; i += 1024) {
    const int w = min(max(kt[i].m_end - kt[i].m_first, 0), nQT);
    atomicAdd(&hist[nQT - w], 1);             // bin 0 = most work
  }
  __syncthreads();
  int carry = 0;
  for (int base = 0; base < bins; base += 1024) {
    const int i = base + tid;
    const int v = i < bins ? hist[i] : 0;
    int excl, total;
    Scan(scan_tmp).ExclusiveSum(v, excl, total);
    if (i < bins) hist[i] = carry + excl;
    carry += total;
    __syncthreads();
  }
  for (int i = tid; i < items; i += 1024) {
    const int w = min(max(kt[i].m_end - kt[i].m_first, 0), nQT);
    order[atomicAdd(&hist[nQT - w], 1)] = i;
  }
}

static int finish_plan(int32_t* plan, const PlanLayout& pl, int B, int Lq, cudaStream_t stream) {
  const int nQT = (int)pl.nQT, nKT = (int)pl.nKT;
  TileInfo* qt = reinterpret_cast<TileInfo*>(plan + pl.off_qt);
  KeyTileInfo* kt = reinterpret_cast<KeyTileInfo*>(plan + pl.off_kt);
  plan_qtiles_kernel<<<ceil_div(B * nQT * 32, 128), 128, 0, stream>>>(plan + pl.off_lo, plan + pl.off_hi, B, Lq, nQT, qt);
  plan_ktiles_kernel<<<ceil_div(B * nKT * 32, 128), 128, 0, stream>>>(qt, B, nQT, nKT, kt);
  plan_korder_kernel<<<1, 1024, 0, stream>>>(kt, B * nKT, nQT, plan + pl.off_ko);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("plan launch: %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  return XATTN_OK;
}

int build_plan_entry(const XattnPlanArgs* a, cudaStream_t stream) {
  if (!a || !a->plan) { set_error("null plan arguments"); return XATTN_E_INVALID; }
  if (a->batch <= 0 || a->q_len <= 0 || a->k_len <= 0 || a->batch * a->q_len > 0x7fffffffLL || a->k_len > 0x7fffffffLL) {
    set_error("plan sizes out of range"); return XATTN_E_INVALID;
  }
  if (a->visibility < XATTN_VIS_FULL || a->visibility > XATTN_VIS_ALL) { set_error("unknown visibility"); return XATTN_E_INVALID; }
  if (a->visibility == XATTN_VIS_WINDOW && a->span < 0) { set_error("window_size must be nonnegative"); return XATTN_E_INVALID; }
  if (a->visibility == XATTN_VIS_CHUNK && a->span <= 0) { set_error("chunk_size must be positive"); return XATTN_E_INVALID; }
  if ((a->q_segment == nullptr) != (a->k_segment == nullptr)) { set_error("q_segment and k_segment must be given together"); return XATTN_E_INVALID; }
  const int B = (int)a->batch, Lq = (int)a->q_len, Lk = (int)a->k_len;
  const PlanLayout pl(B, Lq, Lk);
  ProfileScope prof(kProfPlan, stream);
  RowArgs r;
  r.B = B; r.Lq = Lq; r.Lk = Lk; r.visibility = a->visibility; r.span = a->span; r.strict = a->strict_past;
  r.reset = a->reset_positions && a->q_segment; r.q_seg = a->q_segment; r.k_seg = a->k_segment;
  r.q_seg_stride = a->q_segment_stride; r.k_seg_stride = a->k_segment_stride;
  r.row_lo = a->plan + pl.off_lo; r.row_hi = a->plan + pl.off_hi;
  r.q_run_start = r.q_run_end = nullptr;
  r.status = a->status;
  if (r.reset) {
    // run starts / ends are staged in the row_lo / row_hi slots; plan_rows_kernel reads
    // its own slot before overwriting it
    run_bounds_kernel<<<B, 256, 0, stream>>>(a->q_segment, a->q_segment_stride, Lq, r.row_lo, r.row_hi);
    r.q_run_start = r.row_lo; r.q_run_end = r.row_hi;
  }
  if (Lq <= kBlockM && !r.reset) {
    plan_one_tile_kernel<<<B, 128, 0, stream>>>(r, (int)pl.nKT, reinterpret_cast<TileInfo*>(a->plan + pl.off_qt),
                                               reinterpret_cast<KeyTileInfo*>(a->plan + pl.off_kt), a->plan + pl.off_ko);
    cudaError_t e1 = cudaGetLastError();
    if (e1 != cudaSuccess) { set_error("plan launch: %s", cudaGetErrorString(e1)); return XATTN_E_CUDA; }
    return XATTN_OK;
  }
  plan_rows_kernel<<<ceil_div(B * Lq, 256), 256, 0, stream>>>(r);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("plan launch: %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  return finish_plan(a->plan, pl, B, Lq, stream);
}

int build_varlen_plan_entry(const XattnVarlenPlanArgs* a, cudaStream_t stream) {
  if (!a || !a->plan || !a->cu_seqlens_q || !a->cu_seqlens_k) { set_error("null varlen plan arguments"); return XATTN_E_INVALID; }
  if (a->total_q <= 0 || a->total_k <= 0 || a->total_q > 0x7fffffffLL || a->total_k > 0x7fffffffLL ||
      a->num_q_seqs < 1 || a->num_k_seqs < a->num_q_seqs) { set_error("bad varlen sizes"); return XATTN_E_INVALID; }
  if (a->visibility == XATTN_VIS_CHUNK && a->span <= 0) { set_error("chunk_size must be positive"); return XATTN_E_INVALID; }
  const PlanLayout pl(1, a->total_q, a->total_k);
  ProfileScope prof(kProfPlan, stream);
  VarlenRowArgs r;
  r.total_q = (int)a->total_q; r.total_k = (int)a->total_k; r.nq = (int)a->num_q_seqs; r.nk = (int)a->num_k_seqs;
  r.cu_q = a->cu_seqlens_q; r.cu_k = a->cu_seqlens_k; r.visibility = a->visibility; r.span = a->span; r.strict = a->strict_past;
  r.row_lo = a->plan + pl.off_lo; r.row_hi = a->plan + pl.off_hi;
  plan_varlen_rows_kernel<<<ceil_div(r.total_q, 256), 256, 0, stream>>>(r);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("plan launch: %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  return finish_plan(a->plan, pl, 1, r.total_q, stream);
}

}  // namespace xb
