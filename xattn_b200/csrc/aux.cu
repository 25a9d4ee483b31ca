// HBM-bound helpers around the attention kernels.
//
//   SoftDelta gate:   y = read - sigmoid(g) * neg_read                    (forward)
//                     read = y + sigmoid(g) * neg_read, d neg_read, dg     (backward, one pass)
//     restated from csrc/softdelta/gate.cu:25-27 (sigmoid in FP32), :76-132 (forward),
//     :228 (backward) and csrc/softdelta/preprocess.cu:98-103 (query reads recovered from y).
//   Constant-key rows: dQ of a row whose visible keys are all the same vector is exactly zero
//     (csrc/attention/precision/constant_keys.cu: key-equality runs, then zero those rows).
//
// Every access is a 16-byte vector (or two for FP32): a lane owns 8 consecutive channels.
#include <cub/block/block_scan.cuh>
#include "common.cuh"

namespace xb {

__device__ __forceinline__ float sigmoid_f32(float x) { return 1.f / (1.f + __expf(-x)); }

template <typename T>
__device__ __forceinline__ void load8(const T* p, float* f) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) { const float2 t = Pack2<T>::unpack(w[k]); f[2 * k] = t.x; f[2 * k + 1] = t.y; }
}
__device__ __forceinline__ void load8_f32(const float* p, float* f) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float* f) {
  uint4 u;
  u.x = Pack2<T>::pack(f[0], f[1]); u.y = Pack2<T>::pack(f[2], f[3]);
  u.z = Pack2<T>::pack(f[4], f[5]); u.w = Pack2<T>::pack(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ __nv_bfloat16 from_f32(float x) { return __float2bfloat16(x); }
template <> __device__ __forceinline__ __half from_f32(float x) { return __float2half(x); }

// rows = B * L; read / y: [rows][H][V], neg: [rows][Hkv][V], g: [rows][H][C] with one gate per
// group of Dg = V / C consecutive channels (C = 1: one gate per head).
//
// A group of 8, 16 or 32 lanes (one 16-byte chunk of the V channels each) takes a unit = (row, KV head)
// and walks the G query heads of that KV head; it keeps kGateUnits units in flight, with the loads of
// all of them issued before the first use.  With u = row * Hkv + kv the addresses need no division:
// neg at u * V, head r of the group at (u * G + r) * V, its gates at (u * G + r) * C.
constexpr int kGateUnits = 4;
constexpr int kGateThreads = 128;   // small blocks: the backward needs ~150 registers per thread

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) { const float2 t = Pack2<T>::unpack(w[k]); f[2 * k] = t.x; f[2 * k + 1] = t.y; }
}

// neg_read of the units in flight: raw 16-bit chunks, or FP32 values (level 1)
template <typename T, bool NEG_F32> struct NegRegs;
template <typename T> struct NegRegs<T, false> {
  uint4 raw[kGateUnits];
  __device__ __forceinline__ void load(int ps, const void* neg, long long off) {
    raw[ps] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(neg) + off));
  }
  __device__ __forceinline__ void clear(int ps) { raw[ps] = make_uint4(0, 0, 0, 0); }
  __device__ __forceinline__ void get(int ps, float* f) const { unpack8<T>(raw[ps], f); }
};
template <typename T> struct NegRegs<T, true> {
  float val[kGateUnits][8];
  __device__ __forceinline__ void load(int ps, const void* neg, long long off) {
    load8_f32(reinterpret_cast<const float*>(neg) + off, val[ps]);
  }
  __device__ __forceinline__ void clear(int ps) {
#pragma unroll
    for (int e = 0; e < 8; ++e) val[ps][e] = 0.f;
  }
  __device__ __forceinline__ void get(int ps, float* f) const {
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = val[ps][e];
  }
};

struct GateLanes {
  int group, per_pass, sub, ch, c;
  bool lane_on;
  long long first, total;
  __device__ __forceinline__ GateLanes(long long rows, int Hkv, int V) {
    const int chunks = V >> 3;
    group = chunks <= 8 ? 8 : (chunks <= 16 ? 16 : 32);
    per_pass = 32 / group;
    const int lane = threadIdx.x & 31;
    sub = lane / group;
    ch = lane % group;
    c = ch * 8;
    lane_on = ch < chunks;
    total = rows * Hkv;
    first = (((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5) * (per_pass * kGateUnits) + sub;
  }
  __device__ __forceinline__ long long unit(int ps) const { return first + (long long)ps * per_pass; }
  __device__ __forceinline__ bool on(int ps) const { return lane_on && unit(ps) < total; }
};

template <typename T, bool NEG_F32>
__global__ void __launch_bounds__(kGateThreads) gate_fwd_kernel(const T* __restrict__ read, const void* __restrict__ neg_,
                                                       const T* __restrict__ g, T* __restrict__ y, long long rows,
                                                       int H, int Hkv, int V, int C, int Dg) {
  const GateLanes ln(rows, Hkv, V);
  const int G = H / Hkv;
  NegRegs<T, NEG_F32> neg;
#pragma unroll
  for (int ps = 0; ps < kGateUnits; ++ps) {
    neg.clear(ps);
    if (ln.on(ps)) neg.load(ps, neg_, ln.unit(ps) * V + ln.c);
  }
  for (int r = 0; r < G; ++r) {
    uint4 xr[kGateUnits];
    T graw[kGateUnits];
#pragma unroll
    for (int ps = 0; ps < kGateUnits; ++ps) {
      xr[ps] = make_uint4(0, 0, 0, 0);
      graw[ps] = from_f32<T>(0.f);
      if (ln.on(ps)) {
        const long long hr = ln.unit(ps) * G + r;
        xr[ps] = *reinterpret_cast<const uint4*>(read + hr * V + ln.c);   // y may be read itself: no __ldg
        if (C == 1) graw[ps] = g[hr];
      }
    }
#pragma unroll
    for (int ps = 0; ps < kGateUnits; ++ps) {
      if (!ln.on(ps)) continue;
      const long long hr = ln.unit(ps) * G + r;
      float x[8], n[8];
      unpack8<T>(xr[ps], x);
      neg.get(ps, n);
      if (C == 1) {
        const float gate = sigmoid_f32(to_f32<T>(graw[ps]));
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = x[e] - gate * n[e];
      } else {
        const T* gh = g + hr * C;
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = x[e] - sigmoid_f32(to_f32<T>(gh[(ln.c + e) / Dg])) * n[e];
      }
      store8<T>(y + hr * V + ln.c, x);
    }
  }
}

template <typename T, bool NEG_F32>
__global__ void __launch_bounds__(kGateThreads) gate_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y,
                                                       const void* __restrict__ neg_, const T* __restrict__ g,
                                                       T* __restrict__ read, T* __restrict__ dneg, T* __restrict__ dg,
                                                       long long rows, int H, int Hkv, int V, int C, int Dg) {
  const GateLanes ln(rows, Hkv, V);
  const int G = H / Hkv;
  NegRegs<T, NEG_F32> neg;
  float dn[kGateUnits][8];
#pragma unroll
  for (int ps = 0; ps < kGateUnits; ++ps) {
    neg.clear(ps);
    if (ln.on(ps)) neg.load(ps, neg_, ln.unit(ps) * V + ln.c);
#pragma unroll
    for (int e = 0; e < 8; ++e) dn[ps][e] = 0.f;
  }
  for (int r = 0; r < G; ++r) {
    uint4 dr[kGateUnits], yr[kGateUnits];
    T graw[kGateUnits];
#pragma unroll
    for (int ps = 0; ps < kGateUnits; ++ps) {
      dr[ps] = make_uint4(0, 0, 0, 0);
      yr[ps] = make_uint4(0, 0, 0, 0);
      graw[ps] = from_f32<T>(0.f);
      if (ln.on(ps)) {
        const long long hr = ln.unit(ps) * G + r;
        dr[ps] = __ldg(reinterpret_cast<const uint4*>(dy + hr * V + ln.c));
        yr[ps] = __ldg(reinterpret_cast<const uint4*>(y + hr * V + ln.c));
        if (C == 1) graw[ps] = g[hr];
      }
    }
#pragma unroll
    for (int ps = 0; ps < kGateUnits; ++ps) {
      const bool on = ln.on(ps);
      const long long hr = ln.unit(ps) * G + r;
      float d[8], yy[8], n[8];
      unpack8<T>(dr[ps], d);
      unpack8<T>(yr[ps], yy);
      neg.get(ps, n);
      if (C == 1) {
        const float gate = sigmoid_f32(to_f32<T>(graw[ps]));
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          dn[ps][e] -= gate * d[e];
          dot += d[e] * n[e];
          yy[e] += gate * n[e];
        }
        for (int o = ln.group >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (on && ln.ch == 0) dg[hr] = from_f32<T>(-dot * gate * (1.f - gate));
      } else {
        const T* gh = g + hr * C;
        if (on) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float gate = sigmoid_f32(to_f32<T>(gh[(ln.c + e) / Dg]));
            dn[ps][e] -= gate * d[e];
            yy[e] += gate * n[e];
          }
        }
        // one gate gradient per value group: the group's share of <dy, neg_read>
        for (int j = 0; j < C; ++j) {
          float dot = 0.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) dot += ((ln.c + e) / Dg == j) ? d[e] * n[e] : 0.f;
          for (int o = ln.group >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
          if (on && ln.ch == 0) {
            const float gate = sigmoid_f32(to_f32<T>(gh[j]));
            dg[hr * C + j] = from_f32<T>(-dot * gate * (1.f - gate));
          }
        }
      }
      if (on) store8<T>(read + hr * V + ln.c, yy);
    }
  }
#pragma unroll
  for (int ps = 0; ps < kGateUnits; ++ps)
    if (ln.on(ps)) store8<T>(dneg + ln.unit(ps) * V + ln.c, dn[ps]);
}

// ---- SoftDelta gradient merge -------------------------------------------------
// out = a + b (+ tail on the last rows of each batch row), FP32 sum, one rounding.  A thread takes
// kMergeChunks 16-byte chunks a block-width apart, all loads first; blockIdx.y is the batch row.
constexpr int kMergeChunks = 4;
template <typename T>
__global__ void __launch_bounds__(256) merge_gradients_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                              const T* __restrict__ tail, T* __restrict__ out,
                                                              long long per_batch, long long tail_start,
                                                              long long tail_per_batch, int B) {
  for (int bi = blockIdx.y; bi < B; bi += gridDim.y) {
    const long long base = (long long)bi * per_batch;
    const long long i0 = ((long long)blockIdx.x * kMergeChunks * blockDim.x + threadIdx.x) * 8;
    uint4 ra[kMergeChunks], rb[kMergeChunks], rt[kMergeChunks];
#pragma unroll
    for (int u = 0; u < kMergeChunks; ++u) {
      const long long i = i0 + (long long)u * blockDim.x * 8;
      ra[u] = rb[u] = rt[u] = make_uint4(0, 0, 0, 0);
      if (i < per_batch) {
        ra[u] = *reinterpret_cast<const uint4*>(a + base + i);       // out may be a: no read-only path
        rb[u] = __ldg(reinterpret_cast<const uint4*>(b + base + i));
        if (tail && i >= tail_start)
          rt[u] = __ldg(reinterpret_cast<const uint4*>(tail + (long long)bi * tail_per_batch + (i - tail_start)));
      }
    }
#pragma unroll
    for (int u = 0; u < kMergeChunks; ++u) {
      const long long i = i0 + (long long)u * blockDim.x * 8;
      if (i >= per_batch) continue;
      float fa[8], fb[8], ft[8];
      unpack8<T>(ra[u], fa);
      unpack8<T>(rb[u], fb);
      unpack8<T>(rt[u], ft);
#pragma unroll
      for (int e = 0; e < 8; ++e) fa[e] = (fa[e] + fb[e]) + ft[e];
      store8<T>(out + base + i, fa);
    }
  }
}

// ---- constant-key rows ------------------------------------------------------
// flag[b][kvh][j] = 1 when key j differs (bitwise) from key j-1, or j == 0
template <typename T>
__global__ void __launch_bounds__(256) key_change_kernel(const T* __restrict__ k, int64_t sb, int64_t sl, int64_t sh,
                                                         int B, int Lk, int Hkv, int D, int* __restrict__ flag) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)B * Hkv * Lk) return;
  const int j = (int)(w % Lk);
  const long long bh = w / Lk;
  const int kv = (int)(bh % Hkv);
  const int b = (int)(bh / Hkv);
  bool diff = (j == 0);
  if (j > 0) {
    const T* a = k + b * sb + (long long)j * sl + kv * sh;
    const T* p = a - sl;
    for (int c = lane * 8; c < D; c += 256) {
      const uint4 x = *reinterpret_cast<const uint4*>(a + c), y = *reinterpret_cast<const uint4*>(p + c);
      diff |= (x.x != y.x) | (x.y != y.y) | (x.z != y.z) | (x.w != y.w);
    }
  }
  diff = __any_sync(0xffffffffu, diff);
  if (lane == 0) flag[w] = diff ? 1 : 0;
}

// in-place inclusive sum along the last axis, one block per row
__global__ void __launch_bounds__(256) row_cumsum_kernel(int* data, int L) {
  typedef cub::BlockScan<int, 256> Scan;
  __shared__ typename Scan::TempStorage tmp;
  __shared__ int carry;
  int* row = data + (size_t)blockIdx.x * L;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < L; base += 256) {
    const int i = base + threadIdx.x;
    const int v = i < L ? row[i] : 0;
    int out;
    Scan(tmp).InclusiveSum(v, out);
    out += carry;
    if (i < L) row[i] = out;
    __syncthreads();
    if (threadIdx.x == 255) carry = out;
    __syncthreads();
  }
}

template <typename T>
__global__ void __launch_bounds__(256) zero_constant_rows_kernel(T* __restrict__ dq, const int* __restrict__ row_lo,
                                                                 const int* __restrict__ row_hi,
                                                                 const int* __restrict__ run_id, int B, int Lq, int Lk,
                                                                 int Hq, int Hkv, int D) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)B * Lq * Hq) return;
  const int h = (int)(w % Hq);
  const long long bi = w / Hq;
  const int b = (int)(bi / Lq);
  const int lo = row_lo[bi], hi = row_hi[bi];
  if (hi <= lo) return;
  const int kv = h / (Hq / Hkv);
  const int* ids = run_id + ((size_t)b * Hkv + kv) * Lk;
  if (ids[lo] != ids[hi - 1]) return;
  T* out = dq + w * D;
  for (int c = lane * 8; c < D; c += 256) *reinterpret_cast<uint4*>(out + c) = make_uint4(0, 0, 0, 0);
}

// ---- host entries -------------------------------------------------------------
static int check_gate(const XattnGateArgs* a) {
  if (!a) { set_error("null arguments"); return XATTN_E_INVALID; }
  if (a->dtype != XATTN_DTYPE_F16 && a->dtype != XATTN_DTYPE_BF16) { set_error("dtype must be fp16 or bf16"); return XATTN_E_INVALID; }
  if (a->rows <= 0 || a->q_heads <= 0 || a->kv_heads <= 0 || a->q_heads % a->kv_heads || a->v_dim < 8 || a->v_dim > 256 || a->v_dim % 8) {
    set_error("bad gate sizes"); return XATTN_E_INVALID;
  }
  if (!a->y || !a->neg_read || !a->g) { set_error("null tensor pointer"); return XATTN_E_INVALID; }
  if (a->value_groups < 0 || (a->value_groups > 1 && a->v_dim % a->value_groups)) {
    set_error("value_groups must divide v_dim"); return XATTN_E_INVALID;
  }
  return XATTN_OK;
}

// warps needed when a warp takes kGateUnits * (32 / lanes per unit) units
static long long gate_warps(const XattnGateArgs* a) {
  const int chunks = (int)a->v_dim >> 3;
  const int per_warp = kGateUnits * 32 / (chunks <= 8 ? 8 : (chunks <= 16 ? 16 : 32));
  return (a->rows * a->kv_heads + per_warp - 1) / per_warp;
}

template <typename T>
static void launch_gate_fwd(const XattnGateArgs* a, cudaStream_t s) {
  const int groups = a->value_groups > 1 ? (int)a->value_groups : 1;
  const long long warps = gate_warps(a);
  const unsigned blocks = (unsigned)((warps * 32 + kGateThreads - 1) / kGateThreads);
  if (a->neg_is_f32)
    gate_fwd_kernel<T, true><<<blocks, kGateThreads, 0, s>>>((const T*)a->read, a->neg_read, (const T*)a->g, (T*)a->y, a->rows, (int)a->q_heads, (int)a->kv_heads, (int)a->v_dim, groups, (int)a->v_dim / groups);
  else
    gate_fwd_kernel<T, false><<<blocks, kGateThreads, 0, s>>>((const T*)a->read, a->neg_read, (const T*)a->g, (T*)a->y, a->rows, (int)a->q_heads, (int)a->kv_heads, (int)a->v_dim, groups, (int)a->v_dim / groups);
}
template <typename T>
static void launch_gate_bwd(const XattnGateArgs* a, cudaStream_t s) {
  const int groups = a->value_groups > 1 ? (int)a->value_groups : 1;
  const long long warps = gate_warps(a);
  const unsigned blocks = (unsigned)((warps * 32 + kGateThreads - 1) / kGateThreads);
  if (a->neg_is_f32)
    gate_bwd_kernel<T, true><<<blocks, kGateThreads, 0, s>>>((const T*)a->dy, (const T*)a->y, a->neg_read, (const T*)a->g, (T*)a->read, (T*)a->dneg_read, (T*)a->dg, a->rows, (int)a->q_heads, (int)a->kv_heads, (int)a->v_dim, groups, (int)a->v_dim / groups);
  else
    gate_bwd_kernel<T, false><<<blocks, kGateThreads, 0, s>>>((const T*)a->dy, (const T*)a->y, a->neg_read, (const T*)a->g, (T*)a->read, (T*)a->dneg_read, (T*)a->dg, a->rows, (int)a->q_heads, (int)a->kv_heads, (int)a->v_dim, groups, (int)a->v_dim / groups);
}

int gate_fwd_entry(const XattnGateArgs* a, cudaStream_t s) {
  if (int rc = check_gate(a)) return rc;
  if (!a->read) { set_error("null read pointer"); return XATTN_E_INVALID; }
  ProfileScope prof(kProfGate, s);
  if (a->dtype == XATTN_DTYPE_BF16) launch_gate_fwd<__nv_bfloat16>(a, s); else launch_gate_fwd<__half>(a, s);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("gate forward launch: %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  return XATTN_OK;
}

int gate_bwd_entry(const XattnGateArgs* a, cudaStream_t s) {
  if (int rc = check_gate(a)) return rc;
  if (!a->dy || !a->read || !a->dneg_read || !a->dg) { set_error("null gradient pointer"); return XATTN_E_INVALID; }
  ProfileScope prof(kProfGate, s);
  if (a->dtype == XATTN_DTYPE_BF16) launch_gate_bwd<__nv_bfloat16>(a, s); else launch_gate_bwd<__half>(a, s);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("gate backward launch: %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  return XATTN_OK;
}

int merge_gradients_entry(const XattnMergeArgs* a, cudaStream_t s) {
  if (!a || !a->a || !a->b || !a->out) { set_error("null arguments"); return XATTN_E_INVALID; }
  if (a->dtype != XATTN_DTYPE_F16 && a->dtype != XATTN_DTYPE_BF16) { set_error("dtype must be fp16 or bf16"); return XATTN_E_INVALID; }
  if (a->batch <= 0 || a->k_len <= 0 || a->kv_heads <= 0 || a->dim <= 0 || a->dim % 8 ||
      (a->tail && (a->tail_len <= 0 || a->tail_len > a->k_len))) { set_error("bad merge sizes"); return XATTN_E_INVALID; }
  const uintptr_t align = reinterpret_cast<uintptr_t>(a->a) | reinterpret_cast<uintptr_t>(a->b) |
                          reinterpret_cast<uintptr_t>(a->out) | reinterpret_cast<uintptr_t>(a->tail);
  if (align & 15) { set_error("merge tensors must be 16-byte aligned"); return XATTN_E_INVALID; }
  const long long row = a->kv_heads * a->dim;
  const long long per_batch = a->k_len * row;
  const long long tail_per_batch = a->tail ? a->tail_len * row : 0;
  const long long tail_start = per_batch - tail_per_batch;
  const long long per_block = 256LL * kMergeChunks * 8;
  const long long blocks = (per_batch + per_block - 1) / per_block;
  if (blocks > 0x7fffffffLL) { set_error("merge grid out of range"); return XATTN_E_INVALID; }
  const dim3 grid((unsigned)blocks, (unsigned)(a->batch < 65535 ? a->batch : 65535));
  ProfileScope prof(kProfGate, s);
  if (a->dtype == XATTN_DTYPE_BF16)
    merge_gradients_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)a->a, (const __nv_bfloat16*)a->b, (const __nv_bfloat16*)a->tail,
                                                            (__nv_bfloat16*)a->out, per_batch, tail_start, tail_per_batch, (int)a->batch);
  else
    merge_gradients_kernel<__half><<<grid, 256, 0, s>>>((const __half*)a->a, (const __half*)a->b, (const __half*)a->tail, (__half*)a->out,
                                                     per_batch, tail_start, tail_per_batch, (int)a->batch);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("merge launch: %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  return XATTN_OK;
}

int zero_constant_entry(const XattnConstantKeyArgs* a, cudaStream_t s) {
  if (!a || !a->dq || !a->k || !a->plan || !a->workspace) { set_error("null arguments"); return XATTN_E_INVALID; }
  if (a->dtype != XATTN_DTYPE_F16 && a->dtype != XATTN_DTYPE_BF16) { set_error("dtype must be fp16 or bf16"); return XATTN_E_INVALID; }
  const int B = (int)a->batch, Lq = (int)a->q_len, Lk = (int)a->k_len, Hq = (int)a->q_heads, Hkv = (int)a->kv_heads, D = (int)a->qk_dim;
  if (B <= 0 || Lq <= 0 || Lk <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || D % 8 || D > 256) { set_error("bad sizes"); return XATTN_E_INVALID; }
  const PlanLayout pl(B, Lq, Lk);
  ProfileScope prof(kProfRepair, s);
  int* flags = a->workspace;
  {
    const long long warps = (long long)B * Hkv * Lk;
    const unsigned blocks = (unsigned)((warps * 32 + 255) / 256);
    if (a->dtype == XATTN_DTYPE_BF16)
      key_change_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)a->k, a->k_strides[0], a->k_strides[1], a->k_strides[2], B, Lk, Hkv, D, flags);
    else
      key_change_kernel<__half><<<blocks, 256, 0, s>>>((const __half*)a->k, a->k_strides[0], a->k_strides[1], a->k_strides[2], B, Lk, Hkv, D, flags);
  }
  row_cumsum_kernel<<<B * Hkv, 256, 0, s>>>(flags, Lk);
  {
    const long long warps = (long long)B * Lq * Hq;
    const unsigned blocks = (unsigned)((warps * 32 + 255) / 256);
    if (a->dtype == XATTN_DTYPE_BF16)
      zero_constant_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((__nv_bfloat16*)a->dq, a->plan + pl.off_lo, a->plan + pl.off_hi, flags, B, Lq, Lk, Hq, Hkv, D);
    else
      zero_constant_rows_kernel<__half><<<blocks, 256, 0, s>>>((__half*)a->dq, a->plan + pl.off_lo, a->plan + pl.off_hi, flags, B, Lq, Lk, Hq, Hkv, D);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("constant-key launch: %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  return XATTN_OK;
}

// ---------------------------------------------------------------------------
// Ring attention: fold one K/V block's normalised partial output into the running result.
//   new = log(exp(lse_acc) + exp(lse_part)),  y_acc = y_acc exp(lse_acc - new) + y_part exp(lse_part - new)
// One warp per (batch row, query row, head), in place; a row neither side has a key for keeps
// y = 0 and lse = -inf.  HBM-bound: reads both partial results once, writes one.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128) merge_outputs_kernel(float* __restrict__ y_acc, float* __restrict__ lse_acc,
                                                            const float* __restrict__ y_part,
                                                            const float* __restrict__ lse_part, long long units,
                                                            int rows, int heads, int v_dim, int acc_rows,
                                                            int row_offset) {
  const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (unit >= units) return;
  const int lane = threadIdx.x & 31;
  const int h = (int)(unit % heads);
  const long long br = unit / heads;
  const int i = (int)(br % rows);
  const long long b = br / rows;
  const size_t l_acc = ((size_t)b * heads + h) * acc_rows + row_offset + i;
  const float l0 = lse_acc[l_acc], l1 = lse_part[((size_t)b * heads + h) * rows + i];
  const float mx = fmaxf(l0, l1);
  float w0 = 0.f, w1 = 0.f, merged = -INFINITY;
  if (mx != -INFINITY) {
    const float e0 = expf(l0 - mx), e1 = expf(l1 - mx);
    const float sum = e0 + e1;
    merged = mx + logf(sum);
    w0 = e0 / sum;
    w1 = e1 / sum;
  }
  float4* acc = reinterpret_cast<float4*>(y_acc + (((size_t)b * acc_rows + row_offset + i) * heads + h) * v_dim);
  const float4* part = reinterpret_cast<const float4*>(y_part + (((size_t)b * rows + i) * heads + h) * v_dim);
  for (int c = lane; c < v_dim / 4; c += 32) {
    const float4 a = acc[c], p = part[c];
    acc[c] = make_float4(a.x * w0 + p.x * w1, a.y * w0 + p.y * w1, a.z * w0 + p.z * w1, a.w * w0 + p.w * w1);
  }
  if (lane == 0) lse_acc[l_acc] = merged;
}

int merge_outputs_entry(const XattnMergeOutputsArgs* a, cudaStream_t s) {
  if (!a || !a->y_acc || !a->lse_acc || !a->y_part || !a->lse_part) { set_error("null merge arguments"); return XATTN_E_INVALID; }
  if (a->batch <= 0 || a->rows <= 0 || a->heads <= 0 || a->v_dim <= 0 || a->v_dim % 4 || a->row_offset < 0 ||
      a->row_offset + a->rows > a->acc_rows) { set_error("bad merge sizes"); return XATTN_E_INVALID; }
  for (const void* ptr : {(const void*)a->y_acc, (const void*)a->y_part}) {
    if (reinterpret_cast<uintptr_t>(ptr) & 15) { set_error("partial outputs must be 16-byte aligned"); return XATTN_E_INVALID; }
  }
  const long long units = (long long)a->batch * a->rows * a->heads;
  const long long blocks = (units + 3) / 4;
  if (blocks > 0x7fffffffLL) { set_error("merge grid out of range"); return XATTN_E_INVALID; }
  merge_outputs_kernel<<<(unsigned)blocks, 128, 0, s>>>(a->y_acc, a->lse_acc, a->y_part, a->lse_part, units, (int)a->rows,
                                                        (int)a->heads, (int)a->v_dim, (int)a->acc_rows, (int)a->row_offset);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("merge launch: %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  return XATTN_OK;
}

// ---------------------------------------------------------------------------
// Self-test of the bounded wait: one CTA waits on a barrier that nothing will ever complete, with a
// short time limit, and must come back with (site << 8) | kStatusWaitTimeout in the status word
// instead of hanging.  This is the path every tensor kernel takes when a bulk copy or a product never
// signals; nothing faults and the context stays usable.
// ---------------------------------------------------------------------------
constexpr int kProbeSite = 99;

__global__ void __launch_bounds__(64) wait_timeout_probe_kernel(int* status, unsigned long long budget_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  WaitCtx ctx{&abort_flag, status, budget_ns};
  WaitCtx patient{&abort_flag, status, 8 * budget_ns};
  if (threadIdx.x == 0) mbar_wait(ctx, &bar, 0, kProbeSite);                // runs out: sets the flag and the status
  else if (threadIdx.x == 32) mbar_wait(patient, &bar, 0, kProbeSite + 1);   // leaves when it sees the flag
  __syncthreads();
}

int wait_timeout_probe_entry(int32_t* status, int64_t budget_us, cudaStream_t s) {
  if (!status) { set_error("null status word"); return XATTN_E_INVALID; }
  if (budget_us < 1 || budget_us > 100000) { set_error("the probe's time limit must be 1 .. 100000 microseconds"); return XATTN_E_INVALID; }
  wait_timeout_probe_kernel<<<1, 64, 0, s>>>(status, (unsigned long long)budget_us * 1000ull);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("probe launch: %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  return XATTN_OK;
}

}  // namespace xb
