// HBM-bound helpers around the attention kernels.
//
//   SoftDelta gate:   y = read - sigmoid(g) * neg_read                    (forward)
//                     read = y + sigmoid(g) * neg_read, d neg_read, dg     (backward, one pass)
//     restated from csrc/softdelta/gate.cu:25-27 (sigmoid in FP32), :76-132 (forward),
//     :228 (backward) and csrc/softdelta/preprocess.cu:98-103 (query reads recovered from y).
//   Constant-key rows: dQ of a row whose visible keys are all the same vector is exactly zero
//     (csrc/attention/precision/constant_keys.cu: key-equality runs, then zero those rows).
//
// One warp per (batch, token, KV head); each lane owns 8 consecutive channels per 256-channel
// slab, so every access is a 16-byte vector (or two for FP32).
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
// group of Dg = V / C consecutive channels (C = 1: one gate per head)
template <typename T, bool NEG_F32>
__global__ void __launch_bounds__(256) gate_fwd_kernel(const T* __restrict__ read, const void* __restrict__ neg_,
                                                       const T* __restrict__ g, T* __restrict__ y, long long rows,
                                                       int H, int Hkv, int V, int C, int Dg) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= rows * Hkv) return;
  const long long row = w / Hkv;
  const int kv = (int)(w - row * Hkv);
  const int G = H / Hkv;
  for (int c = lane * 8; c < V; c += 256) {
    float n[8];
    if (NEG_F32) load8_f32(reinterpret_cast<const float*>(neg_) + (row * Hkv + kv) * V + c, n);
    else load8<T>(reinterpret_cast<const T*>(neg_) + (row * Hkv + kv) * V + c, n);
    for (int r = 0; r < G; ++r) {
      const int h = kv * G + r;
      const T* gh = g + (row * H + h) * C;
      float x[8];
      load8<T>(read + (row * H + h) * V + c, x);
      if (C == 1) {
        const float gate = sigmoid_f32(to_f32<T>(gh[0]));
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = x[e] - gate * n[e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = x[e] - sigmoid_f32(to_f32<T>(gh[(c + e) / Dg])) * n[e];
      }
      store8<T>(y + (row * H + h) * V + c, x);
    }
  }
}

template <typename T, bool NEG_F32>
__global__ void __launch_bounds__(256) gate_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y,
                                                       const void* __restrict__ neg_, const T* __restrict__ g,
                                                       T* __restrict__ read, T* __restrict__ dneg, T* __restrict__ dg,
                                                       long long rows, int H, int Hkv, int V, int C, int Dg) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= rows * Hkv) return;
  const long long row = w / Hkv;
  const int kv = (int)(w - row * Hkv);
  const int G = H / Hkv;
  // V <= 256: one slab per lane
  const int c = lane * 8;
  const bool act = c < V;
  float n[8], dn[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { n[e] = 0.f; dn[e] = 0.f; }
  if (act) {
    if (NEG_F32) load8_f32(reinterpret_cast<const float*>(neg_) + (row * Hkv + kv) * V + c, n);
    else load8<T>(reinterpret_cast<const T*>(neg_) + (row * Hkv + kv) * V + c, n);
  }
  for (int r = 0; r < G; ++r) {
    const int h = kv * G + r;
    const T* gh = g + (row * H + h) * C;
    float d[8], yy[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) { d[e] = 0.f; yy[e] = 0.f; }
    if (act) {
      load8<T>(dy + (row * H + h) * V + c, d);
      load8<T>(y + (row * H + h) * V + c, yy);
    }
    if (C == 1) {
      const float gate = sigmoid_f32(to_f32<T>(gh[0]));
      float dot = 0.f;
      if (act) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          dn[e] -= gate * d[e];
          dot += d[e] * n[e];
          yy[e] += gate * n[e];
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      if (lane == 0) dg[row * H + h] = from_f32<T>(-dot * gate * (1.f - gate));
    } else {
      if (act) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float gate = sigmoid_f32(to_f32<T>(gh[(c + e) / Dg]));
          dn[e] -= gate * d[e];
          yy[e] += gate * n[e];
        }
      }
      // one gate gradient per value group: the group's share of <dy, neg_read>
      for (int j = 0; j < C; ++j) {
        float dot = 0.f;
        if (act) {
#pragma unroll
          for (int e = 0; e < 8; ++e) dot += ((c + e) / Dg == j) ? d[e] * n[e] : 0.f;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (lane == 0) {
          const float gate = sigmoid_f32(to_f32<T>(gh[j]));
          dg[(row * H + h) * C + j] = from_f32<T>(-dot * gate * (1.f - gate));
        }
      }
    }
    if (act) store8<T>(read + (row * H + h) * V + c, yy);
  }
  if (act) store8<T>(dneg + (row * Hkv + kv) * V + c, dn);
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

template <typename T>
static void launch_gate_fwd(const XattnGateArgs* a, cudaStream_t s) {
  const int groups = a->value_groups > 1 ? (int)a->value_groups : 1;
  const long long warps = a->rows * a->kv_heads;
  const unsigned blocks = (unsigned)((warps * 32 + 255) / 256);
  if (a->neg_is_f32)
    gate_fwd_kernel<T, true><<<blocks, 256, 0, s>>>((const T*)a->read, a->neg_read, (const T*)a->g, (T*)a->y, a->rows, (int)a->q_heads, (int)a->kv_heads, (int)a->v_dim, groups, (int)a->v_dim / groups);
  else
    gate_fwd_kernel<T, false><<<blocks, 256, 0, s>>>((const T*)a->read, a->neg_read, (const T*)a->g, (T*)a->y, a->rows, (int)a->q_heads, (int)a->kv_heads, (int)a->v_dim, groups, (int)a->v_dim / groups);
}
template <typename T>
static void launch_gate_bwd(const XattnGateArgs* a, cudaStream_t s) {
  const int groups = a->value_groups > 1 ? (int)a->value_groups : 1;
  const long long warps = a->rows * a->kv_heads;
  const unsigned blocks = (unsigned)((warps * 32 + 255) / 256);
  if (a->neg_is_f32)
    gate_bwd_kernel<T, true><<<blocks, 256, 0, s>>>((const T*)a->dy, (const T*)a->y, a->neg_read, (const T*)a->g, (T*)a->read, (T*)a->dneg_read, (T*)a->dg, a->rows, (int)a->q_heads, (int)a->kv_heads, (int)a->v_dim, groups, (int)a->v_dim / groups);
  else
    gate_bwd_kernel<T, false><<<blocks, 256, 0, s>>>((const T*)a->dy, (const T*)a->y, a->neg_read, (const T*)a->g, (T*)a->read, (T*)a->dneg_read, (T*)a->dg, a->rows, (int)a->q_heads, (int)a->kv_heads, (int)a->v_dim, groups, (int)a->v_dim / groups);
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

}  // namespace xb
