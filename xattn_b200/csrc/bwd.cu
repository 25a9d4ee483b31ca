// Backward attention for sm_100a: three kernels, all reductions in a fixed
// order (bitwise repeatable; nothing is accumulated with atomics).
//
//   bwd_pre_kernel   -delta = -rowsum(dy * y), -lse2 = -lse * log2(e)   (HBM-bound)
//   bwd_dq_kernel    query-stationary:  S = Q K^T, dP = dO V^T,
//                    dS = P * (dP - delta),  dQ += dS K                 (tensor-bound)
//   bwd_dkv_kernel   key-stationary, transposed:  S^T = K Q^T, dP^T = V dO^T,
//                    dV += P^T dO,  dK += dS^T Q, looping over the query heads
//                    of the KV head so dK / dV are written once         (tensor-bound)
//
// Arithmetic restated from the reference backward: P = exp2(S*c - lse*log2e)
// from the saved lse, dS = P * (dP - rowsum(dO*O)), P and dS rounded to the
// input dtype before the dV / dK / dQ products, dK and dQ scaled by the softmax
// scale at the end (csrc/attention/hopper/mainloop_bwd_sm90_tma_gmma_ws.hpp:1725-2149,
// :1877-1900, :2247,2302; hopper/bwd_preprocess_kernel.h:165-297;
// hopper/bwd_postprocess_kernel.h:273-288).  Where the reference reduces dQ
// across key tiles with global atomics or semaphores (hopper/mainloop_bwd...:2067-2103,
// :1261-1324), dQ here has its own query-stationary kernel.
#include "common.cuh"

// of every four pairs of exponentials, how many run on the FMA pipe instead of the special-function
// unit: dK / dV kernel (no gain measured there) and dQ kernel
#ifndef XB_DKV_FMA_PAIRS
#define XB_DKV_FMA_PAIRS 0
#endif
#ifndef XB_DQ_FMA_PAIRS
#define XB_DQ_FMA_PAIRS 1
#endif

namespace xb {

struct BwdParams {
  int B, Lq, Lk, Hq, Hkv, D, V;
  int nQT, nKT;
  float scale;
  const int* row_lo;
  const int* row_hi;
  const TileInfo* q_tiles;
  const KeyTileInfo* k_tiles;
  const int* k_order;         // key tiles of all batch rows, most work first
  const void* q;              // for direct loads in the dQ kernel
  int64_t q_sb, q_sl, q_sh;   // element strides of q
  int LqPad;                  // q_len rounded up to whole 128-row tiles: row stride of nlse2 / ndelta
  const float* nlse2;         // [B][Hq][LqPad]  -lse * log2e; -inf for rows without keys and padding
  const float* ndelta;        // [B][Hq][LqPad]  -rowsum(dy * y); 0 in the padding
  const void* row_terms;      // [B][Hq][LqPad][16] bf16: the same numbers as extra GEMM columns
  // high-precision backward only
  const int* anchor;          // [B][Hq][Lq]  key with the row's largest logit (-1: no visible key)
  const float* ndpa;          // [B][Hq][LqPad]  -dP at the anchor key
  float* ndelta_out;          // the statistics kernel writes ndelta and row_terms
  void* row_terms_out;
  const float* grad_unscale;  // optional device scalar multiplied into dq, dk and dv on the way out
  void* dq;                   // [B][Lq][Hq][D]
  void* dk;                   // [B][Lk][Hkv][D]
  void* dv;                   // [B][Lk][Hkv][V]
  int* status;
};

// ---------------------------------------------------------------------------
// preprocess
// ---------------------------------------------------------------------------
// The dK / dV kernel works on S^T and dP^T, where the per-query numbers lse and delta belong to
// COLUMNS: every thread would need all of them for every step, and filling registers with them
// costs more load bandwidth than the tensor products leave.  So they ride along in the products
// instead.  One extra k-step of 16 columns is appended to Q and dO (this 32-byte row per query)
// and to K and V (constant rows of ones and zeros):
//   S^T + (-lse / scale)  =  [K | 1 1 1 0 ..] [Q | t0 t1 t2 0 ..]^T          t0 + t1 + t2 = -lse / scale
//   dP^T + d + e          =  [V | 0 0 0 1 1 1 1 1 0 ..] [dO | 0 0 0 d0 d1 d2 e0 e1 0 ..]^T
// with each number split into bf16 terms (24 significant bits for t and d, 16 for e) and FP32
// accumulation.  Low precision: d = -delta, e = 0.  High precision: d = -dP at the row's anchor
// key, e = -Delta (the centred row statistic).  All eight terms sit in the first 16 bytes of the
// row.  Rows without keys and padding rows get a huge negative first term, so that P = 0 for them.
__device__ __forceinline__ void write_row_terms(uint4* dst, float t, float d, float e) {
  if (!(t > -1e30f)) t = -1.2676506e30f;          // -2^100, exact in bf16
  const __nv_bfloat16 t0 = __float2bfloat16_rn(t);
  const float tr = t - __bfloat162float(t0);
  const __nv_bfloat16 t1 = __float2bfloat16_rn(tr);
  const __nv_bfloat16 t2 = __float2bfloat16_rn(tr - __bfloat162float(t1));
  const __nv_bfloat16 d0 = __float2bfloat16_rn(d);
  const float dr = d - __bfloat162float(d0);
  const __nv_bfloat16 d1 = __float2bfloat16_rn(dr);
  const __nv_bfloat16 d2 = __float2bfloat16_rn(dr - __bfloat162float(d1));
  const __nv_bfloat16 e0 = __float2bfloat16_rn(e);
  const __nv_bfloat16 e1 = __float2bfloat16_rn(e - __bfloat162float(e0));
  auto bits = [](__nv_bfloat16 x) -> uint32_t { return (uint32_t)__bfloat16_as_ushort(x); };
  dst[0] = make_uint4(bits(t0) | (bits(t1) << 16), bits(t2) | (bits(d0) << 16), bits(d1) | (bits(d2) << 16),
                      bits(e0) | (bits(e1) << 16));
  dst[1] = make_uint4(0u, 0u, 0u, 0u);
}

// A group of 8, 16 or 32 lanes (one 16-byte chunk of the row each) takes a (row, head) of one batch row;
// a warp works on kPrePasses * 32 / group consecutive ones with all their loads (lse included) issued
// before the first use.  Afterwards lane p of a group writes the results of pass p, so the passes'
// epilogues run side by side.  blockIdx.y is the batch row.
constexpr int kPrePasses = 4;
constexpr int kPreThreads = 128;
constexpr int kPreIters = 4;

template <typename T>
__global__ void __launch_bounds__(kPreThreads) bwd_pre_kernel(const T* __restrict__ dy, const T* __restrict__ y,
                                                      const float* __restrict__ lse, int B, int Lq, int Hq, int V,
                                                      int64_t dy_sb, int64_t dy_sl, int64_t dy_sh, int64_t y_sb,
                                                      int64_t y_sl, int64_t y_sh, int LqPad, float scale,
                                                      float* __restrict__ ndelta, float* __restrict__ nlse2,
                                                      uint4* __restrict__ row_terms) {
  const int chunks = V >> 3;
  const int group = chunks <= 8 ? 8 : (chunks <= 16 ? 16 : 32);
  const int per_pass = 32 / group;
  const int lane = threadIdx.x & 31;
  const int sub = lane / group, ch = lane % group;
  // a block makes kPreIters rounds (fewer, longer-lived blocks measured 10 % faster); a round past the
  // end decodes to a row >= LqPad and does nothing
  for (int it = 0; it < kPreIters; ++it) {
  const uint32_t first = ((blockIdx.x * kPreIters + it) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * (uint32_t)(per_pass * kPrePasses) + sub;
  const int h0 = (int)(first % (uint32_t)Hq), i0 = (int)(first / (uint32_t)Hq);
  for (int b = blockIdx.y; b < B; b += gridDim.y) {
  const T* dy_b = dy + b * dy_sb;
  const T* y_b = y + b * y_sb;
  const float* lse_b = lse + (size_t)b * Hq * Lq;
  uint4 a[kPrePasses], o[kPrePasses];
  float l_mine = 0.f;                   // lane p of the group: lse of pass p
  int h_mine = 0, i_mine = LqPad;
#pragma unroll
  for (int ps = 0; ps < kPrePasses; ++ps) {
    int h = h0 + ps * per_pass, i = i0;
    while (h >= Hq) { h -= Hq; ++i; }
    a[ps] = make_uint4(0, 0, 0, 0);
    o[ps] = make_uint4(0, 0, 0, 0);
    if (i < Lq && ch < chunks) {
      a[ps] = __ldg(reinterpret_cast<const uint4*>(dy_b + i * dy_sl + h * dy_sh + ch * 8));
      o[ps] = __ldg(reinterpret_cast<const uint4*>(y_b + i * y_sl + h * y_sh + ch * 8));
    }
    if (ch == ps) {
      h_mine = h; i_mine = i;
      if (i < Lq) l_mine = __ldg(lse_b + (size_t)h * Lq + i);
    }
  }
  float acc_mine = 0.f;
#pragma unroll
  for (int ps = 0; ps < kPrePasses; ++ps) {
    const uint32_t aw[4] = {a[ps].x, a[ps].y, a[ps].z, a[ps].w};
    const uint32_t ow[4] = {o[ps].x, o[ps].y, o[ps].z, o[ps].w};
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 fa = Pack2<T>::unpack(aw[k]);
      const float2 fo = Pack2<T>::unpack(ow[k]);
      acc = fmaf(fa.x, fo.x, acc);
      acc = fmaf(fa.y, fo.y, acc);
    }
    for (int off = group >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (ch == ps) acc_mine = acc;
  }
  if (ch < kPrePasses && i_mine < LqPad) {
    const size_t idx = ((size_t)b * Hq + h_mine) * LqPad + i_mine;
    if (i_mine >= Lq) {
      // padding up to whole tiles: rows that contribute nothing
      ndelta[idx] = 0.f;
      nlse2[idx] = -INFINITY;
      write_row_terms(row_terms + 2 * idx, -INFINITY, 0.f, 0.f);
    } else {
      const float l = l_mine;
      ndelta[idx] = -acc_mine;
      nlse2[idx] = (l == -INFINITY) ? -INFINITY : -l * 1.4426950408889634f;
      write_row_terms(row_terms + 2 * idx, (l == -INFINITY) ? -INFINITY : -l / scale, -acc_mine, 0.f);
    }
  }
  }
  }
}


// High-precision preprocess.  The low-precision delta = rowsum(dy * y) inherits the rounding of y to
// 16 bits, which is fatal when one key holds nearly all of a row's probability and dO V^T is huge
// (tests/test_high_precision.py:278-310 of the reference).  The reference's remedy is to centre dP on
// the row's anchor key, the one with the largest logit (csrc/attention/precision/row_statistics_sm90.cuh:144-186):
// dS_ij = P_ij ((dP_ij - dP_ia) - Delta_i) with Delta_i = sum_j P_ij (dP_ij - dP_ia), which is exact
// on the anchor and needs no cancellation of large numbers.  This kernel computes dP_ia = dO_i . V_a
// with one 16-lane group per (row, head); Delta follows in the statistics pass of the dQ kernel.
template <typename T>
__global__ void __launch_bounds__(128) bwd_pre_hp_kernel(const T* __restrict__ dy, const T* __restrict__ v,
                                                         const float* __restrict__ lse, const int* __restrict__ anchor,
                                                         int B, int Lq, int Lk, int Hq, int Hkv, int V,
                                                         int64_t dy_sb, int64_t dy_sl, int64_t dy_sh, int64_t v_sb,
                                                         int64_t v_sl, int64_t v_sh, int LqPad,
                                                         float* __restrict__ ndpa, float* __restrict__ nlse2) {
  const int sub = threadIdx.x & 15;
  const long long units = (long long)B * Hq * LqPad;
  const long long unit = (long long)blockIdx.x * 8 + (threadIdx.x >> 4);
  const bool in_range = unit < units;
  const int i = in_range ? (int)(unit % LqPad) : 0;
  const long long bh = in_range ? unit / LqPad : 0;
  const int h = (int)(bh % Hq), b = (int)(bh / Hq);
  const bool live = in_range && i < Lq;
  int a = -1;
  float l = -INFINITY;
  if (live) {
    a = anchor[((size_t)b * Hq + h) * Lq + i];
    l = lse[((size_t)b * Hq + h) * Lq + i];
  }
  float acc = 0.f;
  if (live && a >= 0 && a < Lk) {
    const T* dy_row = dy + b * dy_sb + i * dy_sl + h * dy_sh;
    const T* v_row = v + b * v_sb + (int64_t)a * v_sl + (h / (Hq / Hkv)) * v_sh;
    for (int c = sub * 8; c < V; c += 128) {
      const uint4 x = __ldg(reinterpret_cast<const uint4*>(dy_row + c));
      const uint4 w = __ldg(reinterpret_cast<const uint4*>(v_row + c));
      const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 fa = Pack2<T>::unpack(xw[k]);
        const float2 fb = Pack2<T>::unpack(ww[k]);
        acc = fmaf(fa.x, fb.x, acc);
        acc = fmaf(fa.y, fb.y, acc);
      }
    }
  }
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (in_range && sub == 0) {
    ndpa[unit] = -acc;
    nlse2[unit] = (l == -INFINITY) ? -INFINITY : -l * 1.4426950408889634f;
  }
}


// ---------------------------------------------------------------------------
// dQ kernel
// ---------------------------------------------------------------------------
// One CTA owns 128 query rows of one head and walks the key tiles they see:
//   S = Q K^T, dP = dO V^T  ->  P = exp2(S c - lse2), dS = P (dP - delta)  ->  dQ += dS K.
// Q, the A operand of S for the whole life of the CTA, is staged in TMEM (packed); dO stays in
// shared memory.
// HD <= 128: key tiles of BN = 128.  TMEM: Q 0, dS 64 (packed), S 128, dP 256, dQ 384.
// HD  = 256: BN = 64; no room for dS, which is written over dP.  TMEM: Q 0 (128 columns), S 128,
//            dP 192, dQ 256.
// S and dP are handed to the element-wise warpgroups separately, and the three products have an
// issuing thread each: S of the next key tile is issued as soon as this
// one's S sits in registers, dP likewise (HD = 256: once dQ has read the dS lying over it), and dQ
// as soon as dS is in TMEM.
template <int HD, int BN>
struct DqSmem {
  static constexpr int kDoBytes = kBlockM * HD * 2;
  static constexpr int kKvBytes = BN * HD * 2;
  // K is held from S of its key tile until dQ of the same tile, V only for dP
#ifndef XB_DQ_KSTAGES
#define XB_DQ_KSTAGES 3
#endif
  static constexpr int kKStages = HD <= 128 ? XB_DQ_KSTAGES : 2;
  alignas(1024) uint8_t d_o[kDoBytes];
  alignas(1024) uint8_t k[kKStages][kKvBytes];
  alignas(1024) uint8_t v[2][kKvBytes];
  uint64_t do_full, q_ready;
  uint64_t k_full[kKStages], k_empty[kKStages], v_full[2], v_empty[2];
  uint64_t s_full, s_free, dp_full, dp_free, ds_full, dq_done, dq_staged;
  uint32_t tmem_base;
  int abort_flag;
  float red[kBlockM];          // statistics pass: the second column half's partial sums
};

// MODE of the dQ kernel.  kDqPlain: the low-precision backward.  kDqStats / kDqHigh: the two passes of the
// high-precision backward (restating csrc/attention/precision/row_statistics_sm90.cuh:39-188 and the
// high-precision branch of hopper/mainloop_bwd_sm90_tma_gmma_ws.hpp:1811-1868 on this kernel's
// structure).  Both compute P as the square of root = exp2((S c - lse2) / 2), so that a probability
// below the smallest normal FP32 number still multiplies a huge dP correctly (root * (root * x)), and
// centre dP on the row's anchor key, where the centred value is exactly zero.
//   kDqStats  no dQ product: Delta_i = sum_j P_ij (dP_ij - dP_ia), written with the row's extra GEMM
//             columns for the dK / dV kernel
//   kDqHigh   dS_ij = P_ij ((dP_ij - dP_ia) - Delta_i), dQ += dS K
enum { kDqPlain = 0, kDqStats = 1, kDqHigh = 2 };

// warps 0-3 / 4-7: element-wise warpgroups (thread = query row; first / second half of the key-tile columns)
// warps 8, 11, 10: issuers of S, dP and dQ (an issuing thread stalls while its products run, so each
// product has its own and none holds another back), warp 9: TMA producer + TMEM owner
template <typename T, int HD, int BN, int MODE>
__global__ void __launch_bounds__(384, 1)
bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_do, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_dq, const BwdParams p) {
  using Smem = DqSmem<HD, BN>;
  constexpr bool kHigh = MODE != kDqPlain, kStats = MODE == kDqStats;
  // kDqHigh feeds dS to the dQ product as two 16-bit parts, hi + lo (the rounding residue of hi), so the
  // operand carries 16 significant bits instead of 8 (bf16) / 11 (fp16): the split of the reference's
  // high-precision mainloop (hopper/mainloop_bwd_sm90_tma_gmma_ws.hpp:1811-1868).  Both parts lie over
  // the dP columns they came from (hi in the first half of each 32-column chunk, lo in the second).
  constexpr bool kSplit = MODE == kDqHigh;
  constexpr bool kDsOverDp = (HD > 128 || kSplit) && !kStats;   // dS is written over dP
  constexpr int kKStages = Smem::kKStages;
  constexpr int kDoBox = kBlockM * 64 * 2;     // 64-column box of the 128-row dO tile
  constexpr int kKvBox = BN * 64 * 2;          // 64-column box of a BN-row K / V tile
  constexpr int CH = BN / 2;                   // key columns per element-wise thread
  constexpr uint32_t kTmemCols = 512;
  constexpr int kFormat = Pack2<T>::kFormat;
  // of every four pairs of exponentials, how many run on the FMA pipe
  constexpr int kFmaPairs = XB_DQ_FMA_PAIRS;
  // TMEM columns.  dS, packed: 16 columns per 32-column chunk of dP, side by side from cDS, or
  // (HD = 256) over the first 16 columns of the chunk itself.
  constexpr uint32_t cQ = 0, cDS = 64;
  constexpr uint32_t cS = 128, cDP = HD > 128 ? 192 : 256;
  constexpr uint32_t cDQ = HD > 128 ? 256 : 384;

  extern __shared__ uint8_t smem_raw[];
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const int G = p.Hq / p.Hkv;
  const int per_bk = p.nQT * G;
  const int bk = blockIdx.x / per_bk;
  const int rem = blockIdx.x - bk * per_bk;
  const int qt = p.nQT - 1 - rem / G;
  const int kvh = bk % p.Hkv;
  const int h = kvh * G + (rem % G);
  const int b = bk / p.Hkv;

  // This thread's half of its Q row (element-wise warps: thread = query row, hf = column half) is
  // requested from global memory before anything else: it goes to TMEM as the A operand of S = Q K^T,
  // every CTA starts with the chain  row load -> TMEM store -> first S product, and the set-up below
  // (barriers, TMEM allocation, the CTA-wide barrier) fits inside the load's latency.
  constexpr int kQRegs = HD / 4;              // packed 16-bit pairs per half row
  uint32_t q_pre[kQRegs];
  if (warp < 8) {
    const int hf = warp >> 2, row = qt * kBlockM + (tid & 127);
    const T* src = reinterpret_cast<const T*>(p.q) + b * p.q_sb + (row < p.Lq ? row : 0) * p.q_sl + h * p.q_sh;
#pragma unroll
    for (int c = 0; c < kQRegs; c += 4) {
      const int e = (hf * kQRegs + c) * 2;     // first element of this 16-byte chunk
      uint4 u = make_uint4(0, 0, 0, 0);
      if (row < p.Lq && e < p.D) u = *reinterpret_cast<const uint4*>(src + e);
      q_pre[c] = u.x; q_pre[c + 1] = u.y; q_pre[c + 2] = u.z; q_pre[c + 3] = u.w;
    }
  }

  if (warp == 9 && lane == 0) {
    // The dO tile needs nothing but the block index: its load starts before anything else, the
    // mask plan's tile summary included (its barrier is initialised here, by its first user).
    tma_prefetch_desc(&tm_do);
    mbar_init(&s.do_full, 1);
    fence_mbar_init();
    mbar_arrive_expect_tx(&s.do_full, ((p.V + 63) / 64) * kDoBox);
    for (int bx = 0; bx < (p.V + 63) / 64; ++bx)
      tma_load_4d(s.d_o + bx * kDoBox, &tm_do, &s.do_full, bx * 64, h, qt * kBlockM, b);
    tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_dq);
  }
  int n_lo = 0, n_hi = 0, full_lo = 0x7fffffff, full_hi = 0;
  {
    const TileInfo ti = p.q_tiles[(size_t)b * p.nQT + qt];
    if (ti.max_hi > ti.min_lo) {
      n_lo = ti.min_lo / BN;
      n_hi = (ti.max_hi + BN - 1) / BN;
      full_lo = ti.max_lo;
      full_hi = ti.min_hi;
    }
  }
  const int iters = n_hi - n_lo;
  // the first K and V tiles are requested as soon as the tile summary says which they are, before
  // the CTA's set-up barrier
  if (warp == 9 && lane == 0) {
    for (int i = 0; i < kKStages; ++i) mbar_init(&s.k_full[i], 1);
    for (int i = 0; i < 2; ++i) mbar_init(&s.v_full[i], 1);
    fence_mbar_init();
    if (iters > 0) {
      mbar_arrive_expect_tx(&s.k_full[0], ((p.D + 63) / 64) * kKvBox);
      for (int bx = 0; bx < (p.D + 63) / 64; ++bx)
        tma_load_4d(s.k[0] + bx * kKvBox, &tm_k, &s.k_full[0], bx * 64, kvh, n_lo * BN, b);
      mbar_arrive_expect_tx(&s.v_full[0], ((p.V + 63) / 64) * kKvBox);
      for (int bx = 0; bx < (p.V + 63) / 64; ++bx)
        tma_load_4d(s.v[0] + bx * kKvBox, &tm_v, &s.v_full[0], bx * 64, kvh, n_lo * BN, b);
    }
  }

  if (tid == 0) {
    s.abort_flag = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 2 : 0;
    mbar_init(&s.q_ready, 8);
    for (int i = 0; i < kKStages; ++i) mbar_init(&s.k_empty[i], 1);     // k_full, v_full: by the TMA thread, above
    for (int i = 0; i < 2; ++i) mbar_init(&s.v_empty[i], 1);
    mbar_init(&s.s_full, 1);
    mbar_init(&s.s_free, 8);
    mbar_init(&s.dp_full, 1);
    mbar_init(&s.dp_free, 8);
    mbar_init(&s.ds_full, 8);
    mbar_init(&s.dq_done, 1);
    mbar_init(&s.dq_staged, 8);
    fence_mbar_init();
  }
  if (warp == 9) { tmem_alloc(&s.tmem_base, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  WaitCtx ctx{&s.abort_flag, p.status, 2000000000ull};
  const bool dead = s.abort_flag != 0;

  const int nbox_qk = (p.D + 63) / 64, nbox_v = (p.V + 63) / 64;
  const int ksteps_qk = (p.D + 15) / 16, ksteps_v = (p.V + 15) / 16;
  const int d_pad = (p.D + 15) & ~15;

  // 384 threads start with 168 registers each; the element-wise warpgroups take most of the other
  // warps' share
  // registers move between warps of this CTA only: the gain must not exceed what the others give up
  static_assert(256 * (216 - 168) <= 128 * (168 - 72), "register budget");
  if (warp < 8) setmaxnreg_inc<216>(); else setmaxnreg_dec<72>();
  if (dead) {
  } else if (warp < 8) {
    const int hf = warp >> 2;                 // which half of the key-tile columns
    const int r = tid & 127;
    const int row = qt * kBlockM + r;
    const bool live = row < p.Lq;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    T* dq_row = reinterpret_cast<T*>(p.dq) + (((size_t)b * p.Lq + (live ? row : 0)) * p.Hq + h) * p.D;
    // statistics pass: what a row hands to the dK / dV kernel
    auto write_stats = [&](float delta) {
      const size_t idx = ((size_t)b * p.Hq + h) * p.LqPad + row;
      float nl2 = -INFINITY, npa = 0.f;
      if (live) { nl2 = p.nlse2[idx]; npa = p.ndpa[idx]; }
      p.ndelta_out[idx] = -delta;
      write_row_terms(reinterpret_cast<uint4*>(p.row_terms_out) + 2 * idx,
                      nl2 == -INFINITY ? -INFINITY : nl2 / (p.scale * 1.4426950408889634f), npa, -delta);
    };
    if (iters == 0) {
      if (kStats) {
        if (hf == 0) write_stats(0.f);
      } else if (live) {
        for (int c = hf * (HD / 2); c < (hf + 1) * (HD / 2) && c < p.D; c += 8)
          *reinterpret_cast<uint4*>(dq_row + c) = make_uint4(0, 0, 0, 0);
      }
    } else {
      // this thread's half of the Q row (requested at the top of the kernel) goes to TMEM: packed
      // pairs, row = lane
      {
        constexpr int kStep = kQRegs < 32 ? kQRegs : 32;
#pragma unroll
        for (int c0 = 0; c0 < kQRegs; c0 += kStep) {
          if (kStep == 32) tmem_st_x32(tmem + lane_off + cQ + hf * kQRegs + c0, q_pre + c0);
          else tmem_st_x16(tmem + lane_off + cQ + hf * kQRegs + c0, q_pre + c0);
        }
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive_warp(&s.q_ready);
      int lo = 0, hi = 0, anchor = -1;
      float nlse2 = -INFINITY, ndelta = 0.f, ndpa = 0.f;
      if (live) {
        lo = p.row_lo[(size_t)b * p.Lq + row];
        hi = p.row_hi[(size_t)b * p.Lq + row];
        nlse2 = p.nlse2[((size_t)b * p.Hq + h) * p.LqPad + row];
        if (!kStats) ndelta = p.ndelta[((size_t)b * p.Hq + h) * p.LqPad + row];
        if (kHigh) {
          ndpa = p.ndpa[((size_t)b * p.Hq + h) * p.LqPad + row];
          anchor = p.anchor[((size_t)b * p.Hq + h) * p.Lq + row];
        }
      }
      // high precision: the exponent is halved, P = root * root
      const float c_log2 = p.scale * 1.4426950408889634f * (kHigh ? 0.5f : 1.f);
      if (kHigh) nlse2 *= 0.5f;
      const float2 cc = make_float2(c_log2, c_log2), nl = make_float2(nlse2, nlse2);
      const float2 nd = make_float2(ndelta, ndelta), npa = make_float2(ndpa, ndpa);
      float2 stat_a = make_float2(0.f, 0.f), stat_b = make_float2(0.f, 0.f);
      bool ok = true;
      for (int i = 0; i < iters && ok; ++i) {
        const int col0 = (n_lo + i) * BN + hf * CH;
        // ---- P = exp2(S c - lse2), masked ----
        ok = mbar_wait(ctx, &s.s_full, i & 1, 50);
        if (!ok) break;
        tc_fence_after();
        float pv[CH];
#pragma unroll
        for (int c = 0; c < CH; c += 32) tmem_ld_x32(tmem + lane_off + cS + hf * CH + c, reinterpret_cast<uint32_t*>(pv) + c);
        tc_wait_ld();
        tc_fence_before();
        mbar_arrive_warp(&s.s_free);
        const bool tile_full = ((n_lo + i) * BN >= full_lo) && ((n_lo + i + 1) * BN <= full_hi);
        const int rl = lo - col0, rh = hi - col0;
#pragma unroll
        for (int c = 0; c < CH; c += 2) {
          // a share of the exponentials on the FMA pipe: the special-function unit bounds this loop
          const float2 x = fma2(make_float2(pv[c], pv[c + 1]), cc, nl);
          const float2 pr = (!kHigh && ((c >> 1) & 3) < kFmaPairs) ? ex2_pair_fma(x) : ex2_pair_sfu(x);
          pv[c] = pr.x; pv[c + 1] = pr.y;
        }
        if (!tile_full) {
#pragma unroll
          for (int c = 0; c < CH; ++c) pv[c] = (c >= rl && c < rh) ? pv[c] : 0.f;
        }
        // ---- dS = P (dP - delta) ----
        ok = mbar_wait(ctx, &s.dp_full, i & 1, 51);
        if (!ok) break;
        tc_fence_after();
        uint32_t pk[CH / 2];
        uint32_t pk_lo[kSplit ? CH / 2 : 1];
        const int ac = anchor - col0;         // the anchor's column in this thread's share, if any
#pragma unroll
        for (int c0 = 0; c0 < CH; c0 += 32) {
          float dpv[32];
          const uint32_t t_dp = tmem + lane_off + cDP + hf * CH + c0;
          tmem_ld_x32(t_dp, reinterpret_cast<uint32_t*>(dpv));
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            const float2 pr = make_float2(pv[c0 + c], pv[c0 + c + 1]);
            if (kHigh) {
              float2 cent = add2(make_float2(dpv[c], dpv[c + 1]), npa);
              cent.x = (c0 + c == ac) ? 0.f : cent.x;
              cent.y = (c0 + c + 1 == ac) ? 0.f : cent.y;
              if (kStats) {
                if (c & 2) stat_b = fma2(pr, mul2(pr, cent), stat_b);
                else stat_a = fma2(pr, mul2(pr, cent), stat_a);
              } else {
                const float2 ds = mul2(pr, mul2(pr, add2(cent, nd)));
                const uint32_t hi = Pack2<T>::pack(ds.x, ds.y);
                pk[(c0 + c) >> 1] = hi;
                if (kSplit) {
                  const float2 back = Pack2<T>::unpack(hi);
                  pk_lo[(c0 + c) >> 1] = Pack2<T>::pack(ds.x - back.x, ds.y - back.y);
                }
              }
            } else {
              const float2 ds = mul2(pr, add2(make_float2(dpv[c], dpv[c + 1]), nd));
              pk[(c0 + c) >> 1] = Pack2<T>::pack(ds.x, ds.y);
            }
          }
          if (kDsOverDp) tmem_st_x16(t_dp, pk + (c0 >> 1));
          if (kSplit) tmem_st_x16(t_dp + 16, pk_lo + (c0 >> 1));
        }
        if (kStats) {
          tc_fence_before();
          mbar_arrive_warp(&s.dp_free);        // dP has been read: the next one may be issued
          continue;
        }
        if (!kDsOverDp) {
          tc_fence_before();
          mbar_arrive_warp(&s.dp_free);        // dP sits in registers: the next one may be issued
          if (i > 0) {
            ok = mbar_wait(ctx, &s.dq_done, (i - 1) & 1, 53);   // dQ has read the previous dS
            if (!ok) break;
            tc_fence_after();
          }
#pragma unroll
          for (int c0 = 0; c0 < CH; c0 += 32) tmem_st_x16(tmem + lane_off + cDS + (hf * CH + c0) / 2, pk + (c0 >> 1));
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive_warp(&s.ds_full);
      }
      if (kStats) {
        // Delta = first half's sum + second half's sum, in that order
        const float part = (stat_a.x + stat_a.y) + (stat_b.x + stat_b.y);
        if (hf == 1) s.red[r] = part;
        mbar_arrive_warp(&s.dq_staged);
        if (ok && hf == 0) {
          ok = mbar_wait(ctx, &s.dq_staged, 0, 55);
          if (ok) write_stats(live ? part + s.red[r] : 0.f);
        }
      }
      if (ok && !kStats) ok = mbar_wait(ctx, &s.dq_done, (iters - 1) & 1, 52);
      if (ok && !kStats) {
        const float out_scale = p.scale * (p.grad_unscale ? __ldg(p.grad_unscale) : 1.f);
        tc_fence_after();
        // This warpgroup has columns [hf*HD/2, (hf+1)*HD/2) of dQ.  They leave through shared memory
        // (the dO tile's buffer: every dP product has run) and bulk tensor stores: coalesced, clipped
        // to the tensor by the hardware.  Layout: 64-column boxes of 128-byte rows in the 128-byte
        // swizzle (16-byte chunk c of row r sits at chunk c ^ (r & 7)).
#pragma unroll
        for (int c0 = 0; c0 < HD / 2; c0 += 32) {
          const int cbase = hf * (HD / 2) + c0;
          uint32_t o[32];
          tmem_ld_x32(tmem + lane_off + cDQ + cbase, o);
          tc_wait_ld();
          uint8_t* box = s.d_o + (cbase >> 6) * kDoBox + r * 128;
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 u;
            u.x = Pack2<T>::pack(__uint_as_float(o[c + 0]) * out_scale, __uint_as_float(o[c + 1]) * out_scale);
            u.y = Pack2<T>::pack(__uint_as_float(o[c + 2]) * out_scale, __uint_as_float(o[c + 3]) * out_scale);
            u.z = Pack2<T>::pack(__uint_as_float(o[c + 4]) * out_scale, __uint_as_float(o[c + 5]) * out_scale);
            u.w = Pack2<T>::pack(__uint_as_float(o[c + 6]) * out_scale, __uint_as_float(o[c + 7]) * out_scale);
            const int chunk = ((cbase & 63) + c) >> 3;
            *reinterpret_cast<uint4*>(box + ((chunk ^ (r & 7)) << 4)) = u;
          }
        }
        fence_proxy_async_smem();
        mbar_arrive_warp(&s.dq_staged);
        if (tid == 0) {
          ok = mbar_wait(ctx, &s.dq_staged, 0, 54);
          if (ok) {
            for (int bx = 0; bx < nbox_qk; ++bx) tma_store_4d(&tm_dq, s.d_o + bx * kDoBox, bx * 64, h, qt * kBlockM, b);
            tma_store_commit();
            tma_store_wait_read_all();
          }
        }
      }
    }
  } else if (warp == 8 && lane == 0 && iters > 0) {
    // ------------------------------ S issuer ------------------------------
    const uint32_t idesc_s = make_idesc(kBlockM, BN, kFormat, 0, 0);
    bool ok = mbar_wait(ctx, &s.q_ready, 0, 61);
    for (int i = 0; i < iters && ok; ++i) {
      const int ks = i % kKStages;
      ok = mbar_wait(ctx, &s.k_full[ks], (i / kKStages) & 1, 62);
      if (ok && i > 0) ok = mbar_wait(ctx, &s.s_free, (i - 1) & 1, 66);     // S of the tile before sits in registers
      if (!ok) break;
      tc_fence_after();
      const uint32_t ka = smem_u32(s.k[ks]);
      for (int js = 0; js < ksteps_qk; ++js) {
        umma_ts(tmem + cS, tmem + cQ + js * 8, make_smem_desc(ka + (js >> 2) * kKvBox + (js & 3) * 32, 16, 1024),
                idesc_s, js > 0);
      }
      umma_commit(&s.s_full);
      if (kStats) umma_commit(&s.k_empty[ks]);   // no dQ product holds the K tile any longer
    }
  } else if (warp == 11 && lane == 0 && iters > 0) {
    // ------------------------------ dP issuer ------------------------------
    const uint32_t idesc_s = make_idesc(kBlockM, BN, kFormat, 0, 0);
    bool ok = mbar_wait(ctx, &s.do_full, 0, 60);
    for (int i = 0; i < iters && ok; ++i) {
      const int vs = i & 1;
      ok = mbar_wait(ctx, &s.v_full[vs], (i >> 1) & 1, 63);
      // dP of the tile before sits in registers, or (dS lying over it) its dS has been read
      if (ok && i > 0) ok = mbar_wait(ctx, kDsOverDp ? &s.dq_done : &s.dp_free, (i - 1) & 1, 64);
      if (!ok) break;
      tc_fence_after();
      const uint32_t va = smem_u32(s.v[vs]), da = smem_u32(s.d_o);
      for (int js = 0; js < ksteps_v; ++js) {
        const uint64_t bv = make_smem_desc(va + (js >> 2) * kKvBox + (js & 3) * 32, 16, 1024);
        umma_ss(tmem + cDP, make_smem_desc(da + (js >> 2) * kDoBox + (js & 3) * 32, 16, 1024), bv, idesc_s, js > 0);
      }
      umma_commit(&s.dp_full);
      umma_commit(&s.v_empty[vs]);
    }
  } else if (warp == 10 && lane == 0 && iters > 0 && !kStats) {
    // ------------------------------ dQ issuer ------------------------------
    const uint32_t idesc_dq = make_idesc(kBlockM, d_pad, kFormat, 0, 1);
    bool ok = true;
    for (int i = 0; i < iters && ok; ++i) {
      const int ks = i % kKStages;
      ok = mbar_wait(ctx, &s.k_full[ks], (i / kKStages) & 1, 65);
      if (ok) ok = mbar_wait(ctx, &s.ds_full, i & 1, 67);
      if (!ok) break;
      tc_fence_after();
      const uint32_t ka = smem_u32(s.k[ks]);
#pragma unroll
      for (int js = 0; js < BN / 16; ++js) {
        // k-step js (16 keys) of dS: 8 packed columns
        const uint32_t a_col = kDsOverDp ? cDP + (js >> 1) * 32 + (js & 1) * 8 : cDS + js * 8;
        umma_ts(tmem + cDQ, tmem + a_col, make_smem_desc(ka + js * 2048, kKvBox, 1024), idesc_dq,
                (i > 0 || js > 0) ? 1u : 0u);
        if (kSplit) umma_ts(tmem + cDQ, tmem + a_col + 16, make_smem_desc(ka + js * 2048, kKvBox, 1024), idesc_dq, 1u);
      }
      umma_commit(&s.dq_done);
      umma_commit(&s.k_empty[ks]);
    }
  } else if (warp == 9 && lane == 0 && iters > 0) {
    // ------------------------------ TMA producer ------------------------------
    bool ok = true;
    for (int i = 1; i < iters && ok; ++i) {       // tile 0 was requested before the set-up barrier
      const int st = i & 1, ks = i % kKStages, n = n_lo + i;
      if (i >= kKStages) ok = mbar_wait(ctx, &s.k_empty[ks], ((i / kKStages) - 1) & 1, 70);
      if (!ok) break;
      mbar_arrive_expect_tx(&s.k_full[ks], nbox_qk * kKvBox);
      for (int bx = 0; bx < nbox_qk; ++bx)
        tma_load_4d(s.k[ks] + bx * kKvBox, &tm_k, &s.k_full[ks], bx * 64, kvh, n * BN, b);
      if (i >= 2) ok = mbar_wait(ctx, &s.v_empty[st], ((i >> 1) - 1) & 1, 71);
      if (!ok) break;
      mbar_arrive_expect_tx(&s.v_full[st], nbox_v * kKvBox);
      for (int bx = 0; bx < nbox_v; ++bx)
        tma_load_4d(s.v[st] + bx * kKvBox, &tm_v, &s.v_full[st], bx * 64, kvh, n * BN, b);
    }
  }

  if ((dead || iters == 0) && warp == 9 && lane == 0) {
    // the dO load was issued before anything was known: let it land (bounded)
    for (int i = 0; i < (1 << 20) && !mbar_try_wait(&s.do_full, 0); ++i) { }
    if (iters > 0) {
      for (int i = 0; i < (1 << 20) && !mbar_try_wait(&s.k_full[0], 0); ++i) { }
      for (int i = 0; i < (1 << 20) && !mbar_try_wait(&s.v_full[0], 0); ++i) { }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (s.abort_flag == 1) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { }
    __syncthreads();
  }
  if (warp == 9) { __syncwarp(); tmem_dealloc(tmem, kTmemCols); }
}


// ---------------------------------------------------------------------------
// dK / dV kernel
// ---------------------------------------------------------------------------
// MODE 0: dK and dV together (HD <= 128).  MODE 1: dV only, MODE 2: dK only (HD = 256, where
// the two accumulators do not fit TMEM side by side).  SM: query rows per inner step.
enum { kDkvBoth = 0, kDvOnly = 1, kDkOnly = 2 };

template <int HD, int MODE, int SM>
struct DkvSmem {
  static constexpr int kKvBytes = kBlockN * HD * 2;
  static constexpr int kQBytes = SM * HD * 2;
  static constexpr int kStages = (MODE == kDkvBoth && SM <= 64) ? 4 : 2;
  alignas(1024) uint8_t k[kKvBytes];
  alignas(1024) uint8_t v[MODE == kDvOnly ? 1024 : kKvBytes];
  alignas(1024) uint8_t q[kStages][kQBytes];
  alignas(1024) uint8_t d_o[kStages][kQBytes];
  // the extra k-step: per-query rows (-lse / scale and -delta in bf16 terms) of each stage, and the
  // constant rows of ones that pick them up on the key side (32-byte rows, 32-byte swizzle)
  alignas(1024) uint8_t terms[kStages][SM * 32];
  alignas(1024) uint8_t ones_s[kBlockN * 32];
  alignas(1024) uint8_t ones_dp[kBlockN * 32];
  uint64_t kv_full;
  uint64_t q_full[kStages], q_empty[kStages];
  // per TMEM buffer: S^T / dP^T written by their products, P^T / dS^T written by the warpgroups,
  // and the two regions read by dV / dK and free for the next products
  uint64_t s_full[2], dp_full[2], p_full[2][2], ds_full[2], s_free[2], dp_free[2];   // p_full: per chunk
  uint64_t all_done, out_staged[2];
  uint32_t tmem_base;
  int abort_flag;
  // one bit per query tile of [m_first, m_first + kTileCache): it sees this key tile at all / every
  // one of its rows sees all of it.  Built once, so that stepping to the next item reads no table.
  static constexpr int kTileCache = 768;
  uint32_t overlap_bits[kTileCache / 32], full_bits[kTileCache / 32];
};

// Enumerates the (query head of the group, SM-row query sub-tile) pairs a key
// tile has to visit, in the same order for every role.
template <int SM>
struct DkvIter {
  static constexpr int kParts = kBlockM / SM;
  int g, m, part;        // head within the group, 128-row query tile, which SM-row part
  int G, m_first, m_end, Lq, k0;
  const TileInfo* qt;        // global table of this batch row
  const uint32_t* bits;      // shared-memory bitmap over query tiles [m_first, m_first + cache_n)
  int cache_n;
  uint32_t word;             // the bitmap word last read, and which one it is
  int word_i;
  __device__ __forceinline__ bool tile_overlaps(int mm) {
    const int rel = mm - m_first;
    if (rel < cache_n) {
      if ((rel >> 5) != word_i) { word_i = rel >> 5; word = bits[word_i]; }
      return (word >> (rel & 31)) & 1u;
    }
    const TileInfo t = qt[mm];
    return t.max_hi > t.min_lo && t.min_lo < k0 + kBlockN && t.max_hi > k0;
  }
  __device__ __forceinline__ bool valid() const { return g < G; }
  __device__ __forceinline__ int row0() const { return m * kBlockM + part * SM; }
  // position on the first valid item at or after the current one
  __device__ __forceinline__ void settle() {
    while (g < G) {
      if (m >= m_end) { m = m_first; part = 0; ++g; continue; }
      if (part >= kParts) { part = 0; ++m; continue; }
      if (part == 0 && !tile_overlaps(m)) { ++m; continue; }
      if (row0() >= Lq) { part = 0; ++m; continue; }
      return;
    }
  }
  __device__ __forceinline__ void init(int G_, int m_first_, int m_end_, int Lq_, int k0_, const TileInfo* qt_,
                                       const uint32_t* bits_, int cache_n_) {
    G = G_; m_first = m_first_; m_end = m_end_; Lq = Lq_; k0 = k0_; qt = qt_;
    bits = bits_; cache_n = cache_n_; word = 0; word_i = -1;
    g = (m_end_ > m_first_) ? 0 : G_;
    m = m_first_; part = 0;
    settle();
  }
  __device__ __forceinline__ void next() { ++part; settle(); }
};

// warps 0-3 / 4-7: element-wise warpgroups, thread = (key row, half of the sub-tile's query columns).
// warp 8: issuer of S^T / dP^T, warp 10: issuer of dV / dK (an issuing thread stalls while its
// products run, so the two kinds get a thread each; a third thread, splitting S^T from dP^T, was
// measured slower), warp 9: TMA producer + TMEM owner, warp 11 idle.
// With two S^T / dP^T buffers (SM <= 64) sub-tiles alternate between them.  With one (SM = 128, the
// widest products: a tcgen05.mma costs about the same for 64 columns as for 128) the
// S^T -> P^T -> dV and dP^T -> dS^T -> dK chains of a step overlap each other and the next step's S^T.
template <typename T, int HD, int MODE, int SM, bool HP>
__global__ void __launch_bounds__(384, 1)
bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
               const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
               const __grid_constant__ CUtensorMap tm_terms, const __grid_constant__ CUtensorMap tm_dk,
               const __grid_constant__ CUtensorMap tm_dv, const BwdParams p) {
  using Smem = DkvSmem<HD, MODE, SM>;
  using Iter = DkvIter<SM>;
  constexpr int kStages = Smem::kStages;
  constexpr bool kWantDk = MODE != kDvOnly, kWantDv = MODE != kDkOnly;
  constexpr int kKvBox = kBlockN * 64 * 2;     // 64-column box of a 128-row tile
  constexpr int kQBox = SM * 64 * 2;           // 64-column box of an SM-row tile
  constexpr uint32_t kTmemCols = 512;
  constexpr int kFormat = Pack2<T>::kFormat;
  // TMEM columns: S^T buffer(s) from 0, dP^T buffer(s) from 128, accumulators from 256.  Two
  // buffers of each while they fit 128 columns (SM <= 64), else one.
  constexpr int kBufs = SM <= 64 ? 2 : 1;
  constexpr uint32_t cS = 0, cDP = 128;
  constexpr uint32_t cDK = 256, cDV = MODE == kDkvBoth ? 384 : 256;

  extern __shared__ uint8_t smem_raw[];
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const int G = p.Hq / p.Hkv;
  // key tiles with the most query tiles to visit first (the plan's order), their KV heads side by side
  const int kvh = blockIdx.x % p.Hkv;
  const int item = p.k_order[blockIdx.x / p.Hkv];
  const int b = item / p.nKT;
  const int n = item - b * p.nKT;
  const KeyTileInfo kti = p.k_tiles[(size_t)b * p.nKT + n];
  const TileInfo* qt_info = p.q_tiles + (size_t)b * p.nQT;

  if (tid == 0) {
    s.abort_flag = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 2 : 0;
    mbar_init(&s.kv_full, 1);
    for (int i = 0; i < kStages; ++i) { mbar_init(&s.q_full[i], 1); mbar_init(&s.q_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.s_full[i], 1); mbar_init(&s.dp_full[i], 1);
      mbar_init(&s.p_full[i][0], 8); mbar_init(&s.p_full[i][1], 8); mbar_init(&s.ds_full[i], 8);
      mbar_init(&s.s_free[i], 1); mbar_init(&s.dp_free[i], 1);
    }
    mbar_init(&s.all_done, 1);
    mbar_init(&s.out_staged[0], 4); mbar_init(&s.out_staged[1], 4);
    fence_mbar_init();
  }
  if (warp == 9) { tmem_alloc(&s.tmem_base, kTmemCols); tmem_relinquish(); }
  if (tid < kBlockN) {
    // key-side rows of the extra k-step: bf16 ones in columns 0-2 (S^T) or 3-7 (dP^T), the same
    // in both 16-byte halves of the row so that the swizzle cannot matter (the query-side rows
    // are zero in their second half)
    const uint4 os = make_uint4(0x3f803f80u, 0x00003f80u, 0u, 0u);
    const uint4 od = make_uint4(0u, 0x3f800000u, 0x3f803f80u, 0x3f803f80u);
    uint4* ps = reinterpret_cast<uint4*>(s.ones_s + tid * 32);
    uint4* pd = reinterpret_cast<uint4*>(s.ones_dp + tid * 32);
    ps[0] = os; ps[1] = os; pd[0] = od; pd[1] = od;
    fence_proxy_async_smem();
  }
  const int cache_n = min(max(kti.m_end - kti.m_first, 0), Smem::kTileCache);
  for (int base = 0; base < Smem::kTileCache; base += 384) {
    const int i = base + tid;
    bool sees = false, full = false;
    if (i < cache_n) {
      const TileInfo t = qt_info[kti.m_first + i];
      sees = t.max_hi > t.min_lo && t.min_lo < (n + 1) * kBlockN && t.max_hi > n * kBlockN;
      full = (n * kBlockN >= t.max_lo) && ((n + 1) * kBlockN <= t.min_hi);
    }
    const uint32_t ws = __ballot_sync(0xffffffffu, sees), wf = __ballot_sync(0xffffffffu, full);
    if (lane == 0) { s.overlap_bits[i >> 5] = ws; s.full_bits[i >> 5] = wf; }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  WaitCtx ctx{&s.abort_flag, p.status, 2000000000ull};
  const bool dead = s.abort_flag != 0;

  const int nbox_qk = (p.D + 63) / 64, nbox_v = (p.V + 63) / 64;
  const int ksteps_qk = (p.D + 15) / 16, ksteps_v = (p.V + 15) / 16;
  const int d_pad = (p.D + 15) & ~15, v_pad = (p.V + 15) & ~15;

  Iter it0;
  it0.init(G, kti.m_first, kti.m_end, p.Lq, n * kBlockN, qt_info, s.overlap_bits, cache_n);
  const bool any_work = it0.valid();

  // registers move between warps of this CTA only: the gain must not exceed what the others give up
  static_assert(256 * (216 - 168) <= 128 * (168 - 72), "register budget");
  if (warp < 8) setmaxnreg_inc<216>(); else setmaxnreg_dec<72>();
  if (dead) {
  } else if (warp < 8) {
    // ------------------------ element-wise warpgroups ------------------------
    constexpr int kHalf = SM / 2;             // query columns per warpgroup and step
    constexpr int kChunk = kHalf < 32 ? kHalf : 32;   // columns per TMEM load / store
    constexpr int kPerLane = kHalf / kChunk;  // lo / hi columns each lane looks after
    const int wg = warp >> 2;                 // which half of the columns
    const int wt = tid & 127;
    const int r = wt;                         // key row inside the tile
    const int key = n * kBlockN + r;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    // high precision: root = exp2(x / 2), P = root * root (see the dQ kernel's modes)
    const float c_log2 = p.scale * 1.4426950408889634f * (HP ? 0.5f : 1.f);
    const float2 cc = make_float2(c_log2, c_log2);
    bool ok = true;
    // Bit of the bitmap word: every row of query tile mm sees all of this key tile, no masking.
    // The word is fetched a step ahead and looked at only when needed.
    auto full_word = [&](int mm, int& bit) -> uint32_t {
      const int rel = mm - kti.m_first;
      if (rel < cache_n) { bit = rel & 31; return s.full_bits[rel >> 5]; }
      const TileInfo t = qt_info[mm];
      bit = 0;
      return ((n * kBlockN >= t.max_lo) && ((n + 1) * kBlockN <= t.min_hi)) ? 1u : 0u;
    };
    // lse and delta of the query columns arrive inside S^T and dP^T (the extra k-step), so the
    // only per-column numbers left are the visible-key bounds of a step that masks: lane c reads
    // lo / hi of columns c, c + 32, ... straight from global memory a step ahead, never touching
    // them in between (an instruction using a loaded value stalls the warp for the load's whole
    // latency), and hands them round by shuffle.
    auto bound_index = [&](const Iter& item, int j) -> size_t {
      const int qrow = item.row0() + wg * kHalf + j * kChunk + (lane & (kChunk - 1));
      return (size_t)b * p.Lq + (qrow < p.Lq ? qrow : p.Lq - 1);
    };
    int my_lo[kPerLane], my_hi[kPerLane];
    // High precision: on a query's anchor key the centred dP is exactly zero, so dS there is
    // P (0 - Delta).  Lane c fetches anchor and -Delta of its columns like the bounds above; a warp
    // looks at a column only when that column's anchor is one of the warp's own 32 keys.
    int my_anchor[kPerLane];
    float my_nd[kPerLane];
    auto fetch_anchor = [&](const Iter& item, int j) {
      const int qrow = item.row0() + wg * kHalf + j * kChunk + (lane & (kChunk - 1));
      const int qr = qrow < p.Lq ? qrow : p.Lq - 1;
      const size_t bh = (size_t)b * p.Hq + kvh * G + item.g;
      my_anchor[j] = qrow < p.Lq ? p.anchor[bh * p.Lq + qr] : -1;
      my_nd[j] = p.ndelta[bh * p.LqPad + qr];
    };
    Iter it = it0;
    uint32_t fw = 0;
    int fbit = 0;
    if (it.valid()) {
#pragma unroll
      for (int j = 0; j < kPerLane; ++j) {
        const size_t bi = bound_index(it, j);
        my_lo[j] = p.row_lo[bi]; my_hi[j] = p.row_hi[bi];
        if (HP) fetch_anchor(it, j);
      }
      fw = full_word(it.m, fbit);
    }
    int kk = 0;
    while (it.valid() && ok) {
      const int sub = kk % kBufs;             // TMEM buffer of this step
      const uint32_t ph = (kk / kBufs) & 1;   // and the phase of its barriers
      Iter n1 = it; n1.next();
      const bool tile_full = (fw >> fbit) & 1u;
      // which of this thread's columns see its key, as bits
      uint32_t seen[kPerLane];
#pragma unroll
      for (int j = 0; j < kPerLane; ++j) {
        seen[j] = 0xffffffffu;
        if (!tile_full) {
          const bool col_live = it.row0() + wg * kHalf + j * kChunk + (lane & (kChunk - 1)) < p.Lq;
          const int lo_c = col_live ? my_lo[j] : 0, hi_c = col_live ? my_hi[j] : 0;
          seen[j] = 0u;
#pragma unroll
          for (int c = 0; c < kChunk; ++c) {
            const int lo = __shfl_sync(0xffffffffu, lo_c, c), hi = __shfl_sync(0xffffffffu, hi_c, c);
            seen[j] |= (key >= lo && key < hi ? 1u : 0u) << c;
          }
        }
      }
      uint32_t hit[kPerLane];
      int anchor_now[kPerLane];
      float nd_now[kPerLane];
      if (HP) {
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) {
          const int rel = my_anchor[j] - (key - lane);
          hit[j] = __ballot_sync(0xffffffffu, rel >= 0 && rel < 32) & (kChunk == 32 ? 0xffffffffu : ((1u << kChunk) - 1u));
          anchor_now[j] = my_anchor[j]; nd_now[j] = my_nd[j];
        }
      }
      if (n1.valid()) {
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) {
          const size_t bi = bound_index(n1, j);
          my_lo[j] = p.row_lo[bi]; my_hi[j] = p.row_hi[bi];
          if (HP) fetch_anchor(n1, j);
        }
        fw = full_word(n1.m, fbit);
      }
      const uint32_t t_s = tmem + lane_off + cS + sub * SM + wg * kHalf;
      const uint32_t t_dp = tmem + lane_off + cDP + sub * SM + wg * kHalf;
      // ---- P^T = exp2((S^T - lse / scale) * c), masked ----
      ok = mbar_wait(ctx, &s.s_full[sub], ph, 80);
      if (!ok) break;
      tc_fence_after();
      float pv[kHalf];
#pragma unroll
      for (int j = 0; j < kPerLane; ++j) {
        if (kChunk == 32) tmem_ld_x32(t_s + j * kChunk, reinterpret_cast<uint32_t*>(pv) + j * kChunk);
        else tmem_ld_x16(t_s + j * kChunk, reinterpret_cast<uint32_t*>(pv) + j * kChunk);
      }
      tc_wait_ld();
#pragma unroll
      for (int j = 0; j < kPerLane; ++j) {
#pragma unroll
        for (int c = j * kChunk; c < (j + 1) * kChunk; c += 2) {
          // a share of the exponentials on the FMA pipe: the special-function unit bounds this loop
          const float2 x = mul2(make_float2(pv[c], pv[c + 1]), cc);
          const float2 e = (!HP && ((c >> 1) & 3) < XB_DKV_FMA_PAIRS) ? ex2_pair_fma(x) : ex2_pair_sfu(x);
          pv[c] = e.x; pv[c + 1] = e.y;
        }
        if (!tile_full) {
#pragma unroll
          for (int c = 0; c < kChunk; ++c) pv[j * kChunk + c] = ((seen[j] >> c) & 1u) ? pv[j * kChunk + c] : 0.f;
        }
        // the 16-bit results go over the first half of the chunk's own columns
        if (kWantDv) {
          uint32_t pp[kChunk / 2];
          uint32_t pp_lo[HP ? kChunk / 2 : 1];
#pragma unroll
          for (int c = 0; c < kChunk; c += 2) {
            float2 pr = make_float2(pv[j * kChunk + c], pv[j * kChunk + c + 1]);
            if (HP) pr = mul2(pr, pr);
            pp[c >> 1] = Pack2<T>::pack(pr.x, pr.y);
            if (HP) {
              // high precision: P goes to the dV product as hi + lo, the lo part in the second half
              // of the chunk's own columns (the dQ kernel's kSplit says why)
              const float2 back = Pack2<T>::unpack(pp[c >> 1]);
              pp_lo[c >> 1] = Pack2<T>::pack(pr.x - back.x, pr.y - back.y);
            }
          }
          if (kChunk == 32) tmem_st_x16(t_s + j * kChunk, pp); else tmem_st_x8(t_s + j * kChunk, pp);
          if (HP) {
            if (kChunk == 32) tmem_st_x16(t_s + j * kChunk + kChunk / 2, pp_lo);
            else tmem_st_x8(t_s + j * kChunk + kChunk / 2, pp_lo);
          }
          tc_wait_st();
        }
        // chunk by chunk, so that dV starts on the first while the second is still being computed
        tc_fence_before();
        mbar_arrive_warp(&s.p_full[sub][j]);  // also: this chunk of S^T has been read
      }
      // ---- dS^T = P^T * (dP^T - delta), the subtraction already done by the product ----
      if (kWantDk) {
        ok = mbar_wait(ctx, &s.dp_full[sub], ph, 83);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) {
          float dpv[kChunk];
          if (kChunk == 32) tmem_ld_x32(t_dp + j * kChunk, reinterpret_cast<uint32_t*>(dpv));
          else tmem_ld_x16(t_dp + j * kChunk, reinterpret_cast<uint32_t*>(dpv));
          tc_wait_ld();
          if (HP && hit[j]) {
#pragma unroll
            for (int c = 0; c < kChunk; ++c) {
              if ((hit[j] >> c) & 1u) {                      // the same for the whole warp
                const int a = __shfl_sync(0xffffffffu, anchor_now[j], c);
                const float ndl = __shfl_sync(0xffffffffu, nd_now[j], c);
                if (key == a) dpv[c] = ndl;
              }
            }
          }
          uint32_t pd[kChunk / 2];
          uint32_t pd_lo[HP ? kChunk / 2 : 1];
#pragma unroll
          for (int c = 0; c < kChunk; c += 2) {
            const int g2 = j * kChunk + c;
            const float2 pr = make_float2(pv[g2], pv[g2 + 1]);
            float2 d = mul2(pr, make_float2(dpv[c], dpv[c + 1]));
            if (HP) d = mul2(pr, d);
            pd[c >> 1] = Pack2<T>::pack(d.x, d.y);
            if (HP) {
              const float2 back = Pack2<T>::unpack(pd[c >> 1]);
              pd_lo[c >> 1] = Pack2<T>::pack(d.x - back.x, d.y - back.y);
            }
          }
          if (kChunk == 32) tmem_st_x16(t_dp + j * kChunk, pd); else tmem_st_x8(t_dp + j * kChunk, pd);
          if (HP) {
            if (kChunk == 32) tmem_st_x16(t_dp + j * kChunk + kChunk / 2, pd_lo);
            else tmem_st_x8(t_dp + j * kChunk + kChunk / 2, pd_lo);
          }
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive_warp(&s.ds_full[sub]);
      }
      it = n1;
      ++kk;
    }
    // epilogue: warpgroup 0 writes dK (scaled), warpgroup 1 writes dV
    if (ok && any_work) ok = mbar_wait(ctx, &s.all_done, 0, 81);
    const bool mine = (wg == 0) ? kWantDk : kWantDv;
    if (ok && mine) {
      tc_fence_after();
      const bool live = key < p.Lk;
      const int width = wg == 0 ? p.D : p.V;
      const int pad = wg == 0 ? d_pad : v_pad;
      const float mul = (wg == 0 ? p.scale : 1.f) * (p.grad_unscale ? __ldg(p.grad_unscale) : 1.f);
      const uint32_t col = wg == 0 ? cDK : cDV;
      T* out = wg == 0
          ? reinterpret_cast<T*>(p.dk) + (((size_t)b * p.Lk + (live ? key : 0)) * p.Hkv + kvh) * p.D
          : reinterpret_cast<T*>(p.dv) + (((size_t)b * p.Lk + (live ? key : 0)) * p.Hkv + kvh) * p.V;
      // With 128-row steps the gradients leave through shared memory (a stage buffer: every product
      // has run) and bulk tensor stores: coalesced and clipped to the tensor by the hardware.
      // Layout: 64-column boxes of 128-byte rows in the 128-byte swizzle.
      constexpr bool kStoreByTma = SM == kBlockN;
      uint8_t* stage_buf = wg == 0 ? s.q[0] : s.d_o[0];
      for (int c0 = 0; c0 < pad; c0 += 32) {
        uint32_t o[32];
        if (any_work) {
          tmem_ld_x32(tmem + lane_off + col + c0, o);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] = 0u;
        }
        if (kStoreByTma) {
          uint8_t* box = stage_buf + (c0 >> 6) * kKvBox + r * 128;
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 u;
            u.x = Pack2<T>::pack(__uint_as_float(o[c + 0]) * mul, __uint_as_float(o[c + 1]) * mul);
            u.y = Pack2<T>::pack(__uint_as_float(o[c + 2]) * mul, __uint_as_float(o[c + 3]) * mul);
            u.z = Pack2<T>::pack(__uint_as_float(o[c + 4]) * mul, __uint_as_float(o[c + 5]) * mul);
            u.w = Pack2<T>::pack(__uint_as_float(o[c + 6]) * mul, __uint_as_float(o[c + 7]) * mul);
            const int chunk = ((c0 & 63) + c) >> 3;
            *reinterpret_cast<uint4*>(box + ((chunk ^ (r & 7)) << 4)) = u;
          }
        } else if (live) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            if (c0 + c < width) {
              uint4 u;
              u.x = Pack2<T>::pack(__uint_as_float(o[c + 0]) * mul, __uint_as_float(o[c + 1]) * mul);
              u.y = Pack2<T>::pack(__uint_as_float(o[c + 2]) * mul, __uint_as_float(o[c + 3]) * mul);
              u.z = Pack2<T>::pack(__uint_as_float(o[c + 4]) * mul, __uint_as_float(o[c + 5]) * mul);
              u.w = Pack2<T>::pack(__uint_as_float(o[c + 6]) * mul, __uint_as_float(o[c + 7]) * mul);
              *reinterpret_cast<uint4*>(out + c0 + c) = u;
            }
          }
        }
      }
      if (kStoreByTma) {
        fence_proxy_async_smem();
        mbar_arrive_warp(&s.out_staged[wg]);
        if (wt == 0) {
          ok = mbar_wait(ctx, &s.out_staged[wg], 0, 84);
          if (ok) {
            const int nbox = ((wg == 0 ? p.D : p.V) + 63) / 64;
            for (int bx = 0; bx < nbox; ++bx)
              tma_store_4d(wg == 0 ? &tm_dk : &tm_dv, stage_buf + bx * kKvBox, bx * 64, kvh, n * kBlockN, b);
            tma_store_commit();
            tma_store_wait_read_all();
          }
        }
      }
    }
  } else if (warp == 8 && lane == 0 && any_work) {
    // ------------------------------ S^T / dP^T issuer ------------------------------
    const uint32_t idesc_st = make_idesc(kBlockN, SM, kFormat, 0, 0);
    const uint32_t idesc_terms = make_idesc(kBlockN, SM, 1, 0, 0);      // the extra k-step is bf16 whatever T is
    const uint32_t ka = smem_u32(s.k), va = smem_u32(s.v);
    bool ok = mbar_wait(ctx, &s.kv_full, 0, 90);
    int cnt = 0;
    for (Iter it = it0; it.valid() && ok; it.next(), ++cnt) {
      const int buf = cnt % kBufs, st = cnt % kStages;
      const uint32_t prev = ((cnt / kBufs) - 1) & 1;     // phase of the buffer's previous use
      ok = mbar_wait(ctx, &s.q_full[st], (cnt / kStages) & 1, 91);
      // the buffer's previous P^T has been read by its dV product
      if (ok && cnt >= kBufs) ok = mbar_wait(ctx, &s.s_free[buf], prev, 93);
      if (!ok) break;
      tc_fence_after();
      const uint32_t qa = smem_u32(s.q[st]), da = smem_u32(s.d_o[st]);
      for (int js = 0; js < ksteps_qk; ++js) {
        umma_ss(tmem + cS + buf * SM, make_smem_desc(ka + (js >> 2) * kKvBox + (js & 3) * 32, 16, 1024),
                make_smem_desc(qa + (js >> 2) * kQBox + (js & 3) * 32, 16, 1024), idesc_st, js > 0);
      }
      umma_ss(tmem + cS + buf * SM, make_smem_desc_sw32(smem_u32(s.ones_s)), make_smem_desc_sw32(smem_u32(s.terms[st])),
              idesc_terms, 1u);
      umma_commit(&s.s_full[buf]);
      if (kWantDk) {
        if (cnt >= kBufs) ok = mbar_wait(ctx, &s.dp_free[buf], prev, 95);
        if (!ok) break;
        tc_fence_after();
        for (int js = 0; js < ksteps_v; ++js) {
          umma_ss(tmem + cDP + buf * SM, make_smem_desc(va + (js >> 2) * kKvBox + (js & 3) * 32, 16, 1024),
                  make_smem_desc(da + (js >> 2) * kQBox + (js & 3) * 32, 16, 1024), idesc_st, js > 0);
        }
        umma_ss(tmem + cDP + buf * SM, make_smem_desc_sw32(smem_u32(s.ones_dp)),
                make_smem_desc_sw32(smem_u32(s.terms[st])), idesc_terms, 1u);
        umma_commit(&s.dp_full[buf]);
      }
    }
  } else if (warp == 10 && lane == 0 && any_work) {
    // ------------------------------ dV / dK issuer ------------------------------
    // P^T / dS^T: each 32-column chunk (16 for SM = 32) of S^T / dP^T holds its packed results in
    // its own first half, so k-step js (16 query rows) sits at chunk js / kStepsPerChunk
    constexpr int kChunk = SM / 2 < 32 ? SM / 2 : 32, kStepsPerChunk = kChunk / 16;
    constexpr int kChunksPerWg = SM / 2 / kChunk;
    const uint32_t idesc_dv = make_idesc(kBlockN, v_pad, kFormat, 0, 1);
    const uint32_t idesc_dk = make_idesc(kBlockN, d_pad, kFormat, 0, 1);
    bool ok = true;
    int cnt = 0;
    for (Iter it = it0; it.valid() && ok; it.next(), ++cnt) {
      const int buf = cnt % kBufs, st = cnt % kStages;
      const uint32_t ph = (cnt / kBufs) & 1;
      ok = mbar_wait(ctx, &s.q_full[st], (cnt / kStages) & 1, 94);
      if (!ok) break;
      const uint32_t qa = smem_u32(s.q[st]), da = smem_u32(s.d_o[st]);
      // chunk j of both warpgroups arrives together: its k-steps go first
      bool fresh = cnt == 0;
#pragma unroll
      for (int j = 0; j < kChunksPerWg; ++j) {
        ok = mbar_wait(ctx, &s.p_full[buf][j], ph, 92);
        if (!ok) break;
        tc_fence_after();
        if (kWantDv) {
#pragma unroll
          for (int w = 0; w < 2; ++w) {
#pragma unroll
            for (int i = 0; i < kStepsPerChunk; ++i) {
              const int chunk = w * kChunksPerWg + j;
              const int js = chunk * kStepsPerChunk + i;       // k-step: 16 query rows
              const uint32_t a_col = tmem + cS + buf * SM + chunk * kChunk + i * 8;
              umma_ts(tmem + cDV, a_col, make_smem_desc(da + js * 2048, kQBox, 1024), idesc_dv, fresh ? 0u : 1u);
              if (HP) umma_ts(tmem + cDV, a_col + kChunk / 2, make_smem_desc(da + js * 2048, kQBox, 1024), idesc_dv, 1u);
              fresh = false;
            }
          }
        }
      }
      if (!ok) break;
      umma_commit(&s.s_free[buf]);
      if (kWantDk) {
        ok = mbar_wait(ctx, &s.ds_full[buf], ph, 96);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int js = 0; js < SM / 16; ++js) {
          const uint32_t a_col = tmem + cDP + buf * SM + (js / kStepsPerChunk) * kChunk + (js % kStepsPerChunk) * 8;
          umma_ts(tmem + cDK, a_col, make_smem_desc(qa + js * 2048, kQBox, 1024), idesc_dk, (cnt > 0 || js > 0) ? 1u : 0u);
          if (HP) umma_ts(tmem + cDK, a_col + kChunk / 2, make_smem_desc(qa + js * 2048, kQBox, 1024), idesc_dk, 1u);
        }
        umma_commit(&s.dp_free[buf]);
      }
      umma_commit(&s.q_empty[st]);
    }
    if (ok) umma_commit(&s.all_done);
  } else if (warp == 9 && lane == 0 && any_work) {
    // ------------------------------ TMA producer ------------------------------
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_do); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_terms);
    mbar_arrive_expect_tx(&s.kv_full, nbox_qk * kKvBox + (kWantDk ? nbox_v * kKvBox : 0));
    for (int bx = 0; bx < nbox_qk; ++bx) tma_load_4d(s.k + bx * kKvBox, &tm_k, &s.kv_full, bx * 64, kvh, n * kBlockN, b);
    if (kWantDk) {
      for (int bx = 0; bx < nbox_v; ++bx) tma_load_4d(s.v + bx * kKvBox, &tm_v, &s.kv_full, bx * 64, kvh, n * kBlockN, b);
    }
    bool ok = true;
    int cnt = 0;
    for (Iter it = it0; it.valid() && ok; it.next(), ++cnt) {
      const int st = cnt % kStages;
      if (cnt >= kStages) ok = mbar_wait(ctx, &s.q_empty[st], ((cnt / kStages) - 1) & 1, 95);
      if (!ok) break;
      const int h = kvh * G + it.g;
      const int row0 = it.row0();
      mbar_arrive_expect_tx(&s.q_full[st], (nbox_qk + nbox_v) * kQBox + SM * 32);
      tma_load_4d(s.terms[st], &tm_terms, &s.q_full[st], 0, row0, h, b);
      for (int bx = 0; bx < nbox_qk; ++bx) tma_load_4d(s.q[st] + bx * kQBox, &tm_q, &s.q_full[st], bx * 64, h, row0, b);
      for (int bx = 0; bx < nbox_v; ++bx) tma_load_4d(s.d_o[st] + bx * kQBox, &tm_do, &s.q_full[st], bx * 64, h, row0, b);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (s.abort_flag == 1) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { }
    __syncthreads();
  }
  if (warp == 9) { __syncwarp(); tmem_dealloc(tmem, kTmemCols); }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
template <typename T, int HD, int BN, int MODE>
static int launch_dq(const XattnBwdArgs& a, const BwdParams& p, cudaStream_t stream) {
  CUtensorMap tdo, tk, tv;
  if (make_tile_map(&tdo, a.dy, a.dtype, a.batch, a.q_len, a.q_heads, a.v_dim, a.dy_strides[0], a.dy_strides[1], a.dy_strides[2], kBlockM)) return XATTN_E_INVALID;
  if (make_tile_map(&tk, a.k, a.dtype, a.batch, a.k_len, a.kv_heads, a.qk_dim, a.k_strides[0], a.k_strides[1], a.k_strides[2], BN)) return XATTN_E_INVALID;
  if (make_tile_map(&tv, a.v, a.dtype, a.batch, a.k_len, a.kv_heads, a.v_dim, a.v_strides[0], a.v_strides[1], a.v_strides[2], BN)) return XATTN_E_INVALID;
  CUtensorMap tdq;
  if (make_tile_map(&tdq, a.dq, a.dtype, a.batch, a.q_len, a.q_heads, a.qk_dim, a.q_len * a.q_heads * a.qk_dim,
                    a.q_heads * a.qk_dim, a.qk_dim, kBlockM)) return XATTN_E_INVALID;
  auto kern = bwd_dq_kernel<T, HD, BN, MODE>;
  const size_t smem = sizeof(DqSmem<HD, BN>) + 1024;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_error("cudaFuncSetAttribute(dq): %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  const long long grid = (long long)p.nQT * p.Hq * p.B;
  if (grid > 0x7fffffffLL) { set_error("dQ grid out of range"); return XATTN_E_INVALID; }
  {
    ProfileScope prof(MODE == kDqStats ? kProfBwdStats : kProfBwdDq, stream);
    kern<<<(unsigned)grid, 384, smem, stream>>>(tdo, tk, tv, tdq, p);
  }
  return XATTN_OK;
}

template <typename T, int HD, int MODE, int SM, bool HP>
static int launch_dkv(const XattnBwdArgs& a, const BwdParams& p, cudaStream_t stream) {
  CUtensorMap tq, tdo, tk, tv;
  if (make_tile_map(&tq, a.q, a.dtype, a.batch, a.q_len, a.q_heads, a.qk_dim, a.q_strides[0], a.q_strides[1], a.q_strides[2], SM)) return XATTN_E_INVALID;
  if (make_tile_map(&tdo, a.dy, a.dtype, a.batch, a.q_len, a.q_heads, a.v_dim, a.dy_strides[0], a.dy_strides[1], a.dy_strides[2], SM)) return XATTN_E_INVALID;
  if (make_tile_map(&tk, a.k, a.dtype, a.batch, a.k_len, a.kv_heads, a.qk_dim, a.k_strides[0], a.k_strides[1], a.k_strides[2], kBlockN)) return XATTN_E_INVALID;
  if (make_tile_map(&tv, a.v, a.dtype, a.batch, a.k_len, a.kv_heads, a.v_dim, a.v_strides[0], a.v_strides[1], a.v_strides[2], kBlockN)) return XATTN_E_INVALID;
  CUtensorMap tt, tdk, tdv;
  if (make_row_map(&tt, p.row_terms, p.B, p.Hq, p.LqPad, SM)) return XATTN_E_INVALID;
  if (make_tile_map(&tdk, a.dk, a.dtype, a.batch, a.k_len, a.kv_heads, a.qk_dim, a.k_len * a.kv_heads * a.qk_dim,
                    a.kv_heads * a.qk_dim, a.qk_dim, kBlockN)) return XATTN_E_INVALID;
  if (make_tile_map(&tdv, a.dv, a.dtype, a.batch, a.k_len, a.kv_heads, a.v_dim, a.k_len * a.kv_heads * a.v_dim,
                    a.kv_heads * a.v_dim, a.v_dim, kBlockN)) return XATTN_E_INVALID;
  auto kern = bwd_dkv_kernel<T, HD, MODE, SM, HP>;
  const size_t smem = sizeof(DkvSmem<HD, MODE, SM>) + 1024;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_error("cudaFuncSetAttribute(dkv): %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  const long long grid = (long long)p.nKT * p.Hkv * p.B;
  if (grid > 0x7fffffffLL) { set_error("dK/dV grid out of range"); return XATTN_E_INVALID; }
  {
    ProfileScope prof(kProfBwdDkv, stream);
    kern<<<(unsigned)grid, 384, smem, stream>>>(tq, tdo, tk, tv, tt, tdk, tdv, p);
  }
  return XATTN_OK;
}

// Which parts of the backward a call runs (XattnBwdArgs.phases; 0 means all three).
constexpr int kPhasePre = XATTN_BWD_PHASE_PRE, kPhaseDq = XATTN_BWD_PHASE_DQ, kPhaseDkv = XATTN_BWD_PHASE_DKV;

template <typename T, bool HP>
static int launch_bwd(const XattnBwdArgs& a, BwdParams& p, cudaStream_t stream) {
  const int phases = a.phases ? a.phases : (kPhasePre | kPhaseDq | kPhaseDkv);
  // 1. preprocess
  // workspace: -delta, -lse2 (FP32 each), the 32-byte rows of extra GEMM columns, and (high precision)
  // -dP at the anchor key
  const size_t rows = (size_t)p.B * p.Hq * p.LqPad;
  float* ndelta = a.workspace;
  float* nlse2 = a.workspace + rows;
  uint4* row_terms = reinterpret_cast<uint4*>(a.workspace + 2 * rows);
  float* ndpa = a.workspace + 10 * rows;
  p.ndelta = ndelta; p.nlse2 = nlse2; p.row_terms = row_terms;
  p.ndpa = HP ? ndpa : nullptr; p.ndelta_out = ndelta; p.row_terms_out = row_terms;
  if (!(phases & kPhasePre)) {
    // the statistics are in the workspace already (an earlier call with the same arguments)
  } else if (HP) {
    const long long blocks = ((long long)rows + 7) / 8;
    if (blocks > 0x7fffffffLL) { set_error("backward preprocess grid out of range"); return XATTN_E_INVALID; }
    ProfileScope prof(kProfBwdPre, stream);
    bwd_pre_hp_kernel<T><<<(unsigned)blocks, 128, 0, stream>>>(
        reinterpret_cast<const T*>(a.dy), reinterpret_cast<const T*>(a.v), a.lse, a.anchor, p.B, p.Lq, p.Lk, p.Hq,
        p.Hkv, p.V, a.dy_strides[0], a.dy_strides[1], a.dy_strides[2], a.v_strides[0], a.v_strides[1],
        a.v_strides[2], p.LqPad, ndpa, nlse2);
  } else {
    const int chunks = p.V >> 3;
    const int per_block = kPreIters * (kPreThreads / 32) * kPrePasses * 32 / (chunks <= 8 ? 8 : (chunks <= 16 ? 16 : 32));
    const long long blocks = ((long long)p.LqPad * p.Hq + per_block - 1) / per_block;
    if (blocks > 0x7fffffffLL) { set_error("backward preprocess grid out of range"); return XATTN_E_INVALID; }
    ProfileScope prof(kProfBwdPre, stream);
    bwd_pre_kernel<T><<<dim3((unsigned)blocks, (unsigned)(p.B < 65535 ? p.B : 65535)), kPreThreads, 0, stream>>>(
        reinterpret_cast<const T*>(a.dy), reinterpret_cast<const T*>(a.y), a.lse, p.B, p.Lq, p.Hq, p.V,
        a.dy_strides[0], a.dy_strides[1], a.dy_strides[2], a.y_strides[0], a.y_strides[1], a.y_strides[2], p.LqPad,
        p.scale, ndelta, nlse2, row_terms);
  }
  const int hd = p.D > p.V ? p.D : p.V;
  constexpr int kDq = HP ? kDqHigh : kDqPlain;
  int rc;
  const bool pre = phases & kPhasePre, dq = phases & kPhaseDq, dkv = phases & kPhaseDkv;
  // (high precision: the statistics pass belongs to the preprocess phase)   2. dQ   3. dK / dV
  if (hd <= 64) {
    if (HP && pre && (rc = launch_dq<T, 64, 128, kDqStats>(a, p, stream))) return rc;
    if (dq && (rc = launch_dq<T, 64, 128, kDq>(a, p, stream))) return rc;
    if (dkv && (rc = launch_dkv<T, 64, kDkvBoth, 128, HP>(a, p, stream))) return rc;
  } else if (hd <= 128) {
    if (HP && pre && (rc = launch_dq<T, 128, 128, kDqStats>(a, p, stream))) return rc;
    if (dq && (rc = launch_dq<T, 128, 128, kDq>(a, p, stream))) return rc;
    if (dkv && (rc = launch_dkv<T, 128, kDkvBoth, 128, HP>(a, p, stream))) return rc;
  } else {
    if (HP && pre && (rc = launch_dq<T, 256, 64, kDqStats>(a, p, stream))) return rc;
    if (dq && (rc = launch_dq<T, 256, 64, kDq>(a, p, stream))) return rc;
    if (dkv && (rc = launch_dkv<T, 256, kDvOnly, 64, HP>(a, p, stream))) return rc;
    if (dkv && (rc = launch_dkv<T, 256, kDkOnly, 32, HP>(a, p, stream))) return rc;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("backward launch: %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  return XATTN_OK;
}

int bwd_entry(const XattnBwdArgs* a, cudaStream_t stream) {
  if (!a) { set_error("null arguments"); return XATTN_E_INVALID; }
  if (a->dtype != XATTN_DTYPE_F16 && a->dtype != XATTN_DTYPE_BF16) { set_error("Q/K/V dtype must be fp16 or bf16"); return XATTN_E_INVALID; }
  if (a->batch <= 0 || a->q_len <= 0 || a->k_len <= 0 || a->q_heads <= 0 || a->kv_heads <= 0 ||
      a->q_heads % a->kv_heads != 0) { set_error("bad batch / length / head counts"); return XATTN_E_INVALID; }
  if (a->qk_dim < 8 || a->qk_dim > 256 || a->qk_dim % 8 || a->v_dim < 8 || a->v_dim > 256 || a->v_dim % 8) {
    set_error("head dimensions must be multiples of 8 in [8, 256]"); return XATTN_E_INVALID;
  }
  if (!(a->scale > 0.f) || !isfinite(a->scale)) { set_error("scale must be finite and positive"); return XATTN_E_INVALID; }
  if (!a->q || !a->k || !a->v || !a->y || !a->dy || !a->lse || !a->plan || !a->dq || !a->dk || !a->dv ||
      !a->workspace || !a->status) { set_error("null tensor pointer"); return XATTN_E_INVALID; }
  if (a->phases & ~(XATTN_BWD_PHASE_PRE | XATTN_BWD_PHASE_DQ | XATTN_BWD_PHASE_DKV)) { set_error("unknown backward phase bits"); return XATTN_E_INVALID; }
  if (a->high_precision && !a->anchor) { set_error("the high-precision backward needs the forward's anchor keys"); return XATTN_E_INVALID; }
  for (const void* ptr : {a->q, a->y, a->dy, (const void*)a->dq, (const void*)a->dk, (const void*)a->dv,
                          (const void*)a->workspace}) {
    if (reinterpret_cast<uintptr_t>(ptr) & 15) { set_error("tensors must be 16-byte aligned"); return XATTN_E_INVALID; }
  }
  for (const int64_t* st : {a->q_strides, a->y_strides, a->dy_strides}) {
    for (int i = 0; i < 3; ++i) if (st[i] % 8) { set_error("q / y / dy strides must be multiples of 8 elements"); return XATTN_E_INVALID; }
  }
  BwdParams p;
  p.B = (int)a->batch; p.Lq = (int)a->q_len; p.Lk = (int)a->k_len; p.Hq = (int)a->q_heads; p.Hkv = (int)a->kv_heads;
  p.D = (int)a->qk_dim; p.V = (int)a->v_dim;
  const PlanLayout pl(a->batch, a->q_len, a->k_len);
  p.nQT = (int)pl.nQT; p.nKT = (int)pl.nKT;
  p.LqPad = p.nQT * kBlockM;
  p.scale = a->scale;
  p.row_lo = a->plan + pl.off_lo; p.row_hi = a->plan + pl.off_hi;
  p.q_tiles = reinterpret_cast<const TileInfo*>(a->plan + pl.off_qt);
  p.k_tiles = reinterpret_cast<const KeyTileInfo*>(a->plan + pl.off_kt);
  p.k_order = a->plan + pl.off_ko;
  p.q = a->q; p.q_sb = a->q_strides[0]; p.q_sl = a->q_strides[1]; p.q_sh = a->q_strides[2];
  p.dq = a->dq; p.dk = a->dk; p.dv = a->dv; p.status = a->status;
  p.anchor = a->anchor; p.grad_unscale = a->grad_unscale;
  if (a->dtype == XATTN_DTYPE_BF16) {
    return a->high_precision ? launch_bwd<__nv_bfloat16, true>(*a, p, stream) : launch_bwd<__nv_bfloat16, false>(*a, p, stream);
  }
  return a->high_precision ? launch_bwd<__half, true>(*a, p, stream) : launch_bwd<__half, false>(*a, p, stream);
}

}  // namespace xb
