// Forward attention for sm_100a.
//
// One CTA owns one tile of 128 query rows of one (batch, query head) and walks the key tiles its
// visible-key intervals touch.  Roles (XB_FWD_PARTS = 2: 16 warps):
//   warps 0-7         two softmax warpgroups: thread = (query row, half of the key tile's 128
//                     columns); the parts exchange their row maxima through shared memory
//   warps 8-11        correction warpgroup (rescales O in TMEM); the epilogue (y and lse) is shared by
//                     warps 0-11
//   warp 12           tcgen05.mma issuer of O += P V (one thread)
//   warp 13           TMA producer (one thread); also owns the TMEM allocation
//   warp 14           tcgen05.mma issuer of S = Q K^T (one thread): an issuing thread stalls while
//                     its products run, so two of them keep the tensor pipe fed while one waits
// S has two TMEM buffers, so S = Q K^T of the next key tiles is already running while the softmax of
// the current one works: softmax in registers -> P (16-bit) into TMEM -> O += P V (P from TMEM, V
// from shared memory, O in TMEM).  For head dimensions up to 128 P has TMEM columns of its own, so
// that the next S product never has to wait for a P V product to release its buffer; at 256 the
// accumulator leaves no room and P is written over its own half of S.
//
// Semantics restated from the reference: online softmax in the exp2 domain
// (csrc/attention/cuda/softmax.h:124-207), rows without a visible key give y = 0 and lse = -inf
// (csrc/attention/hopper/epilogue_fwd.hpp:474-566), key tiles no row can see are skipped
// (hopper/mainloop_fwd_sm90_tma_gmma_ws.hpp:1169-1172).
#include "common.cuh"

#ifndef XB_FWD_FMA_PAIRS
#define XB_FWD_FMA_PAIRS 1
#endif
// softmax warpgroups per CTA: each takes 128 / XB_FWD_PARTS columns of a key tile.  2 or 4; four
// (24 warps, 32 columns per thread) measured 10 % slower than two: the per-tile synchronisation of a
// softmax warp costs as much as its arithmetic then.
#ifndef XB_FWD_PARTS
#define XB_FWD_PARTS 2
#endif


namespace xb {

struct FwdParams {
  int B, Lq, Lk, Hq, Hkv, D, V;
  int nQT;                // 128-row query tiles per batch row
  float scale;
  const int* row_lo;      // [B][Lq]
  const int* row_hi;      // [B][Lq]
  const TileInfo* q_tiles;  // [B][nQT]
  void* y;                // [B][Lq][Hq][V]
  float* lse;             // [B][Hq][Lq]
  float* y_state;         // optional fp32 copy of y
  int* anchor;            // optional (HP): [B][Hq][Lq] key index of the row's largest logit
  int* status;
  // decode shape only (template flag DEC): the query heads of a KV group share the tile, the key
  // tiles are divided among `splits` CTAs per (batch, KV head), partial results go to the workspace
  int splits;
  int g_shift;            // log2 of the group size Hq / Hkv
  float* part_y;          // [splits][B][Lq][Hq][V], normalised per split
  float* part_lse;        // [splits][B][Hq][Lq], natural log; -inf where the split saw no key
};

template <int HD>
struct FwdSmem {
  static constexpr int kTileBytes = kBlockM * HD * 2;
  static constexpr int kKStages = HD <= 128 ? 3 : 1;
  static constexpr int kVStages = HD <= 128 ? 2 : 1;
  static constexpr int kLookahead = HD <= 128 ? 2 : 1;   // K tiles the producer loads ahead of V
  alignas(1024) uint8_t q[kTileBytes];
  alignas(1024) uint8_t k[kKStages][kTileBytes];
  alignas(1024) uint8_t v[kVStages][kTileBytes];
  float scale_buf[2][kBlockM];       // rescale factors, double-buffered by iteration parity
  float xmax[4][XB_FWD_PARTS][kBlockM];   // row maxima of the column parts, by iteration mod 4
  float final_l[XB_FWD_PARTS][kBlockM];
  float final_m[kBlockM];
  float best_s[XB_FWD_PARTS][kBlockM];   // HP: largest logit of each column part and its key index
  int best_i[XB_FWD_PARTS][kBlockM];
  uint64_t q_full;
  uint64_t k_full[kKStages], k_empty[kKStages];
  uint64_t v_full[kVStages], v_empty[kVStages];
  uint64_t s_full[2], s_free[2], p_full[2], p_free[2], max_x[4];
  uint64_t o_ready, pv_done, corr_full, final_full, y_staged, o_final;
  uint32_t tmem_base;
  int abort_flag;
};

// T: __nv_bfloat16 or __half.  HD: padded head dimension of the shared-memory tiles (64, 128 or 256).
// HP: high-precision softmax.
// DEC: decode shape, Lq * (Hq / Hkv) <= 128.  Tile row r holds query row r / G of head kvh * G + r % G
// (one TMA box over G heads), so K and V are read once per KV head instead of once per query head; the
// CTA takes one share of the key tiles and writes a normalised FP32 partial result with its lse, which
// fwd_combine_kernel merges.  Everything between the Q load and the epilogue is the same code.
constexpr int kFwdParts = XB_FWD_PARTS;                 // softmax warpgroups
constexpr int kFwdThreads = (4 * kFwdParts + 8) * 32;   // + correction warpgroup + issuers / TMA

template <typename T, int HD, bool HP, bool DEC>
__global__ void __launch_bounds__(kFwdThreads, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
           const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_y, const FwdParams p) {
  using Smem = FwdSmem<HD>;
  constexpr bool kAliasP = HD > 128;                    // P over S instead of in columns of its own
  constexpr int kKStages = Smem::kKStages, kVStages = Smem::kVStages, kLA = Smem::kLookahead;
  constexpr int kBoxBytes = kBlockM * 64 * 2;          // one 64-column box of a tile
  constexpr uint32_t kTmemCols = 512;
  // TMEM columns: S buffers at 0 / 128, O at 256, P buffers (64 packed columns each) at 384 / 448
  constexpr uint32_t cS = 0, cO = 256, cP = 384;
  constexpr int kFormat = Pack2<T>::kFormat;
  constexpr int kParts = kFwdParts;                     // softmax warpgroups
  constexpr int kCols = kBlockN / kParts;               // key-tile columns per softmax thread
  constexpr int kCorrWarp = 4 * kParts, kPvWarp = kCorrWarp + 4, kTmaWarp = kCorrWarp + 5, kQkWarp = kCorrWarp + 6;
  // of every four pairs of exponentials, how many are computed on the FMA pipe (low precision only)
  constexpr int kFmaPairs = XB_FWD_FMA_PAIRS;

  extern __shared__ uint8_t smem_raw[];
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // ---- which work item -----------------------------------------------------
  const int G = p.Hq / p.Hkv;
  const int per_bk = DEC ? p.splits : p.nQT * G;
  const int bk = blockIdx.x / per_bk;
  const int rem = blockIdx.x - bk * per_bk;
  const int qt = DEC ? 0 : p.nQT - 1 - rem / G;       // later (heavier under causal masks) tiles first
  const int kvh = bk % p.Hkv;
  const int h = DEC ? kvh * G : kvh * G + (rem % G);  // DEC: first head of the group
  const int b = bk / p.Hkv;
  const int split = DEC ? rem : 0;

  if (warp == kTmaWarp && lane == 0) {
    // The Q tile needs nothing but the block index: its load starts before anything else, the mask
    // plan's tile summary included (its barrier is initialised here, by the thread that uses it first).
    tma_prefetch_desc(&tm_q);
    mbar_init(&s.q_full, 1);
    fence_mbar_init();
    mbar_arrive_expect_tx(&s.q_full, ((p.D + 63) / 64) * kBoxBytes);
    for (int bx = 0; bx < (p.D + 63) / 64; ++bx)
      tma_load_4d(s.q + bx * kBoxBytes, &tm_q, &s.q_full, bx * 64, h, qt * kBlockM, b);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_y);
  }
  int n_lo = 0, n_hi = 0, full_lo = 0x7fffffff, full_hi = 0;
  {
    const TileInfo ti = p.q_tiles[(size_t)b * p.nQT + qt];
    if (ti.max_hi > ti.min_lo) {
      n_lo = ti.min_lo / kBlockN;
      n_hi = (ti.max_hi + kBlockN - 1) / kBlockN;
      full_lo = ti.max_lo;
      full_hi = ti.min_hi;
    }
  }
  if (DEC) {
    // this CTA's share of the key tiles (possibly none)
    const int per = (n_hi - n_lo + p.splits - 1) / p.splits;
    n_lo = min(n_lo + split * per, n_hi);
    n_hi = min(n_lo + per, n_hi);
  }
  const int iters = n_hi - n_lo;
  // The first K tiles are requested as soon as the tile summary says which they are, before the
  // CTA's set-up barrier: tile summary -> K load -> first S product is the chain every CTA starts
  // with, and with short key ranges (packed segments) it is a good part of the CTA's life.
  constexpr int kEarlyK = kKStages < 2 ? kKStages : 2;
  if (warp == kTmaWarp && lane == 0) {
    for (int i = 0; i < kKStages; ++i) mbar_init(&s.k_full[i], 1);
    fence_mbar_init();
    for (int i = 0; i < kEarlyK && i < iters; ++i) {
      mbar_arrive_expect_tx(&s.k_full[i], ((p.D + 63) / 64) * kBoxBytes);
      for (int bx = 0; bx < (p.D + 63) / 64; ++bx)
        tma_load_4d(s.k[i] + bx * kBoxBytes, &tm_k, &s.k_full[i], bx * 64, kvh, (n_lo + i) * kBlockN, b);
    }
  }

  // ---- set-up ----------------------------------------------------------------
  if (tid == 0) {
    // an earlier CTA gave up: do not pile on
    s.abort_flag = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 2 : 0;
    for (int i = 0; i < kKStages; ++i) mbar_init(&s.k_empty[i], 1);       // k_full: by the TMA thread, above
    for (int i = 0; i < kVStages; ++i) { mbar_init(&s.v_full[i], 1); mbar_init(&s.v_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.s_full[i], 1); mbar_init(&s.p_full[i], 4 * kParts);
      mbar_init(&s.max_x[2 * i], 4 * kParts); mbar_init(&s.max_x[2 * i + 1], 4 * kParts);
      mbar_init(&s.p_free[i], 1);              // the P V product has read the P buffer
      // an S buffer is free again once the softmax holds it in registers, or, where P lies over S,
      // once the P V product has read it
      mbar_init(&s.s_free[i], kAliasP ? 1 : 4 * kParts);
    }
    mbar_init(&s.o_ready, 4);
    mbar_init(&s.pv_done, 1);
    mbar_init(&s.corr_full, 4);
    mbar_init(&s.final_full, 4 * kParts);
    mbar_init(&s.y_staged, 4 * (kParts + 1));
    mbar_init(&s.o_final, 1);               // the last O += P V product has run
    fence_mbar_init();
  }
  if (warp == kTmaWarp) {
    tmem_alloc(&s.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  WaitCtx ctx{&s.abort_flag, p.status, 2000000000ull};

  const int nbox_qk = (p.D + 63) / 64;
  const int nbox_v = (p.V + 63) / 64;
  const int ksteps_qk = (p.D + 15) / 16;
  const int v_pad = (p.V + 15) & ~15;
  const bool dead = s.abort_flag != 0;

  // Registers move between warps of this CTA only: what the softmax warps gain must not exceed what
  // the others give up, or setmaxnreg.inc waits for ever.  512 threads start with 128 each, 768 with 80.
  if (kParts == 2) {
    static_assert(kParts != 2 || 256 * (152 - 128) <= 128 * (128 - 104) + 128 * (128 - 48), "register budget");
    if (warp < 8) setmaxnreg_inc<152>(); else if (warp < 12) setmaxnreg_dec<104>(); else setmaxnreg_dec<48>();
  } else {
    static_assert(kParts != 4 || 512 * (88 - 80) <= 128 * (80 - 40), "register budget");
    if (warp < 16) setmaxnreg_inc<88>(); else if (warp >= 20) setmaxnreg_dec<40>();
  }

  // Epilogue: y = O / l, lse = ln2 * (m * c + log2 l).  Shared by all warpgroups that worked on the
  // tile (softmax parts 0 .. kParts-1, correction = kParts): each converts every (kParts+1)-th
  // 16-column chunk of the rows' output.  The conversion is a chain of latencies (TMEM load, convert,
  // shared-memory store) that four warps alone do not hide: in-kernel cycle counters gave 1 300 clk
  // for the staging of a 128 x 128 tile by three warpgroups.  A lambda, so that every role
  // instantiates it inside its own register allotment (a code path shared across the roles would
  // be compiled for the smallest of them).
  auto epilogue = [&](const int part, bool ok) {
    const int r = tid & 127;
    const int row = DEC ? (r >> p.g_shift) : qt * kBlockM + r;
    const int hr = DEC ? h + (r & (G - 1)) : h;       // this row's query head
    const bool live = row < p.Lq;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    if (ok) ok = mbar_wait(ctx, &s.final_full, 0, 24);
    // (not pv_done: a warp that has not followed that barrier's phases cannot tell the last product
    // from the one two before it)
    if (ok && iters > 0) ok = mbar_wait(ctx, &s.o_final, 0, 26);
    if (ok && iters == 0) ok = mbar_wait(ctx, &s.q_full, 0, 28);   // the Q load has landed: its buffer is reused below
    if (ok) {
      tc_fence_after();
      float l = 0.f;
#pragma unroll
      for (int o = 0; o < kParts; ++o) l += s.final_l[o][r];
      const float m = s.final_m[r];
      const bool has = l > 0.f && iters > 0;
      float inv = 0.f;
      if (has) inv = HP ? __frcp_rn(l) : __fdividef(1.f, l);
      if (live && part == kParts) {
        const float c_log2 = p.scale * 1.4426950408889634f;
        float* lse_out = DEC ? p.part_lse + (size_t)split * p.B * p.Hq * p.Lq : p.lse;
        lse_out[((size_t)b * p.Hq + hr) * p.Lq + row] =
            has ? (m * c_log2 + log2f(l)) * 0.6931471805599453f : -INFINITY;
        if (HP && !DEC && p.anchor) {
          float bs = -INFINITY;
          int bi = -1;
          if (iters > 0) {
#pragma unroll
            for (int o = 0; o < kParts; ++o) {
              const float v = s.best_s[o][r];
              const int i = s.best_i[o][r];
              if (i >= 0 && (v > bs || (v == bs && i < bi))) { bs = v; bi = i; }
            }
          }
          p.anchor[((size_t)b * p.Hq + hr) * p.Lq + row] = bi;
        }
      }
      // y leaves through shared memory and bulk tensor stores (the Q tile's buffer is free by now:
      // every S product has run): coalesced, clipped to the tensor by the hardware, and the CTA
      // does not have to wait for the writes themselves.  Layout: 64-column boxes of 128-byte
      // rows in the 128-byte swizzle (16-byte chunk c of row r sits at chunk c ^ (r & 7)).
      const uint32_t t_o = tmem + lane_off + cO;
      float* ys_base = DEC ? p.part_y + (size_t)split * p.B * p.Lq * p.Hq * p.V : p.y_state;
      float* ys_row = ys_base ? ys_base + (((size_t)b * p.Lq + (live ? row : 0)) * p.Hq + hr) * p.V : nullptr;
      for (int c0 = 16 * part; c0 < v_pad; c0 += 16 * (kParts + 1)) {
        uint32_t o[16];
        if (iters > 0) {
          tmem_ld_x16(t_o + c0, o);   // warp-collective: executed by all lanes
          tc_wait_ld();
        } else {
#pragma unroll
          for (int c = 0; c < 16; ++c) o[c] = 0u;
        }
        uint8_t* box = s.q + (c0 >> 6) * kBoxBytes + r * 128;
#pragma unroll
        for (int c = 0; c < 16; c += 8) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(o[c + e]) * inv;
          uint4 pk;
          pk.x = Pack2<T>::pack(f[0], f[1]);
          pk.y = Pack2<T>::pack(f[2], f[3]);
          pk.z = Pack2<T>::pack(f[4], f[5]);
          pk.w = Pack2<T>::pack(f[6], f[7]);
          const int chunk = ((c0 & 63) + c) >> 3;
          if (!DEC) *reinterpret_cast<uint4*>(box + ((chunk ^ (r & 7)) << 4)) = pk;
          if (ys_row && live && c0 + c < p.V) {
            *reinterpret_cast<float4*>(ys_row + c0 + c) = make_float4(f[0], f[1], f[2], f[3]);
            *reinterpret_cast<float4*>(ys_row + c0 + c + 4) = make_float4(f[4], f[5], f[6], f[7]);
          }
        }
      }
      fence_proxy_async_smem();
      mbar_arrive_warp(&s.y_staged);
      if (!DEC && warp == kCorrWarp && lane == 0) {
        ok = mbar_wait(ctx, &s.y_staged, 0, 27);
        if (ok) {
          for (int bx = 0; bx < nbox_v; ++bx) tma_store_4d(&tm_y, s.q + bx * kBoxBytes, bx * 64, h, qt * kBlockM, b);
          tma_store_commit();
          tma_store_wait_read_all();
        }
      }
    }
  };

  if (dead) {
    // nothing to do
  } else if (warp < 4 * kParts) {
    // =========================== softmax warpgroups ===========================
    const int hf = warp >> 2;                   // which part of the key-tile columns
    const int r = tid & 127;
    const int row = DEC ? (r >> p.g_shift) : qt * kBlockM + r;
    int lo = 0, hi = 0;
    if (row < p.Lq) {
      lo = p.row_lo[(size_t)b * p.Lq + row];
      hi = p.row_hi[(size_t)b * p.Lq + row];
    }
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const float c_log2 = p.scale * 1.4426950408889634f;
    float m = -INFINITY, l = 0.f;
    float best = -INFINITY;                     // HP: this part's largest logit so far and where it was
    int best_idx = -1;
    bool ok = true;
    for (int j = 0; j < iters && ok; ++j) {
      const int buf = j & 1;
      const int col0 = (n_lo + j) * kBlockN + hf * kCols;
      const uint32_t t_s = tmem + lane_off + cS + buf * 128 + hf * kCols;
      ok = mbar_wait(ctx, &s.s_full[buf], (j >> 1) & 1, 10);
      if (!ok) break;
      tc_fence_after();
      float sc[kCols];
#pragma unroll
      for (int c = 0; c < kCols; c += 32) tmem_ld_x32(t_s + c, reinterpret_cast<uint32_t*>(sc) + c);
      tc_wait_ld();
      if (!kAliasP) {
        tc_fence_before();
        mbar_arrive_warp(&s.s_free[buf]);
      }
      const bool tile_full = ((n_lo + j) * kBlockN >= full_lo) && ((n_lo + j + 1) * kBlockN <= full_hi);
      if (!tile_full) {
        const int rl = lo - col0, rh = hi - col0;
#pragma unroll
        for (int c = 0; c < kCols; ++c) sc[c] = (c >= rl && c < rh) ? sc[c] : -INFINITY;
      }
      float mx4[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) mx4[e] = max3(sc[8 * e], sc[8 * e + 1], sc[8 * e + 2]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        mx4[e] = max3(mx4[e], sc[8 * e + 3], sc[8 * e + 4]);
        mx4[e] = max3(mx4[e], sc[8 * e + 5], sc[8 * e + 6]);
        mx4[e] = fmaxf(mx4[e], sc[8 * e + 7]);
      }
#pragma unroll
      for (int c = 32; c < kCols; c += 8) {
        const int e = (c >> 3) & 3;
        mx4[e] = max3(mx4[e], sc[c], sc[c + 1]);
        mx4[e] = max3(mx4[e], sc[c + 2], sc[c + 3]);
        mx4[e] = max3(mx4[e], sc[c + 4], sc[c + 5]);
        mx4[e] = max3(mx4[e], sc[c + 6], sc[c + 7]);
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      if (HP && mx > best) {
        // the anchor key of the high-precision backward: the first key holding the row's maximum
        best = mx;
#pragma unroll
        for (int c = kCols - 1; c >= 0; --c) best_idx = (sc[c] == mx) ? col0 + c : best_idx;
      }
      // The row maximum over all column parts.  Four slots: a part can be here for tile j + 4 only
      // after every part has loaded S of tile j + 2 (the S buffer it needs is free no earlier), that
      // is after every part has finished with the slot of tile j.  With two slots a part running
      // ahead could overwrite a maximum another part has not read yet.
      s.xmax[j & 3][hf][r] = mx;
      mbar_arrive_warp(&s.max_x[j & 3]);
      ok = mbar_wait(ctx, &s.max_x[j & 3], (j >> 2) & 1, 11);
      if (!ok) break;
#pragma unroll
      for (int o = 1; o < kParts; ++o) mx = fmaxf(mx, s.xmax[j & 3][(hf + o) % kParts][r]);
      float m_new = fmaxf(m, mx);
      if (!HP) {
        // keep the old reference while the maximum grew by less than 2^8: the accumulator is then
        // left untouched and P stays below 256
        if (m != -INFINITY && (m_new - m) * c_log2 <= 8.f) m_new = m;
      }
      float factor = 1.f;
      if (m != -INFINITY && m_new != m) factor = HP ? exp2f((m - m_new) * c_log2) : ex2_approx((m - m_new) * c_log2);
      m = m_new;
      const float m_ref = (m == -INFINITY) ? 0.f : m;
      const float neg_mc = -m_ref * c_log2;
      uint32_t pk[kCols / 2];
      float sum = 0.f;
      if (HP) {
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < kCols; c += 2) {
          const float p0 = exp2f(__fmul_rn(__fsub_rn(sc[c], m_ref), c_log2));
          const float p1 = exp2f(__fmul_rn(__fsub_rn(sc[c + 1], m_ref), c_log2));
          sum4[(c >> 1) & 3] += p0 + p1;
          pk[c >> 1] = Pack2<T>::pack(p0, p1);
        }
        sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      } else {
        // A share of the exponentials runs on the FMA pipe: the special-function unit (16 results
        // per clock and SM) is what bounds this loop.  Which elements take which route does not
        // depend on the tile, so that a row gets the same bits however its neighbours are masked;
        // the FMA route cannot return 0 for -inf, hence the extra selects on tiles that mask.
        const float2 cc = make_float2(c_log2, c_log2), nm = make_float2(neg_mc, neg_mc);
        float2 s2a = make_float2(0.f, 0.f), s2b = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < kCols; c += 8) {
          float2 pr[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 x = fma2(make_float2(sc[c + 2 * e], sc[c + 2 * e + 1]), cc, nm);
            if (e < kFmaPairs) {
              pr[e] = ex2_pair_fma(x);
              if (!tile_full) {
                pr[e].x = sc[c + 2 * e] == -INFINITY ? 0.f : pr[e].x;
                pr[e].y = sc[c + 2 * e + 1] == -INFINITY ? 0.f : pr[e].y;
              }
            } else {
              pr[e] = ex2_pair_sfu(x);
            }
            pk[(c >> 1) + e] = Pack2<T>::pack(pr[e].x, pr[e].y);
          }
          s2a = add2(s2a, add2(pr[0], pr[1]));
          s2b = add2(s2b, add2(pr[2], pr[3]));
        }
        const float2 s2 = add2(s2a, s2b);
        sum = s2.x + s2.y;
      }
      // kCols / 2 packed columns per part: next to each other in the P buffer (once the product two
      // tiles back has read it), or (HD = 256) over the first half of the part's own S columns
      if (!kAliasP && j >= 2) {
        ok = mbar_wait(ctx, &s.p_free[buf], ((j >> 1) - 1) & 1, 12);
        if (!ok) break;
        tc_fence_after();
      }
      // The rescale factor goes to the correction warpgroup only now: the softmax may run two tiles
      // ahead of the P V products, and the product two tiles back having finished (the wait above;
      // with P over S the S buffer itself could not have been refilled earlier) is what guarantees
      // that the correction warpgroup has taken the factor this slot held before.
      if (hf == 0 && j > 0) {
        s.scale_buf[buf][r] = factor;
        mbar_arrive_warp(&s.corr_full);
      }
      {
        const uint32_t t_p = kAliasP ? t_s : tmem + lane_off + cP + buf * 64 + hf * (kCols / 2);
        if (kCols == 64) tmem_st_x32(t_p, pk); else tmem_st_x16(t_p, pk);
      }
      l = l * factor + sum;
      tc_wait_st();
      tc_fence_before();
      mbar_arrive_warp(&s.p_full[buf]);
    }
    // hand the row statistics to the epilogue
    s.final_l[hf][r] = l;
    if (hf == 0) s.final_m[r] = m;
    if (HP) { s.best_s[hf][r] = best; s.best_i[hf][r] = best_idx; }
    mbar_arrive_warp(&s.final_full);
    epilogue(hf, ok);
  } else if (warp < kCorrWarp + 4) {
    // ======================= correction + epilogue warpgroup =======================
    const int r = tid & 127;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    bool ok = true;
    for (int j = 1; j < iters && ok; ++j) {
      ok = mbar_wait(ctx, &s.corr_full, (j - 1) & 1, 20);
      if (!ok) break;
      const float f = s.scale_buf[j & 1][r];
      ok = mbar_wait(ctx, &s.pv_done, (j - 1) & 1, 22);
      if (!ok) break;
      tc_fence_after();
      if (__any_sync(0xffffffffu, f != 1.f)) {
        const uint32_t t_o = tmem + lane_off + cO;
        for (int c0 = 0; c0 < v_pad; c0 += 32) {
          uint32_t o[32];
          tmem_ld_x32(t_o + c0, o);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * f);
          tmem_st_x32(t_o + c0, o);
        }
        tc_wait_st();
      }
      tc_fence_before();
      mbar_arrive_warp(&s.o_ready);
    }
    epilogue(kParts, ok);
  } else if (warp == kQkWarp && lane == 0 && iters > 0) {
    // ------------------------------ S = Q K^T issuer ------------------------------
    const uint32_t idesc_qk = make_idesc(kBlockM, kBlockN, kFormat, 0, 0);
    bool ok = mbar_wait(ctx, &s.q_full, 0, 30);
    for (int i = 0; i < iters && ok; ++i) {
      const int ks = i % kKStages;
      ok = mbar_wait(ctx, &s.k_full[ks], (i / kKStages) & 1, 31);
      if (ok && i >= 2) ok = mbar_wait(ctx, &s.s_free[i & 1], ((i >> 1) - 1) & 1, 35);
      if (!ok) break;
      tc_fence_after();
      const uint32_t ka = smem_u32(s.k[ks]);
      const uint32_t d = tmem + cS + (i & 1) * 128;
      for (int js = 0; js < ksteps_qk; ++js) {
        const uint32_t off = (js >> 2) * kBoxBytes + (js & 3) * 32;
        umma_ss(d, make_smem_desc(smem_u32(s.q) + off, 16, 1024), make_smem_desc(ka + off, 16, 1024), idesc_qk, js > 0);
      }
      umma_commit(&s.s_full[i & 1]);
      umma_commit(&s.k_empty[ks]);
    }
  } else if (warp == kPvWarp && lane == 0 && iters > 0) {
    // ------------------------------ O += P V issuer ------------------------------
    const uint32_t idesc_pv = make_idesc(kBlockM, v_pad, kFormat, 0, 1);
    bool ok = true;
    for (int n = 0; n < iters && ok; ++n) {
      const int vs = n % kVStages;
      ok = mbar_wait(ctx, &s.v_full[vs], (n / kVStages) & 1, 32);
      if (ok) ok = mbar_wait(ctx, &s.p_full[n & 1], (n >> 1) & 1, 33);
      if (ok && n > 0) ok = mbar_wait(ctx, &s.o_ready, (n - 1) & 1, 34);
      if (!ok) break;
      tc_fence_after();
      const uint32_t va = smem_u32(s.v[vs]);
#pragma unroll
      for (int js = 0; js < kBlockN / 16; ++js) {
        // k-step js = 16 keys = 8 packed columns; over S they sit at the start of their part's columns
        constexpr int kStepsPerPart = kCols / 16;
        const uint32_t a_col = kAliasP ? tmem + cS + (n & 1) * 128 + (js / kStepsPerPart) * kCols + (js % kStepsPerPart) * 8
                                       : tmem + cP + (n & 1) * 64 + js * 8;
        umma_ts(tmem + cO, a_col, make_smem_desc(va + js * 2048, kBoxBytes, 1024), idesc_pv,
                (n > 0 || js > 0) ? 1u : 0u);
      }
      umma_commit(&s.pv_done);
      umma_commit(&s.v_empty[vs]);
      umma_commit(&s.p_free[n & 1]);
      if (kAliasP) umma_commit(&s.s_free[n & 1]);
      if (n == iters - 1) umma_commit(&s.o_final);
    }
  } else if (warp == kTmaWarp && lane == 0 && iters > 0) {
    // ------------------------------ TMA producer ------------------------------
    bool ok = true;
    // K runs kLA tiles ahead of V, the order in which the two products consume them
    for (int i = 0; i < iters + kLA && ok; ++i) {
      if (i >= kEarlyK && i < iters) {
        const int st = i % kKStages;
        if (i >= kKStages) ok = mbar_wait(ctx, &s.k_empty[st], ((i / kKStages) - 1) & 1, 40);
        if (!ok) break;
        mbar_arrive_expect_tx(&s.k_full[st], nbox_qk * kBoxBytes);
        for (int bx = 0; bx < nbox_qk; ++bx)
          tma_load_4d(s.k[st] + bx * kBoxBytes, &tm_k, &s.k_full[st], bx * 64, kvh, (n_lo + i) * kBlockN, b);
      }
      const int iv = i - kLA;
      if (iv >= 0) {
        const int st = iv % kVStages;
        if (iv >= kVStages) ok = mbar_wait(ctx, &s.v_empty[st], ((iv / kVStages) - 1) & 1, 41);
        if (!ok) break;
        mbar_arrive_expect_tx(&s.v_full[st], nbox_v * kBoxBytes);
        for (int bx = 0; bx < nbox_v; ++bx)
          tma_load_4d(s.v[st] + bx * kBoxBytes, &tm_v, &s.v_full[st], bx * 64, kvh, (n_lo + iv) * kBlockN, b);
      }
    }
  }

  // ---- tail -----------------------------------------------------------------
  if (dead && warp == kTmaWarp && lane == 0) {
    // the Q and first K loads were issued before the abort flag was read: let them land (bounded)
    for (int i = 0; i < (1 << 20) && !mbar_try_wait(&s.q_full, 0); ++i) { }
    for (int t = 0; t < kEarlyK && t < iters; ++t)
      for (int i = 0; i < (1 << 20) && !mbar_try_wait(&s.k_full[t], 0); ++i) { }
  }
  tc_fence_before();
  __syncthreads();
  if (s.abort_flag == 1) {
    // give bulk copies still in flight time to land before the CTA retires
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { }
    __syncthreads();
  }
  if (warp == kTmaWarp) {
    __syncwarp();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// Merges the partial results of the decode-shape kernel: one warp per (batch, query row, head).
// lse = log sum_s exp(lse_s), y = sum_s exp(lse_s - lse) y_s, in split order (repeatable); a row no
// split saw a key for gives y = 0 and lse = -inf.  HBM-bound: reads splits * (V + 1) floats per row.
template <typename T>
__global__ void __launch_bounds__(128)
fwd_combine_kernel(const FwdParams p) {
  const long long units = (long long)p.B * p.Lq * p.Hq;
  const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (unit >= units) return;
  const int lane = threadIdx.x & 31;
  const int h = (int)(unit % p.Hq);
  const long long br = unit / p.Hq;
  const int row = (int)(br % p.Lq);
  const int b = (int)(br / p.Lq);
  const size_t lse_idx = ((size_t)b * p.Hq + h) * p.Lq + row;
  const size_t lse_stride = (size_t)p.B * p.Hq * p.Lq;
  const size_t y_stride = (size_t)units * p.V;
  float mx = -INFINITY;
  for (int sp = lane; sp < p.splits; sp += 32) mx = fmaxf(mx, p.part_lse[sp * lse_stride + lse_idx]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  if (mx != -INFINITY)
    for (int sp = lane; sp < p.splits; sp += 32) sum += expf(p.part_lse[sp * lse_stride + lse_idx] - mx);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float lse = mx == -INFINITY ? -INFINITY : mx + logf(sum);
  float2 acc[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};   // columns 2 * lane + 64 * i
  if (mx != -INFINITY) {
    for (int sp = 0; sp < p.splits; ++sp) {
      const float ls = p.part_lse[sp * lse_stride + lse_idx];
      if (ls == -INFINITY) continue;
      const float w = expf(ls - lse);
      const float* src = p.part_y + sp * y_stride + (size_t)unit * p.V;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = 2 * lane + 64 * i;
        if (c < p.V) {
          const float2 x = *reinterpret_cast<const float2*>(src + c);
          acc[i].x += w * x.x;
          acc[i].y += w * x.y;
        }
      }
    }
  }
  if (lane == 0) p.lse[lse_idx] = lse;
  T* y = reinterpret_cast<T*>(p.y) + (size_t)unit * p.V;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = 2 * lane + 64 * i;
    if (c < p.V) {
      *reinterpret_cast<uint32_t*>(y + c) = Pack2<T>::pack(acc[i].x, acc[i].y);
      if (p.y_state) *reinterpret_cast<float2*>(p.y_state + (size_t)unit * p.V + c) = acc[i];
    }
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
template <typename T, int HD, bool HP, bool DEC>
static int launch_fwd(const XattnFwdArgs& a, const FwdParams& p, cudaStream_t stream) {
  using Smem = FwdSmem<HD>;
  CUtensorMap tq, tk, tv;
  const int group = p.Hq / p.Hkv;
  // decode shape: one box takes the G heads of a KV group x 128 / G query rows
  if (make_tile_map(&tq, a.q, a.dtype, a.batch, a.q_len, a.q_heads, a.qk_dim, a.q_strides[0], a.q_strides[1],
                    a.q_strides[2], DEC ? kBlockM / group : kBlockM, DEC ? group : 1)) return XATTN_E_INVALID;
  if (make_tile_map(&tk, a.k, a.dtype, a.batch, a.k_len, a.kv_heads, a.qk_dim, a.k_strides[0], a.k_strides[1],
                    a.k_strides[2], kBlockN)) return XATTN_E_INVALID;
  if (make_tile_map(&tv, a.v, a.dtype, a.batch, a.k_len, a.kv_heads, a.v_dim, a.v_strides[0], a.v_strides[1],
                    a.v_strides[2], kBlockN)) return XATTN_E_INVALID;
  CUtensorMap ty;
  if (make_tile_map(&ty, a.y, a.dtype, a.batch, a.q_len, a.q_heads, a.v_dim, a.q_len * a.q_heads * a.v_dim,
                    a.q_heads * a.v_dim, a.v_dim, kBlockM)) return XATTN_E_INVALID;
  const size_t smem = sizeof(Smem) + 1024;
  auto kern = fwd_kernel<T, HD, HP, DEC>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_error("cudaFuncSetAttribute(fwd): %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  const long long grid = DEC ? (long long)p.splits * p.Hkv * p.B : (long long)p.nQT * p.Hq * p.B;
  if (grid <= 0 || grid > 0x7fffffffLL) { set_error("forward grid out of range"); return XATTN_E_INVALID; }
  {
    ProfileScope prof(kProfFwd, stream);
    kern<<<(unsigned)grid, kFwdThreads, smem, stream>>>(tq, tk, tv, ty, p);
    if (DEC) {
      const long long units = (long long)p.B * p.Lq * p.Hq;
      fwd_combine_kernel<T><<<(unsigned)((units + 3) / 4), 128, 0, stream>>>(p);
    }
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("forward launch: %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  return XATTN_OK;
}

template <typename T, bool HP, bool DEC>
static int dispatch_fwd_dim(const XattnFwdArgs& a, const FwdParams& p, cudaStream_t stream) {
  const int hd = (int)(a.qk_dim > a.v_dim ? a.qk_dim : a.v_dim);
  if (hd <= 64) return launch_fwd<T, 64, HP, DEC>(a, p, stream);
  if (hd <= 128) return launch_fwd<T, 128, HP, DEC>(a, p, stream);
  return launch_fwd<T, 256, HP, DEC>(a, p, stream);
}

template <bool DEC>
static int dispatch_fwd(const XattnFwdArgs& a, const FwdParams& p, cudaStream_t stream) {
  if (a.dtype == XATTN_DTYPE_BF16) {
    return a.high_precision ? dispatch_fwd_dim<__nv_bfloat16, true, DEC>(a, p, stream)
                            : dispatch_fwd_dim<__nv_bfloat16, false, DEC>(a, p, stream);
  }
  return a.high_precision ? dispatch_fwd_dim<__half, true, DEC>(a, p, stream)
                          : dispatch_fwd_dim<__half, false, DEC>(a, p, stream);
}

static int check_fwd_args(const XattnFwdArgs* a, FwdParams& p) {
  if (!a) { set_error("null arguments"); return XATTN_E_INVALID; }
  if (a->dtype != XATTN_DTYPE_F16 && a->dtype != XATTN_DTYPE_BF16) { set_error("Q/K/V dtype must be fp16 or bf16"); return XATTN_E_INVALID; }
  if (a->batch <= 0 || a->q_len <= 0 || a->k_len <= 0 || a->q_heads <= 0 || a->kv_heads <= 0 ||
      a->q_heads % a->kv_heads != 0) { set_error("bad batch / length / head counts"); return XATTN_E_INVALID; }
  if (a->qk_dim < 8 || a->qk_dim > 256 || a->qk_dim % 8 || a->v_dim < 8 || a->v_dim > 256 || a->v_dim % 8) {
    set_error("head dimensions must be multiples of 8 in [8, 256]"); return XATTN_E_INVALID;
  }
  if (!(a->scale > 0.f) || !isfinite(a->scale)) { set_error("scale must be finite and positive"); return XATTN_E_INVALID; }
  if (!a->q || !a->k || !a->v || !a->y || !a->lse || !a->plan || !a->status) { set_error("null tensor pointer"); return XATTN_E_INVALID; }
  if ((reinterpret_cast<uintptr_t>(a->y) & 15) || (a->y_state && (reinterpret_cast<uintptr_t>(a->y_state) & 15))) {
    set_error("y must be 16-byte aligned"); return XATTN_E_INVALID;
  }
  p.B = (int)a->batch; p.Lq = (int)a->q_len; p.Lk = (int)a->k_len; p.Hq = (int)a->q_heads; p.Hkv = (int)a->kv_heads;
  p.D = (int)a->qk_dim; p.V = (int)a->v_dim;
  p.nQT = ceil_div(p.Lq, kBlockM);
  p.scale = a->scale;
  const PlanLayout pl(a->batch, a->q_len, a->k_len);
  p.row_lo = a->plan + pl.off_lo;
  p.row_hi = a->plan + pl.off_hi;
  p.q_tiles = reinterpret_cast<const TileInfo*>(a->plan + pl.off_qt);
  p.y = a->y; p.lse = a->lse; p.y_state = a->y_state; p.status = a->status;
  p.anchor = a->high_precision ? a->anchor : nullptr;
  p.splits = 1; p.g_shift = 0; p.part_y = nullptr; p.part_lse = nullptr;
  return XATTN_OK;
}

int fwd_entry(const XattnFwdArgs* a, cudaStream_t stream) {
  FwdParams p;
  const int rc = check_fwd_args(a, p);
  if (rc != XATTN_OK) return rc;
  return dispatch_fwd<false>(*a, p, stream);
}

// Decode shapes qualify when the G = Hq / Hkv heads of a group times the query rows fit one tile.
static bool split_shape_ok(int64_t q_len, int64_t q_heads, int64_t kv_heads) {
  if (q_len <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads) return false;
  const int64_t g = q_heads / kv_heads;
  return g <= kBlockM && (g & (g - 1)) == 0 && q_len * g <= kBlockM;
}

size_t fwd_split_workspace_bytes(int64_t batch, int64_t q_len, int64_t q_heads, int64_t v_dim, int64_t splits) {
  if (batch <= 0 || q_len <= 0 || q_heads <= 0 || v_dim <= 0 || splits <= 0) return 0;
  return (size_t)splits * batch * q_len * q_heads * (v_dim + 1) * sizeof(float);
}

int64_t fwd_split_suggest(int64_t batch, int64_t q_len, int64_t k_len, int64_t q_heads, int64_t kv_heads,
                          int64_t sm_count) {
  if (batch <= 0 || k_len <= 0 || sm_count <= 0 || !split_shape_ok(q_len, q_heads, kv_heads)) return 0;
  const int64_t nkt = (k_len + kBlockN - 1) / kBlockN;
  if (nkt < 4) return 0;                        // nothing to stream: the general kernel is as good
  int64_t splits = sm_count / (batch * kv_heads);  // one wave of CTAs
  if (splits > nkt / 2) splits = nkt / 2;          // at least two key tiles per CTA
  if (splits < 1) splits = 1;
  if (splits > 256) splits = 256;
  if (splits == 1 && q_heads == kv_heads) return 0;   // neither heads to share nor keys to divide
  return splits;
}

int fwd_split_entry(const XattnFwdArgs* a, int64_t splits, void* workspace, size_t workspace_bytes,
                    cudaStream_t stream) {
  FwdParams p;
  const int rc = check_fwd_args(a, p);
  if (rc != XATTN_OK) return rc;
  if (!split_shape_ok(a->q_len, a->q_heads, a->kv_heads)) {
    set_error("split forward needs q_len * (q_heads / kv_heads) <= 128 with a power-of-two group size");
    return XATTN_E_INVALID;
  }
  if (splits < 1 || splits > 256) { set_error("splits must be in [1, 256]"); return XATTN_E_INVALID; }
  const size_t need = fwd_split_workspace_bytes(a->batch, a->q_len, a->q_heads, a->v_dim, splits);
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15) || workspace_bytes < need) {
    set_error("split forward workspace must be 16-byte aligned and hold %zu bytes", need);
    return XATTN_E_INVALID;
  }
  p.splits = (int)splits;
  int g = p.Hq / p.Hkv;
  while (g > 1) { ++p.g_shift; g >>= 1; }
  p.part_y = static_cast<float*>(workspace);
  p.part_lse = p.part_y + (size_t)splits * p.B * p.Lq * p.Hq * p.V;
  return dispatch_fwd<true>(*a, p, stream);
}

}  // namespace xb
