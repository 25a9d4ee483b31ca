// Forward attention for sm_100a.
//
// One CTA owns NT tiles of 128 query rows of one (batch, query head) and walks
// the key tiles their visible-key intervals touch.  Roles (16 warps):
//   warps 0-3 / 4-7   softmax warpgroup of tile 0 / tile 1 (thread = row)
//   warps 8-11        correction + epilogue warpgroup (rescales O in TMEM,
//                     writes y and lse)
//   warp 12           tcgen05.mma issuer (one thread)
//   warp 13           TMA producer (one thread); also owns the TMEM allocation
// Per key tile and query tile:  S = Q K^T (operands in shared memory, S in
// TMEM) -> softmax in registers -> P (16-bit) written over S in TMEM ->
// O += P V (P from TMEM, V from shared memory, O in TMEM).  The two query
// tiles alternate on the tensor core so that one's MMAs cover the other's
// softmax.
//
// Semantics restated from the reference: online softmax in the exp2 domain
// (csrc/attention/cuda/softmax.h:124-207), rows without a visible key give
// y = 0 and lse = -inf (csrc/attention/hopper/epilogue_fwd.hpp:474-566),
// key tiles no row can see are skipped (hopper/mainloop_fwd_sm90_tma_gmma_ws.hpp:1169-1172).
#include "common.cuh"

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
  int* status;
};

template <int HD, int NT>
struct FwdSmem {
  static constexpr int kTileBytes = kBlockM * HD * 2;
  static constexpr int kStages = (HD <= 128) ? 2 : 1;
  alignas(1024) uint8_t q[NT][kTileBytes];
  alignas(1024) uint8_t k[kStages][kTileBytes];
  alignas(1024) uint8_t v[kStages][kTileBytes];
  float scale_buf[NT][2][kBlockM];   // rescale factors, double-buffered by iteration parity
  float final_l[NT][kBlockM];
  float final_m[NT][kBlockM];
  uint64_t q_full[NT];
  uint64_t k_full[kStages], k_empty[kStages];
  uint64_t v_full[kStages], v_empty[kStages];
  uint64_t s_full[NT], p_full[NT], o_ready[NT], pv_done[NT], corr_full[NT];
  uint32_t tmem_base;
  int abort_flag;
};



// T: __nv_bfloat16 or __half.  HD: padded head dimension of the shared-memory
// tiles (64, 128 or 256).  NT: query tiles per CTA.  HP: high-precision softmax.
template <typename T, int HD, int NT, bool HP>
__global__ void __launch_bounds__(512, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
           const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  using Smem = FwdSmem<HD, NT>;
  constexpr int kStages = Smem::kStages;
  constexpr int kBoxBytes = kBlockM * 64 * 2;          // one 64-column box of a tile
  constexpr uint32_t kTmemCols = 512;
  // TMEM columns: S/P of tile t at t*128; O of tile t at NT*128 + t*HD.
  constexpr int kFormat = Pack2<T>::kFormat;

  extern __shared__ uint8_t smem_raw[];
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // ---- which work item -----------------------------------------------------
  const int G = p.Hq / p.Hkv;
  const int n_groups = (p.nQT + NT - 1) / NT;     // groups of NT query tiles
  const int per_bk = n_groups * G;
  const int bk = blockIdx.x / per_bk;
  const int rem = blockIdx.x - bk * per_bk;
  const int grp = n_groups - 1 - rem / G;          // later (heavier under causal masks) groups first
  const int h = (bk % p.Hkv) * G + (rem % G);
  const int kvh = bk % p.Hkv;
  const int b = bk / p.Hkv;

  // key-tile range of each query tile
  int n_lo[NT], n_hi[NT], full_lo[NT], full_hi[NT];
  int u_lo = 0x7fffffff, u_hi = 0;
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    const int qt = grp * NT + t;
    n_lo[t] = n_hi[t] = 0;
    full_lo[t] = 0x7fffffff;
    full_hi[t] = 0;
    if (qt < p.nQT) {
      const TileInfo ti = p.q_tiles[(size_t)b * p.nQT + qt];
      if (ti.max_hi > ti.min_lo) {
        n_lo[t] = ti.min_lo / kBlockN;
        n_hi[t] = (ti.max_hi + kBlockN - 1) / kBlockN;
        full_lo[t] = ti.max_lo;
        full_hi[t] = ti.min_hi;
        u_lo = min(u_lo, n_lo[t]);
        u_hi = max(u_hi, n_hi[t]);
      }
    }
  }
  if (u_hi == 0) u_lo = 0;

  // ---- set-up ----------------------------------------------------------------
  if (tid == 0) {
    // an earlier CTA gave up: do not pile on
    s.abort_flag = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 2 : 0;
    for (int t = 0; t < NT; ++t) {
      mbar_init(&s.q_full[t], 1);
      mbar_init(&s.s_full[t], 1);
      mbar_init(&s.p_full[t], 4);
      mbar_init(&s.o_ready[t], 4);
      mbar_init(&s.pv_done[t], 1);
      mbar_init(&s.corr_full[t], 4);
    }
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&s.k_full[i], 1);
      mbar_init(&s.k_empty[i], 1);
      mbar_init(&s.v_full[i], 1);
      mbar_init(&s.v_empty[i], 1);
    }
    fence_mbar_init();
  }
  if (warp == 13) {
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
  if (dead) {
    // nothing to do
  } else if (warp < 4 * NT) {
    // =========================== softmax warpgroups ===========================
    setmaxnreg_inc<NT == 2 ? 192 : 216>();
    const int t = warp >> 2;
    const int r = tid & 127;
    const int qt = grp * NT + t;
    const int row = qt * kBlockM + r;
    int lo = 0, hi = 0;
    if (qt < p.nQT && row < p.Lq) {
      lo = p.row_lo[(size_t)b * p.Lq + row];
      hi = p.row_hi[(size_t)b * p.Lq + row];
    }
    const uint32_t t_s = tmem + ((uint32_t)((warp & 3) * 32) << 16) + t * 128;
    const float c_log2 = p.scale * 1.4426950408889634f;
    float m = -INFINITY, l = 0.f;
    const int iters = n_hi[t] - n_lo[t];
    bool ok = true;
    for (int j = 0; j < iters && ok; ++j) {
      const int col0 = (n_lo[t] + j) * kBlockN;
      ok = mbar_wait(ctx, &s.s_full[t], j & 1, 10 + t);
      if (!ok) break;
      tc_fence_after();
      float sc[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_x32(t_s + c * 32, reinterpret_cast<uint32_t*>(sc) + c * 32);
      tc_wait_ld();
      const bool tile_full = (col0 >= full_lo[t]) && (col0 + kBlockN <= full_hi[t]);
      if (!tile_full) {
        const int rl = lo - col0, rh = hi - col0;
#pragma unroll
        for (int c = 0; c < 128; ++c) sc[c] = (c >= rl && c < rh) ? sc[c] : -INFINITY;
      }
      float mxa = max3(sc[0], sc[1], sc[2]), mxb = max3(sc[3], sc[4], sc[5]);
      float mxc = max3(sc[6], sc[7], sc[8]), mxd = max3(sc[9], sc[10], sc[11]);
#pragma unroll
      for (int c = 12; c < 124; c += 8) {
        mxa = max3(mxa, sc[c], sc[c + 1]);
        mxb = max3(mxb, sc[c + 2], sc[c + 3]);
        mxc = max3(mxc, sc[c + 4], sc[c + 5]);
        mxd = max3(mxd, sc[c + 6], sc[c + 7]);
      }
      mxa = max3(mxa, sc[124], sc[125]);
      mxb = max3(mxb, sc[126], sc[127]);
      const float mx = fmaxf(fmaxf(mxa, mxb), fmaxf(mxc, mxd));
      float m_new = fmaxf(m, mx);
      if (!HP) {
        // keep the old reference while the maximum grew by less than 2^8: the
        // accumulator is then left untouched and P stays below 256
        if (m != -INFINITY && (m_new - m) * c_log2 <= 8.f) m_new = m;
      }
      float factor = 1.f;
      if (m != -INFINITY && m_new != m) factor = HP ? exp2f((m - m_new) * c_log2) : ex2_approx((m - m_new) * c_log2);
      if (j > 0) {
        s.scale_buf[t][j & 1][r] = factor;
        mbar_arrive_warp(&s.corr_full[t]);
      }
      m = m_new;
      const float m_ref = (m == -INFINITY) ? 0.f : m;
      const float neg_mc = -m_ref * c_log2;
      const uint32_t t_p = t_s;   // P overwrites the first 64 columns of S
      float sum = 0.f;
      if (HP) {
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c0 = 0; c0 < 128; c0 += 32) {
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            const float p0 = exp2f(__fmul_rn(__fsub_rn(sc[c0 + c], m_ref), c_log2));
            const float p1 = exp2f(__fmul_rn(__fsub_rn(sc[c0 + c + 1], m_ref), c_log2));
            sum4[(c >> 1) & 3] += p0 + p1;
            pk[c >> 1] = Pack2<T>::pack(p0, p1);
          }
          tmem_st_x16(t_p + (c0 >> 1), pk);
        }
        sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      } else {
        const float2 cc = make_float2(c_log2, c_log2), nm = make_float2(neg_mc, neg_mc);
        float2 s2a = make_float2(0.f, 0.f), s2b = make_float2(0.f, 0.f);
#pragma unroll
        for (int c0 = 0; c0 < 128; c0 += 32) {
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            const float2 pa = ex2_pair_sfu(fma2(make_float2(sc[c0 + c], sc[c0 + c + 1]), cc, nm));
            const float2 pb = ex2_pair_sfu(fma2(make_float2(sc[c0 + c + 2], sc[c0 + c + 3]), cc, nm));
            s2a = add2(s2a, pa);
            s2b = add2(s2b, pb);
            pk[c >> 1] = Pack2<T>::pack(pa.x, pa.y);
            pk[(c >> 1) + 1] = Pack2<T>::pack(pb.x, pb.y);
          }
          tmem_st_x16(t_p + (c0 >> 1), pk);
        }
        const float2 s2 = add2(s2a, s2b);
        sum = s2.x + s2.y;
      }
      l = l * factor + sum;
      tc_wait_st();
      tc_fence_before();
      mbar_arrive_warp(&s.p_full[t]);
    }
    // hand the row statistics to the epilogue
    s.final_l[t][r] = l;
    s.final_m[t][r] = m;
    mbar_arrive_warp(&s.corr_full[t]);
  } else if (warp < 4 * NT + 4) {
    // ======================= correction + epilogue warpgroup =======================
    // launch allocation is 128 registers per thread: shrink below it, grow above it
    if (NT == 2) setmaxnreg_dec<80>(); else setmaxnreg_inc<152>();
    const int r = tid & 127;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    bool ok = true;
    for (int n = u_lo; n < u_hi && ok; ++n) {
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        if (n < n_lo[t] || n >= n_hi[t]) continue;
        const int j = n - n_lo[t];
        if (j == 0) continue;
        ok = mbar_wait(ctx, &s.corr_full[t], (j - 1) & 1, 20 + t);
        if (!ok) break;
        const float f = s.scale_buf[t][j & 1][r];
        ok = mbar_wait(ctx, &s.pv_done[t], (j - 1) & 1, 22 + t);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, f != 1.f)) {
          const uint32_t t_o = tmem + lane_off + NT * 128 + t * HD;
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
        mbar_arrive_warp(&s.o_ready[t]);
      }
    }
    // epilogue: y = O / l, lse = ln2 * (m * c + log2 l)
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      if (!ok) break;
      const int qt = grp * NT + t;
      const int iters = n_hi[t] - n_lo[t];
      // final statistics are arrival number `max(iters,1) - 1` on corr_full[t]
      const int arrivals_before = iters > 0 ? iters - 1 : 0;
      ok = mbar_wait(ctx, &s.corr_full[t], arrivals_before & 1, 24 + t);
      if (!ok) break;
      if (iters > 0) {
        ok = mbar_wait(ctx, &s.pv_done[t], (iters - 1) & 1, 26 + t);
        if (!ok) break;
      }
      tc_fence_after();
      const int row = qt * kBlockM + r;
      const float l = s.final_l[t][r];
      const float m = s.final_m[t][r];
      const bool live = (qt < p.nQT) && (row < p.Lq);
      const bool has = l > 0.f && iters > 0;
      float inv = 0.f;
      if (has) inv = HP ? __frcp_rn(l) : __fdividef(1.f, l);
      if (live) {
        const float c_log2 = p.scale * 1.4426950408889634f;
        p.lse[((size_t)b * p.Hq + h) * p.Lq + row] =
            has ? (m * c_log2 + log2f(l)) * 0.6931471805599453f : -INFINITY;
      }
      const uint32_t t_o = tmem + lane_off + NT * 128 + t * HD;
      T* y_row = reinterpret_cast<T*>(p.y) + (((size_t)b * p.Lq + (live ? row : 0)) * p.Hq + h) * p.V;
      float* ys_row = p.y_state ? p.y_state + (((size_t)b * p.Lq + (live ? row : 0)) * p.Hq + h) * p.V : nullptr;
      for (int c0 = 0; c0 < v_pad; c0 += 32) {
        uint32_t o[32];
        if (iters > 0) {
          tmem_ld_x32(t_o + c0, o);   // warp-collective: executed by all lanes
          tc_wait_ld();
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] = 0u;
        }
        if (live) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            if (c0 + c < p.V) {
              uint4 pk;
              pk.x = Pack2<T>::pack(__uint_as_float(o[c + 0]) * inv, __uint_as_float(o[c + 1]) * inv);
              pk.y = Pack2<T>::pack(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
              pk.z = Pack2<T>::pack(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
              pk.w = Pack2<T>::pack(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
              *reinterpret_cast<uint4*>(y_row + c0 + c) = pk;
              if (ys_row) {
                float4 a = make_float4(__uint_as_float(o[c + 0]) * inv, __uint_as_float(o[c + 1]) * inv,
                                       __uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
                float4 bq = make_float4(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv,
                                        __uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
                *reinterpret_cast<float4*>(ys_row + c0 + c) = a;
                *reinterpret_cast<float4*>(ys_row + c0 + c + 4) = bq;
              }
            }
          }
        }
      }
    }
  } else {
    // ============================ MMA issuer / TMA producer ============================
    setmaxnreg_dec<48>();
    if (warp == 4 * NT + 4 && lane == 0) {
      // ------------------------------ MMA issuer ------------------------------
      const uint32_t idesc_qk = make_idesc(kBlockM, kBlockN, kFormat, 0, 0);
      const uint32_t idesc_pv = make_idesc(kBlockM, v_pad, kFormat, 0, 1);
      bool ok = true;
      auto issue_qk = [&](int t, int stage) {
        const uint32_t qa = smem_u32(s.q[t]);
        const uint32_t ka = smem_u32(s.k[stage]);
        const uint32_t d = tmem + t * 128;
        for (int js = 0; js < ksteps_qk; ++js) {
          const uint32_t off = (js >> 2) * kBoxBytes + (js & 3) * 32;
          umma_ss(d, make_smem_desc(qa + off, 16, 1024), make_smem_desc(ka + off, 16, 1024), idesc_qk, js > 0);
        }
        umma_commit(&s.s_full[t]);
      };
      auto issue_pv = [&](int t, int stage, bool accumulate) {
        const uint32_t va = smem_u32(s.v[stage]);
        const uint32_t d = tmem + NT * 128 + t * HD;
        const uint32_t pa = tmem + t * 128;
#pragma unroll
        for (int js = 0; js < kBlockN / 16; ++js) {
          umma_ts(d, pa + js * 8, make_smem_desc(va + js * 2048, kBoxBytes, 1024), idesc_pv,
                  (accumulate || js > 0) ? 1u : 0u);
        }
        umma_commit(&s.pv_done[t]);
      };
      if (u_hi > u_lo) {
        // prologue: S for the first key tile
        ok = mbar_wait(ctx, &s.k_full[0], 0, 30);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          if (ok && u_lo >= n_lo[t] && u_lo < n_hi[t]) {
            ok = mbar_wait(ctx, &s.q_full[t], 0, 31);
            if (ok) { tc_fence_after(); issue_qk(t, 0); }
          }
        }
        if (ok) umma_commit(&s.k_empty[0]);
        for (int n = u_lo; n < u_hi && ok; ++n) {
          const int i = n - u_lo;
          const int st = i % kStages;
          const int st_next = (i + 1) % kStages;
          bool v_waited = false, k_waited = false;
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            if (!ok) break;
            if (n >= n_lo[t] && n < n_hi[t]) {
              const int j = n - n_lo[t];
              if (!v_waited) { ok = mbar_wait(ctx, &s.v_full[st], (i / kStages) & 1, 32); v_waited = true; }
              if (ok) ok = mbar_wait(ctx, &s.p_full[t], j & 1, 33);
              if (ok && j > 0) ok = mbar_wait(ctx, &s.o_ready[t], (j - 1) & 1, 34);
              if (!ok) break;
              tc_fence_after();
              issue_pv(t, st, j > 0);
            }
            if (n + 1 < u_hi && n + 1 >= n_lo[t] && n + 1 < n_hi[t]) {
              if (!k_waited) { ok = mbar_wait(ctx, &s.k_full[st_next], ((i + 1) / kStages) & 1, 35); k_waited = true; }
              if (ok && n + 1 == n_lo[t]) ok = mbar_wait(ctx, &s.q_full[t], 0, 36);
              if (!ok) break;
              tc_fence_after();
              issue_qk(t, st_next);
            }
          }
          if (!ok) break;
          // stages are released when every MMA issued so far has finished; a
          // stage no tile used still has to be waited for before its release
          if (!v_waited) ok = mbar_wait(ctx, &s.v_full[st], (i / kStages) & 1, 37);
          if (ok) umma_commit(&s.v_empty[st]);
          if (ok && n + 1 < u_hi) {
            if (!k_waited) ok = mbar_wait(ctx, &s.k_full[st_next], ((i + 1) / kStages) & 1, 38);
            if (ok) umma_commit(&s.k_empty[st_next]);
          }
        }
      }
    } else if (warp == 4 * NT + 5 && lane == 0) {
      // ------------------------------ TMA producer ------------------------------
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      bool ok = true;
      auto load_k = [&](int n, int stage) {
        mbar_arrive_expect_tx(&s.k_full[stage], nbox_qk * kBoxBytes);
        for (int bx = 0; bx < nbox_qk; ++bx)
          tma_load_4d(s.k[stage] + bx * kBoxBytes, &tm_k, &s.k_full[stage], bx * 64, kvh, n * kBlockN, b);
      };
      auto load_v = [&](int n, int stage) {
        mbar_arrive_expect_tx(&s.v_full[stage], nbox_v * kBoxBytes);
        for (int bx = 0; bx < nbox_v; ++bx)
          tma_load_4d(s.v[stage] + bx * kBoxBytes, &tm_v, &s.v_full[stage], bx * 64, kvh, n * kBlockN, b);
      };
      if (u_hi > u_lo) {
        // first K tile, then the query tiles, then the rest of the stream
        load_k(u_lo, 0);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          if (n_hi[t] > n_lo[t]) {
            mbar_arrive_expect_tx(&s.q_full[t], nbox_qk * kBoxBytes);
            for (int bx = 0; bx < nbox_qk; ++bx)
              tma_load_4d(s.q[t] + bx * kBoxBytes, &tm_q, &s.q_full[t], bx * 64, h, (grp * NT + t) * kBlockM, b);
          }
        }
        for (int n = u_lo; n < u_hi && ok; ++n) {
          const int i = n - u_lo;
          const int st = i % kStages;
          if (i > 0) {
            if (i >= kStages) ok = mbar_wait(ctx, &s.k_empty[st], ((i / kStages) - 1) & 1, 40);
            if (!ok) break;
            load_k(n, st);
          }
          if (i >= kStages) ok = mbar_wait(ctx, &s.v_empty[st], ((i / kStages) - 1) & 1, 41);
          if (!ok) break;
          load_v(n, st);
        }
      }
    }
  }

  // ---- tail -----------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (s.abort_flag == 1) {
    // give bulk copies still in flight time to land before the CTA retires
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { }
    __syncthreads();
  }
  if (warp == 13) {
    __syncwarp();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
template <typename T, int HD, int NT, bool HP>
static int launch_fwd(const XattnFwdArgs& a, const FwdParams& p, cudaStream_t stream) {
  using Smem = FwdSmem<HD, NT>;
  CUtensorMap tq, tk, tv;
  if (make_tile_map(&tq, a.q, a.dtype, a.batch, a.q_len, a.q_heads, a.qk_dim, a.q_strides[0], a.q_strides[1],
                    a.q_strides[2], kBlockM)) return XATTN_E_INVALID;
  if (make_tile_map(&tk, a.k, a.dtype, a.batch, a.k_len, a.kv_heads, a.qk_dim, a.k_strides[0], a.k_strides[1],
                    a.k_strides[2], kBlockN)) return XATTN_E_INVALID;
  if (make_tile_map(&tv, a.v, a.dtype, a.batch, a.k_len, a.kv_heads, a.v_dim, a.v_strides[0], a.v_strides[1],
                    a.v_strides[2], kBlockN)) return XATTN_E_INVALID;
  const size_t smem = sizeof(Smem) + 1024;
  auto kern = fwd_kernel<T, HD, NT, HP>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_error("cudaFuncSetAttribute(fwd): %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  const int n_groups = (p.nQT + NT - 1) / NT;
  const long long grid = (long long)n_groups * p.Hq * p.B;
  if (grid <= 0 || grid > 0x7fffffffLL) { set_error("forward grid out of range"); return XATTN_E_INVALID; }
  {
    ProfileScope prof(kProfFwd, stream);
    kern<<<(unsigned)grid, 512, smem, stream>>>(tq, tk, tv, p);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("forward launch: %s", cudaGetErrorString(e)); return XATTN_E_CUDA; }
  return XATTN_OK;
}

template <typename T, bool HP>
static int dispatch_fwd_dim(const XattnFwdArgs& a, const FwdParams& p, cudaStream_t stream) {
  const int hd = (int)(a.qk_dim > a.v_dim ? a.qk_dim : a.v_dim);
  if (hd <= 64) return launch_fwd<T, 64, 2, HP>(a, p, stream);
  if (hd <= 128) return launch_fwd<T, 128, 2, HP>(a, p, stream);
  return launch_fwd<T, 256, 1, HP>(a, p, stream);
}


int fwd_entry(const XattnFwdArgs* a, cudaStream_t stream) {
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
  FwdParams p;
  p.B = (int)a->batch; p.Lq = (int)a->q_len; p.Lk = (int)a->k_len; p.Hq = (int)a->q_heads; p.Hkv = (int)a->kv_heads;
  p.D = (int)a->qk_dim; p.V = (int)a->v_dim;
  p.nQT = ceil_div(p.Lq, kBlockM);
  p.scale = a->scale;
  const PlanLayout pl(a->batch, a->q_len, a->k_len);
  p.row_lo = a->plan + pl.off_lo;
  p.row_hi = a->plan + pl.off_hi;
  p.q_tiles = reinterpret_cast<const TileInfo*>(a->plan + pl.off_qt);
  p.y = a->y; p.lse = a->lse; p.y_state = a->y_state; p.status = a->status;
  if (a->dtype == XATTN_DTYPE_BF16) {
    return a->high_precision ? dispatch_fwd_dim<__nv_bfloat16, true>(*a, p, stream)
                             : dispatch_fwd_dim<__nv_bfloat16, false>(*a, p, stream);
  }
  return a->high_precision ? dispatch_fwd_dim<__half, true>(*a, p, stream)
                           : dispatch_fwd_dim<__half, false>(*a, p, stream);
}

}  // namespace xb
