/* C ABI of libxattn_b200: Blackwell (sm_100a) attention kernels behind the
 * operator table of ifm-ai/xattn.
 *
 * The reference reaches its native code through a pybind module whose ops take
 * and return torch tensors (csrc/xattn_extension.cc:9-20, csrc/bindings.h:11-15).
 * This header is the replacement boundary: plain pointers, sizes, element
 * strides and a CUDA stream; no torch types.  Every pointer is a DEVICE pointer
 * unless the comment says otherwise.  The callee never allocates: outputs and
 * workspaces are provided by the caller (the reference allocates outputs inside
 * the op, csrc/causal_attention/launch.cu:1099-1105; here the Python shim does).
 *
 * Every entry point returns 0 on success and a negative XATTN_E_* code on
 * failure; xattn_b200_last_error() gives the message for the calling thread.
 * Kernels never trap: a device-side wait that runs out of time stores a code
 * in the caller's `status` word (checked with xattn_b200_check_status()).
 */
#ifndef XATTN_B200_H_
#define XATTN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XATTN_B200_ABI_VERSION 2

enum {
  XATTN_OK = 0,
  XATTN_E_INVALID = -1,      /* bad argument (shape, alignment, dtype)      */
  XATTN_E_UNSUPPORTED = -2,  /* valid request this build cannot run         */
  XATTN_E_CUDA = -3,         /* a CUDA runtime / driver call failed         */
  XATTN_E_DEVICE = -4        /* a kernel reported a device-side status code */
};

enum { XATTN_DTYPE_F16 = 0, XATTN_DTYPE_BF16 = 1 };

/* Visibility of keys to the left of a query (tests/_reference.py:50-59,
 * csrc/attention/hopper/semantics/visibility.h:17-180). */
enum { XATTN_VIS_FULL = 0, XATTN_VIS_WINDOW = 1, XATTN_VIS_CHUNK = 2,
       /* every key of the query's segment, later ones too: the off-diagonal blocks of ring attention
          (no counterpart in the reference, which has no non-causal mode) */
       XATTN_VIS_ALL = 3 };

typedef void* xattn_stream_t; /* cudaStream_t */

int xattn_b200_abi_version(void);
const char* xattn_b200_last_error(void);

/* ------------------------------------------------------------------------
 * Mask plan.  Every variant of the reference (causal / window / chunk,
 * segment ids, BOS runs, per-segment reset positions, strict past, short
 * right-aligned Q, packed varlen) makes the keys visible to one query row a
 * single interval [lo, hi) of key indices.  The plan stores that interval per
 * (batch, query row) plus per-tile summaries the kernels use to pick and skip
 * key tiles.  It replaces csrc/attention/hopper/mask.h:197-442,563-713,
 * hopper/block.h:17-179, csrc/attention/partition/segment_index.h:113-391 and
 * the pre-pass kernels of hopper/fwd_template.cuh:186-202 and
 * hopper/bwd_template.cuh:115-239.
 *
 * Layout of the plan buffer (int32 words), with nQT = ceil(Lq/128),
 * nKT = ceil(Lk/128):
 *   row_lo   [B][Lq]
 *   row_hi   [B][Lq]
 *   q_tiles  [B][nQT][4]   (min lo, max hi, max lo, min hi)
 *   k_tiles  [B][nKT][2]   (first query tile, last query tile + 1)
 *   k_order  [B * nKT]     key tiles of all batch rows (b * nKT + tile), those seen by the most
 *                          query tiles first: the launch order of the dK / dV kernel
 * (each section padded to a multiple of 4 words)
 * ---------------------------------------------------------------------- */
size_t xattn_b200_plan_bytes(int64_t batch, int64_t q_len, int64_t k_len);

typedef struct {
  int64_t batch, q_len, k_len;   /* k_len counts previous K/V too              */
  int visibility;                /* XATTN_VIS_*                                */
  int64_t span;                  /* window radius / chunk size                 */
  int strict_past;               /* 1: key position < query position           */
  int reset_positions;           /* 1: positions restart per segment run       */
  const int64_t* q_segment;      /* [B][q_len] or NULL (ids nondecreasing in k)*/
  const int64_t* k_segment;      /* [B][k_len] or NULL                         */
  int64_t q_segment_stride;      /* elements between batch rows                */
  int64_t k_segment_stride;
  int32_t* plan;                 /* xattn_b200_plan_bytes() bytes              */
  int32_t* status;               /* optional status word.  Key ids must never decrease along a row
                                    (the contract of csrc/attention/partition/segment_index.h:362-363:
                                    the keys of one id are found by binary search).  When given, the
                                    plan kernels also compare neighbouring key ids (one more pass
                                    over k_segment) and store (batch row << 8) | 3 on a decrease;
                                    NULL skips the check                        */
} XattnPlanArgs;

/* Builds the plan for dense [B, L, H, D] inputs.
 * Replaces AttentionSegmentFwdSpanKernel (hopper/fwd_template.cuh:186-202),
 * the worklist / interval kernels (hopper/bwd_template.cuh:115-239) and
 * FlashSCABuildDenseResetChunkPositionsKernel
 * (csrc/flash_sca/hopper/sliding_chunk_attention.cu:1942-1965). */
int xattn_b200_build_plan(const XattnPlanArgs* args, xattn_stream_t stream);

typedef struct {
  int64_t total_q, total_k;      /* packed token counts                        */
  int64_t num_q_seqs, num_k_seqs;/* cu_seqlens lengths minus one               */
  const int32_t* cu_seqlens_q;   /* [num_q_seqs + 1]                           */
  const int32_t* cu_seqlens_k;   /* [num_k_seqs + 1]                           */
  int visibility;
  int64_t span;
  int strict_past;
  int32_t* plan;                 /* plan_bytes(1, total_q, total_k)            */
} XattnVarlenPlanArgs;

/* Builds the plan for packed [T, H, D] inputs: sequence r of Q is paired with
 * sequence r + (num_k_seqs - num_q_seqs) of K, right-aligned, positions restart
 * per sequence (csrc/attention/sequence/varlen_metadata.h:17-69,
 * csrc/causal_attention/launch.cu:1455-1695). */
int xattn_b200_build_varlen_plan(const XattnVarlenPlanArgs* args, xattn_stream_t stream);

/* ------------------------------------------------------------------------
 * Forward.  Replaces causal_flash_attn_fwd / flash_swa_fwd / flash_sca_fwd and
 * their strict-past, component and varlen forms
 * (csrc/causal_flash_attn/causal_flash_attn.cc:49-122, csrc/flash_swa/flash_swa.cc:106-178,
 * csrc/flash_sca/sliding_chunk_attention.cc:531-902) — one kernel, the variant
 * is in the plan.  Launch contract follows AttentionFwdParams
 * (csrc/attention/hopper/fwd_params.h:10-87).
 * ---------------------------------------------------------------------- */
typedef struct {
  int dtype;                     /* XATTN_DTYPE_*                              */
  int64_t batch, q_len, k_len;
  int64_t q_heads, kv_heads;
  int64_t qk_dim, v_dim;         /* multiples of 8, <= 256                     */
  const void* q;                 /* [B][q_len][Hq][D]  element strides below   */
  const void* k;                 /* [B][k_len][Hkv][D]                         */
  const void* v;                 /* [B][k_len][Hkv][V]                         */
  int64_t q_strides[3];          /* batch, row, head (last dim contiguous)     */
  int64_t k_strides[3];
  int64_t v_strides[3];
  float scale;                   /* > 0                                        */
  int high_precision;            /* 1: subtract-before-scale softmax, exact
                                    reciprocal (hopper/fwd_template.cuh:228-239,
                                    cuda/softmax.h:103-111)                    */
  const int32_t* plan;
  void* y;                       /* [B][q_len][Hq][V] contiguous, input dtype  */
  float* lse;                    /* [B][Hq][q_len]                             */
  float* y_state;                /* optional FP32 copy of y, same shape, or NULL */
  int32_t* status;               /* one word, zero on entry                    */
  int32_t* anchor;               /* optional, high_precision only: [B][Hq][q_len], the visible key with
                                    the row's largest logit (the first of equals; -1 for a row without
                                    keys) — the anchor of the reference's row statistics
                                    (csrc/attention/precision/row_statistics_sm90.cuh:144-186), which
                                    the high-precision backward centres dP on          */
} XattnFwdArgs;

int xattn_b200_fwd(const XattnFwdArgs* args, xattn_stream_t stream);

/* Forward for decode shapes: q_len * (q_heads / kv_heads) <= 128 with a power-of-two group size (one
 * new token, or a few speculative ones, against a long key cache; the reference routes these through
 * its packed route, xattn/ops/_bos_routing_heuristics.py:52-66, and the split scheduler of
 * csrc/attention/hopper/tile_scheduler.hpp:55-101).  The query heads of a KV group share one tile, so K
 * and V are read once per KV head, and the key tiles of a row are divided among `splits` CTAs whose
 * normalised FP32 partial results (with their lse) a second kernel merges in split order.  Same
 * arguments and results as xattn_b200_fwd; HBM-bound (K and V are streamed once).
 *   xattn_b200_fwd_split_suggest  splits that fill `sm_count` SMs with one wave of CTAs, or 0 when the
 *                                 shape does not qualify or xattn_b200_fwd is as good (short keys)
 *   workspace                     splits * B * q_len * Hq * (V + 1) floats, 16-byte aligned        */
int64_t xattn_b200_fwd_split_suggest(int64_t batch, int64_t q_len, int64_t k_len, int64_t q_heads,
                                     int64_t kv_heads, int64_t sm_count);
size_t xattn_b200_fwd_split_workspace_bytes(int64_t batch, int64_t q_len, int64_t q_heads, int64_t v_dim,
                                            int64_t splits);
int xattn_b200_fwd_split(const XattnFwdArgs* args, int64_t splits, void* workspace, size_t workspace_bytes,
                         xattn_stream_t stream);

/* ------------------------------------------------------------------------
 * Backward.  Replaces causal_flash_attn_bwd / flash_swa_bwd / flash_sca_bwd and
 * their strict-past, component and varlen forms (same files as the forward
 * ops) and the kernels behind them: preprocess
 * (csrc/attention/hopper/bwd_preprocess_kernel.h:23), main loop
 * (hopper/mainloop_bwd_sm90_tma_gmma_ws.hpp:1725-2149), dQ post-process and
 * grouped dK/dV cast (hopper/bwd_postprocess_kernel.h, hopper/bwd_template.cuh:241-308).
 * Launch contract follows AttentionBwdParams (hopper/bwd_params.h:14-120).
 * Gradients are bitwise repeatable (no atomics), so the reference's
 * `deterministic` switch has nothing to select.
 * ---------------------------------------------------------------------- */
typedef struct {
  int dtype;
  int64_t batch, q_len, k_len;
  int64_t q_heads, kv_heads;
  int64_t qk_dim, v_dim;         /* multiples of 8, <= 256                      */
  const void* q;                 /* as in the forward                          */
  const void* k;
  const void* v;
  const void* y;                 /* forward output [B][q_len][Hq][V]           */
  const void* dy;                /* gradient of y, same shape                  */
  int64_t q_strides[3];
  int64_t k_strides[3];
  int64_t v_strides[3];
  int64_t y_strides[3];
  int64_t dy_strides[3];
  const float* lse;              /* [B][Hq][q_len] from the forward            */
  float scale;
  const int32_t* plan;
  void* dq;                      /* [B][q_len][Hq][D] contiguous               */
  void* dk;                      /* [B][k_len][Hkv][D] contiguous              */
  void* dv;                      /* [B][k_len][Hkv][V] contiguous              */
  float* workspace;              /* xattn_b200_bwd_workspace_bytes() bytes     */
  int32_t* status;
  int high_precision;            /* 1: the anchored backward (below); y is not read then */
  const int32_t* anchor;         /* high_precision: [B][Hq][q_len] from the forward */
  const float* grad_unscale;     /* optional device scalar multiplied into dq, dk and dv before they are
                                    rounded (undoes a power-of-two prescale of dy, the reference's
                                    xattn/ops/_precision_backend.py:203-225), or NULL  */
  int phases;                    /* 0: the whole backward.  Else a set of XATTN_BWD_PHASE_* bits: the
                                    call runs only those kernels.  For a caller that wants dK / dV
                                    before dQ (sequence sharding sends the halo's dK / dV to the
                                    previous GPU while the dQ kernel runs): first PRE | DKV, then DQ,
                                    with the same arguments and workspace.  PRE (the row statistics)
                                    must have run before DQ or DKV.  No counterpart in the reference,
                                    a single-GPU library whose backward is one launch sequence        */
} XattnBwdArgs;

enum { XATTN_BWD_PHASE_PRE = 1, XATTN_BWD_PHASE_DQ = 2, XATTN_BWD_PHASE_DKV = 4 };

/* With high_precision = 1 the backward restates the reference's precision pipeline
 * (xattn/ops/_precision_backend.py:29-170) on this library's kernels: `lse` and `anchor` must come
 * from the high-precision forward on the same inputs; dP is centred on each row's anchor key
 * (dP_ia = dO_i . V_a, computed directly), a statistics pass computes
 * Delta_i = sum_j P_ij (dP_ij - dP_ia) (csrc/attention/precision/row_statistics_sm90.cuh:39-188), and both
 * mainloops use dS_ij = P_ij ((dP_ij - dP_ia) - Delta_i) with P = root * root,
 * root = exp2((s_ij c - lse2) / 2), so that a probability below the FP32 normal range still meets a
 * huge dP correctly, and with the centred value exactly zero on the anchor.  P and dS enter the
 * dV / dK / dQ products as two 16-bit parts, hi + lo (hopper/mainloop_bwd_sm90_tma_gmma_ws.hpp:1811-1868).
 * The workspace needs xattn_b200_bwd_workspace_bytes_hp() bytes.  Not reproduced: the FP64 row sums
 * of the operands as fed, with zero-sum and probability repair (csrc/attention/precision/zero_sum_repair.cu,
 * probability_repair.cu): rows sum to zero up to the rounding of their (16-bit-accurate) terms. */
size_t xattn_b200_bwd_workspace_bytes(int64_t batch, int64_t q_heads, int64_t q_len);
size_t xattn_b200_bwd_workspace_bytes_hp(int64_t batch, int64_t q_heads, int64_t q_len);
int xattn_b200_bwd(const XattnBwdArgs* args, xattn_stream_t stream);

/* The same backward for callers that may not allocate device memory (no counterpart in the
 * reference, whose ops allocate their workspaces themselves): a plugin host that owns the device
 * arena, or a serving loop that cannot afford the device-wide stall of a cudaMalloc.  `workspace`
 * in the arguments is ignored; the scratch lives in a fixed 40 MiB array inside the library that
 * every GPU loading it keeps until exit.  Limit: batch * q_heads * q_len', with q_len' = q_len
 * rounded up to a multiple of 128, at most 1048576; larger problems return XATTN_E_INVALID.  Nothing is allocated or freed on any path.  All calls on a
 * device share the array: nothing needs clearing between calls, but calls whose kernels overlap
 * on the GPU race, so serialise them.  The first call on a device looks up the array's address;
 * make it outside any stream capture. */
int xattn_b200_bwd_static_scratch(const XattnBwdArgs* args, xattn_stream_t stream);

/* ------------------------------------------------------------------------
 * SoftDelta gate (HBM-bound).  Replaces _softdelta_gate_fwd, _softdelta_gate_restore
 * and _softdelta_gate_bwd (csrc/softdelta/bindings.cc:11-53, csrc/softdelta/gate.cu:559-627)
 * and the gate part of SoftDeltaBwdPreprocessKernel (csrc/softdelta/preprocess.cu:110-265).
 * All tensors contiguous; `rows` = batch * tokens.
 *   forward :  y[rows][H][V]   = read - sigmoid(g) * neg_read           (y may alias read)
 *   backward:  read            = y + sigmoid(g) * neg_read               (recovered query read)
 *              dneg_read[rows][Hkv][V] = - sum over the group of sigmoid(g) * dy
 *              dg[rows][H]     = - sigmoid'(g) * <dy, neg_read>
 * With value_groups = C > 1 (the reference's internal value-group layout,
 * xattn/ops/softdelta_attention.py `_SoftDeltaFunc`, v [B, L, Hkv, C, Dg], g [B, Lq, H, C, 1]) there is
 * one gate per group of v_dim / C consecutive channels: g and dg are [rows][H][C] and each group's
 * dg takes its own share of <dy, neg_read>.
 * ---------------------------------------------------------------------- */
typedef struct {
  int dtype;
  int neg_is_f32;                /* neg_read is FP32 (level 1) instead of dtype */
  int64_t rows, q_heads, kv_heads, v_dim;
  const void* g;                 /* [rows][H] gate logits, dtype               */
  const void* neg_read;          /* [rows][Hkv][V]                             */
  void* read;                    /* forward: input; backward: output           */
  void* y;                       /* forward: output; backward: input           */
  const void* dy;                /* backward only                              */
  void* dneg_read;               /* backward only, dtype                       */
  void* dg;                      /* backward only, dtype                       */
  int64_t value_groups;          /* 0 or 1: one gate per head; C > 1 must divide v_dim */
} XattnGateArgs;

int xattn_b200_softdelta_gate_fwd(const XattnGateArgs* args, xattn_stream_t stream);
int xattn_b200_softdelta_gate_bwd(const XattnGateArgs* args, xattn_stream_t stream);

/* Level-1 repair: zero the dQ rows whose visible keys are all one vector
 * (replaces _attention_precision_key_runs / _attention_precision_enforce_constant_keys,
 * csrc/attention/precision/bindings.cc:12-24).  `workspace`: batch*kv_heads*k_len int32. */
typedef struct {
  int dtype;
  int64_t batch, q_len, k_len, q_heads, kv_heads, qk_dim;
  void* dq;                      /* [B][q_len][Hq][D] contiguous, updated in place */
  const void* k;                 /* total keys, element strides below          */
  int64_t k_strides[3];
  const int32_t* plan;
  int32_t* workspace;
} XattnConstantKeyArgs;

int xattn_b200_zero_constant_key_rows(const XattnConstantKeyArgs* args, xattn_stream_t stream);

/* SoftDelta backward: the dK (or dV) of the query read and of the strict-past read, and optionally the
 * gradient of the aligned keys used as k_read, summed in FP32 and rounded once
 * (replaces _softdelta_merge_gradients, csrc/softdelta/bindings.cc:25,
 * xattn/ops/softdelta_attention.py:506-516).  out = a + b, plus `tail` on the last tail_len rows of
 * every batch row.  All tensors contiguous in the input dtype; `out` may be `a`. */
typedef struct {
  int dtype;
  int64_t batch, k_len, kv_heads, dim;   /* a, b, out: [B][k_len][Hkv][dim], dim a multiple of 8 */
  const void* a;
  const void* b;
  const void* tail;              /* [B][tail_len][Hkv][dim] or NULL            */
  int64_t tail_len;              /* <= k_len                                   */
  void* out;
} XattnMergeArgs;

int xattn_b200_softdelta_merge_gradients(const XattnMergeArgs* args, xattn_stream_t stream);

/* Ring attention across GPUs (no counterpart in the reference, a single-GPU library): folds the
 * normalised FP32 partial output of one K/V block, with its lse, into the running result, in place:
 *   new = log(exp(lse_acc) + exp(lse_part)),  y_acc = y_acc exp(lse_acc - new) + y_part exp(lse_part - new).
 * The partial result covers query rows [row_offset, row_offset + rows) of the accumulated one.
 * y: [B][rows][H][V] FP32 (the forward's `y_state`), lse: [B][H][rows] FP32; v_dim a multiple of 4. */
typedef struct {
  int64_t batch, rows, heads, v_dim;
  int64_t acc_rows, row_offset;  /* rows of the accumulated result; where the partial one starts */
  float* y_acc;                  /* [B][acc_rows][H][V], updated in place      */
  float* lse_acc;                /* [B][H][acc_rows], updated in place         */
  const float* y_part;           /* [B][rows][H][V]                            */
  const float* lse_part;         /* [B][H][rows]                               */
} XattnMergeOutputsArgs;

int xattn_b200_merge_partial_outputs(const XattnMergeOutputsArgs* args, xattn_stream_t stream);

/* Per-kernel timing for benchmarks (no counterpart in the reference, whose benchmark tool times
 * whole ops from Python, tests/_benchmark.py:22-35).  While enabled, every entry point brackets
 * its kernels with CUDA events on the launch stream.  xattn_b200_profile_read() synchronises
 * those events, writes (kind, milliseconds) pairs and clears the log; it returns the number of
 * records written.  Kinds: 1 plan, 2 forward, 3 backward preprocess, 4 backward dQ,
 * 5 backward dK/dV, 6 SoftDelta gate, 7 constant-key repair, 8 high-precision row statistics. */
int xattn_b200_profile_enable(int enable);
int xattn_b200_profile_read(int* kinds, float* ms, int capacity);

/* Self-test of the bounded device-side wait (no counterpart in the reference, whose kernels wait
 * without a limit): launches one small CTA that waits on a barrier nothing completes, for at most
 * `budget_us` microseconds (1 .. 100000), and then stores (99 << 8) | 1 in `status`, the code every
 * kernel of this library reports when one of its waits runs out.  Nothing faults or hangs; the
 * context stays usable.  `status` must be zero on entry. */
int xattn_b200_selftest_wait_timeout(int32_t* status, int64_t budget_us, xattn_stream_t stream);

/* Reads `status` back (synchronises the stream).  0 when the word is zero. */
int xattn_b200_check_status(const int32_t* status, xattn_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* XATTN_B200_H_ */
