// Shared host/device definitions for the attention kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "ptx.cuh"
#include "../../include/xattn_b200.h"

namespace xb {

constexpr int kBlockM = 128;   // query rows per tile
constexpr int kBlockN = 128;   // keys per tile

// One entry per (batch, 128-row query tile): bounds of the visible-key
// intervals of its non-empty rows.
//   x = min lo, y = max hi      -> key tiles that must be visited
//   z = max lo, w = min hi      -> key tiles inside [z, w) need no masking
// A tile whose rows are all empty has x >= y.  A tile with at least one empty
// row has z = INT_MAX so that no key tile is treated as fully visible.
struct TileInfo {
  int min_lo, max_hi, max_lo, min_hi;
};

// One entry per (batch, 128-key tile): range of 128-row query tiles that hold
// at least one row seeing a key of this tile (first, last+1); first >= last+1
// when no query sees the tile.
struct KeyTileInfo {
  int m_first, m_end;
};

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Offsets (in int32 words) of the four tables inside a plan buffer.  Each
// table starts on a 16-byte boundary.
struct PlanLayout {
  int64_t rows, nQT, nKT;
  int64_t off_lo, off_hi, off_qt, off_kt, off_ko, words;   // off_ko: key tiles of all batch rows, most work first
  __host__ __device__ PlanLayout(int64_t B, int64_t Lq, int64_t Lk) {
    rows = B * Lq;
    nQT = (Lq + kBlockM - 1) / kBlockM;
    nKT = (Lk + kBlockN - 1) / kBlockN;
    const int64_t r4 = (rows + 3) & ~int64_t(3);
    off_lo = 0;
    off_hi = r4;
    off_qt = 2 * r4;
    off_kt = off_qt + 4 * B * nQT;
    off_ko = off_kt + ((2 * B * nKT + 3) & ~int64_t(3));
    words = off_ko + ((B * nKT + 3) & ~int64_t(3));
  }
};

// ---- tensor maps -----------------------------------------------------------
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                      CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                      CUtensorMapFloatOOBfill);
TensorMapEncodeFn tensor_map_encoder();

// Map over a [B, L, H, D] tensor with element strides (sb, sl, sh, 1) of 16-bit
// elements; box = 64 elements of D x `box_heads` heads x `box_rows` rows of L (in shared memory the
// heads of one row lie next to each other), 128-byte swizzle.  Returns 0 on success.
int make_tile_map(CUtensorMap* out, const void* base, int dtype, int64_t B, int64_t L, int64_t H, int64_t D,
                  int64_t sb, int64_t sl, int64_t sh, int box_rows, int box_heads = 1);
// Tensor map over a contiguous [B][H][L][16] bf16 tensor (32-byte rows): boxes of `box_rows` rows of
// one (batch, head), written to shared memory in the 32-byte-swizzle K-major layout.
// Coordinates: (0, row, head, batch).
int make_row_map(CUtensorMap* out, const void* base, int64_t B, int64_t H, int64_t L, int box_rows);

// Last error text of this thread (set by the host entry points).
void set_error(const char* fmt, ...);

// Optional per-kernel timing: when enabled, a ProfileScope brackets the launches made
// inside it with CUDA events on the launch stream.
enum ProfileKind : int {
  kProfPlan = 1, kProfFwd = 2, kProfBwdPre = 3, kProfBwdDq = 4, kProfBwdDkv = 5, kProfGate = 6, kProfRepair = 7, kProfBwdStats = 8,
};
struct ProfileScope {
  ProfileScope(int kind, cudaStream_t stream);
  ~ProfileScope();
  int slot;
  cudaStream_t stream;
};
int profile_enable(int enable);
int profile_read(int* kinds, float* ms, int capacity);

}  // namespace xb
