// Host-side helpers shared by the C-ABI entry points: error reporting, TMA
// tensor-map construction through the driver entry point (the library does not
// link libcuda), per-device immutable properties.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/logo_b200.h"

namespace logo {

// Records a message retrievable through logo_last_error() and returns `code`.
int set_error(int code, const char* fmt, ...);

#define LOGO_CHECK_CUDA(expr)                                                                      \
  do {                                                                                             \
    cudaError_t _e = (expr);                                                                       \
    if (_e != cudaSuccess)                                                                         \
      return ::logo::set_error(LOGO_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e));   \
  } while (0)

#define LOGO_REQUIRE(cond, code, ...)                      \
  do {                                                     \
    if (!(cond)) return ::logo::set_error(code, __VA_ARGS__); \
  } while (0)

// 2-D bf16 tensor map with 128-byte (default) or 32-byte swizzle. `inner` elements are contiguous,
// `outer` rows are `row_stride_bytes` apart. Box = box_inner x box_outer elements;
// box_inner must be 64 (128 bytes) for the 128-byte swizzle, 16 (32 bytes) for the 32-byte one.
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle_bytes = 128);

// 2-D fp32 tensor map without swizzle (rows of `box_inner` floats lie contiguously in shared
// memory): the destination of the bulk reductions that accumulate dQ.
int make_tmap_2d_f32(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                     uint32_t box_inner, uint32_t box_outer);

// Number of SMs of the current device (cached per device).
int sm_count();

// Zeroes the rows of a [n_tokens, row_bytes] tensor that are NOT listed in the ascending index list
// q_idx[0 .. *sq_ptr): the gaps between consecutive selected tokens, before the first and after the
// last. Replaces a memset of the whole tensor (whose selected rows are overwritten anyway).
// row_bytes must be a multiple of 16 and `base` 16-byte aligned.
int launch_zero_unselected_rows(void* base, const int64_t* q_idx, const int32_t* sq_ptr, int n_tokens,
                                size_t row_bytes, cudaStream_t stream);

#ifdef __CUDACC__
// The device side of it, for one warp that is number `part` of `n_parts` warps sharing the job: each
// warp takes runs of 32 consecutive tokens; a binary search finds the first selected token at or after
// the run's start, the next 32 entries of q_idx (one per lane) mark which tokens of the run are
// selected, and the warp zeroes the rows (row_chunks 16-byte pieces each) of the others. Work is
// balanced whatever the selection looks like (an empty selection zeroes everything with all warps).
__device__ __forceinline__ void zero_unselected_rows_part(uint4* __restrict__ base, const int64_t* __restrict__ q_idx,
                                                          int sq, int n_tokens, int row_chunks, int part, int n_parts,
                                                          int lane) {
  const int n_runs = (n_tokens + 31) >> 5;
  for (int run = part; run < n_runs; run += n_parts) {
    const long long t0 = (long long)run * 32;
    int lo = 0, hi = sq;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (__ldg(q_idx + mid) < t0) lo = mid + 1; else hi = mid;
    }
    unsigned bit = 0;
    if (lo + lane < sq) {
      const long long off = __ldg(q_idx + lo + lane) - t0;   // >= 0 by the search
      if (off >= 0 && off < 32) bit = 1u << (int)off;
    }
    const unsigned selected = __reduce_or_sync(0xffffffffu, bit);
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      const long long tok = t0 + i;
      if (tok >= n_tokens || ((selected >> i) & 1u)) continue;
      uint4* row = base + (size_t)tok * row_chunks;
      for (int c = lane; c < row_chunks; c += 32) row[c] = make_uint4(0, 0, 0, 0);
    }
  }
}
#endif

// Per-kernel event timing (see logo_profile_enable): kernels report under these indices.
enum ProfKind {
  PROF_SELECT = 0, PROF_ATTN_FWD = 1, PROF_BWD_PRE = 2, PROF_BWD_DKV = 3, PROF_BWD_DQ = 4, PROF_BWD_FUSED = 5,
  PROF_BWD_FINISH = 6, PROF_KINDS = 7
};
bool prof_enabled();
void prof_begin(int kind, cudaStream_t stream);
void prof_end(int kind, cudaStream_t stream);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace logo
