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

// 2-D bf16 tensor map with 128-byte swizzle. `inner` elements are contiguous,
// `outer` rows are `row_stride_bytes` apart. Box = box_inner x box_outer elements;
// box_inner must be 64 (128 bytes) for the 128-byte swizzle.
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);

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
