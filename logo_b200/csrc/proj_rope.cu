// Per-head re-parameterisation of the global branch fused with the rotary embedding:
//     out[t, h, :] = rope( bf16( x[t, h, :] @ W[h] ) )          (W[h] is [128 in][128 out])
// for every token row, or only for the rows a selection lists (the global QUERY projection is
// needed for the selected rows alone). One pass replaces the batched einsum, the rotary kernel
// and the head-major -> token-major copy that followed it.
//
// A CTA owns one head and a run of 128-row tiles: W[h] is loaded once (TMA, read as an MN-major B
// operand exactly as it lies in memory), each tile of x comes in by TMA (all rows) or is gathered
// row by row through the index list, one 128x128x128 tcgen05 product forms the tile in tensor
// memory, and the epilogue rounds it to bf16 (the rounding of the eager einsum), applies
// (x * cos) + (rotate_half(x) * sin) with its three bf16 roundings, and writes token-major rows
// through a shared-memory staging patch (coalesced 64-byte segments). The loop is single-buffered;
// three CTAs fit one SM (73 KB of shared memory, 128 tensor-memory columns each) and overlap one
// another's loads, product and stores.
// Bytes per row and head (HBM-bound): 256 read + 256 written (+ the cos / sin row, shared by the heads).
#include "attn_common.cuh"
#include "host_common.cuh"

#include <cuda_bf16.h>

namespace logo {

constexpr int PR_THREADS = 128;
constexpr int PR_SMEM_BYTES = 2 * TILE_BYTES + 4 * 2048 + 1024;

struct ProjArgs {
  const __nv_bfloat16* x;      // [n_tokens][x_stride], head h at column h * 128
  long long x_stride;
  const int64_t* rows;         // null: every token; else ascending token indices, *n_rows_ptr of them
  const int32_t* n_rows_ptr;
  const __nv_bfloat16* cos_t;  // [n_tokens][128] or null (no rotation)
  const __nv_bfloat16* sin_t;
  __nv_bfloat16* out;          // [n_tokens][heads * 128]
  int n_tokens, heads, tiles_per_cta;
  int* status;
};

__global__ void __launch_bounds__(PR_THREADS)
    proj_rope_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                     const ProjArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sW = smem;                  // [128 in][128 out] as two [128][64] blocks
  uint8_t* sX = smem + TILE_BYTES;     // [128 rows][128 in] as two [128][64] blocks
  uint8_t* s_stage = smem + 2 * TILE_BYTES;
  __shared__ uint64_t w_full, x_full, mma_done;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = uniform_warp_idx(), lane = tid & 31;
  const int h = blockIdx.y;
  const int n_rows = a.rows ? min(max(__ldg(a.n_rows_ptr), 0), a.n_tokens) : a.n_tokens;
  const int n_tiles = (n_rows + TILE - 1) / TILE;
  const int tile0 = blockIdx.x * a.tiles_per_cta;
  if (tile0 >= n_tiles) return;
  const int tile_end = min(tile0 + a.tiles_per_cta, n_tiles);
  AbortState ab{&abort_flag, a.status};

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&w_full, 1);
    mbar_init(&x_full, 1);
    mbar_init(&mma_done, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_slot, 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t lane_off = (uint32_t)(warp * 32) << 16;

  if (tid == 0) {
    tma_prefetch_desc(&tm_w);
    mbar_arrive_expect_tx(&w_full, TILE_BYTES);
    tma_load_2d(sW, &tm_w, &w_full, 0, h * HEAD_DIM);
    tma_load_2d(sW + BLK_BYTES, &tm_w, &w_full, 64, h * HEAD_DIM);
  }

  uint32_t it = 0;
  for (int t = tile0; t < tile_end; ++t, ++it) {
    const int r0 = t * TILE;
    const int nv = min(n_rows - r0, TILE);
    // ---- the x tile: by TMA when every row is wanted, row by row through the list otherwise ----
    if (!a.rows) {
      if (tid == 0) {
        mbar_arrive_expect_tx(&x_full, TILE_BYTES);
        tma_load_2d(sX, &tm_x, &x_full, h * HEAD_DIM, r0);        // rows past the end are zero-filled
        tma_load_2d(sX + BLK_BYTES, &tm_x, &x_full, h * HEAD_DIM + 64, r0);
      }
    } else {
      const int ch = tid & 15;
      uint4 vals[16];
      bool bad = false;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int r = i * 8 + (tid >> 4);
        long long tok = __ldg(a.rows + r0 + min(r, nv - 1));
        if (tok < 0 || tok >= a.n_tokens) {
          bad = true;
          tok = 0;
        }
        vals[i] = __ldg(reinterpret_cast<const uint4*>(a.x + tok * a.x_stride + h * HEAD_DIM) + ch);
      }
      if (bad && a.status) atomicCAS(a.status, 0, (int)DEV_BAD_INDEX);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int r = i * 8 + (tid >> 4);
        const uint4 v = (r < nv) ? vals[i] : make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(sX + (ch >> 3) * BLK_BYTES + sw128_offset((uint32_t)r, (uint32_t)(ch & 7) * 8)) = v;
      }
      fence_proxy_async_smem();
    }
    __syncthreads();
    // ---- one tile product: D[row][out] = sum_in X[row][in] W[in][out] ----
    if (warp == 0) {
      if (!a.rows) mbar_wait(&x_full, it & 1u, ab);
      if (it == 0) mbar_wait(&w_full, 0, ab);
      tc_fence_after();
      umma_tile_k128<false, true>(tmem, umma_desc_sw128(smem_u32(sX), 0, 1024),
                                  umma_desc_sw128(smem_u32(sW), BLK_BYTES, 1024),
                                  umma_idesc_bf16(TILE, HEAD_DIM, 0, 1), 0u);
      umma_commit(&mma_done);
    }
    const bool ok = mbar_wait(&mma_done, it & 1u, ab);
    tc_fence_after();
    // ---- epilogue: thread = row; columns [32 q, +32) together with their rotation partners [64 + 32 q, +32) ----
    long long tok = -1;
    if (tid < nv) tok = a.rows ? __ldg(a.rows + r0 + tid) : (long long)(r0 + tid);
    const bool store = ok && tok >= 0 && tok < a.n_tokens;
    const long long row_off = store ? tok * (long long)a.heads * HEAD_DIM + (long long)h * HEAD_DIM : -1;
#pragma unroll 1
    for (int q = 0; q < 2; ++q) {
      uint32_t f1[32], f2[32];
      tmem_ld32(tmem + lane_off + 32u * q, f1);
      tmem_ld32(tmem + lane_off + 64u + 32u * q, f2);
      tmem_ld_wait();
      __nv_bfloat162 x1[16], x2[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {   // the rounding of the eager projection output
        x1[i] = __floats2bfloat162_rn(__uint_as_float(f1[2 * i]), __uint_as_float(f1[2 * i + 1]));
        x2[i] = __floats2bfloat162_rn(__uint_as_float(f2[2 * i]), __uint_as_float(f2[2 * i + 1]));
      }
      uint32_t o1[16], o2[16];
      if (a.cos_t) {
        const long long tk = store ? tok : 0;
        const uint4* c1p = reinterpret_cast<const uint4*>(a.cos_t + tk * HEAD_DIM + 32 * q);
        const uint4* c2p = reinterpret_cast<const uint4*>(a.cos_t + tk * HEAD_DIM + 64 + 32 * q);
        const uint4* s1p = reinterpret_cast<const uint4*>(a.sin_t + tk * HEAD_DIM + 32 * q);
        const uint4* s2p = reinterpret_cast<const uint4*>(a.sin_t + tk * HEAD_DIM + 64 + 32 * q);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint4 vc1 = __ldg(c1p + g), vc2 = __ldg(c2p + g), vs1 = __ldg(s1p + g), vs2 = __ldg(s2p + g);
          const __nv_bfloat162* c1 = reinterpret_cast<const __nv_bfloat162*>(&vc1);
          const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&vc2);
          const __nv_bfloat162* s1 = reinterpret_cast<const __nv_bfloat162*>(&vs1);
          const __nv_bfloat162* s2 = reinterpret_cast<const __nv_bfloat162*>(&vs2);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            // first half: x1*cos1 + (-x2)*sin1 ; second half: x2*cos2 + x1*sin2 (one rounding per operation)
            const __nv_bfloat162 r1 =
                __hadd2_rn(__hmul2_rn(x1[4 * g + i], c1[i]), __hmul2_rn(__hneg2(x2[4 * g + i]), s1[i]));
            const __nv_bfloat162 r2 = __hadd2_rn(__hmul2_rn(x2[4 * g + i], c2[i]), __hmul2_rn(x1[4 * g + i], s2[i]));
            o1[4 * g + i] = *reinterpret_cast<const uint32_t*>(&r1);
            o2[4 * g + i] = *reinterpret_cast<const uint32_t*>(&r2);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          o1[i] = *reinterpret_cast<const uint32_t*>(&x1[i]);
          o2[i] = *reinterpret_cast<const uint32_t*>(&x2[i]);
        }
      }
      store_patch_32x32(s_stage + warp * 2048, o1, a.out, row_off >= 0 ? row_off + 32 * q : -1, lane);
      store_patch_32x32(s_stage + warp * 2048, o2, a.out, row_off >= 0 ? row_off + 64 + 32 * q : -1, lane);
    }
    tc_fence_before();
    __syncthreads();   // the x tile and the accumulator are free for the next tile
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 128);
}

}  // namespace logo

extern "C" int logo_proj_rope(const void* x, long long x_stride, const void* w, const int64_t* rows,
                              const int32_t* n_rows, const void* cos_t, const void* sin_t, void* out, int n_tokens,
                              int heads, int d, int32_t* status, logo_stream_t stream_) {
  using namespace logo;
  cudaStream_t stream = (cudaStream_t)stream_;
  LOGO_REQUIRE(d == HEAD_DIM, LOGO_ERR_UNSUPPORTED, "proj_rope: head_dim %d is not supported (only 128)", d);
  LOGO_REQUIRE(n_tokens >= 0 && heads > 0, LOGO_ERR_INVALID, "proj_rope: bad sizes");
  if (n_tokens == 0) return LOGO_OK;
  LOGO_REQUIRE(x && w && out, LOGO_ERR_INVALID, "proj_rope: NULL pointer");
  LOGO_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), LOGO_ERR_INVALID, "proj_rope: cos and sin go together");
  LOGO_REQUIRE((rows == nullptr) == (n_rows == nullptr), LOGO_ERR_INVALID, "proj_rope: rows and n_rows go together");
  LOGO_REQUIRE(x_stride % 8 == 0 && x_stride >= (long long)heads * HEAD_DIM && aligned16(x) && aligned16(w) &&
                   aligned16(out) && (!cos_t || (aligned16(cos_t) && aligned16(sin_t))),
               LOGO_ERR_INVALID, "proj_rope: rows must be 16-byte aligned (strides multiples of 8 elements)");
  CUtensorMap tm_x, tm_w;
  int rc = make_tmap_2d_bf16(&tm_x, x, (uint64_t)heads * HEAD_DIM, (uint64_t)n_tokens, (uint64_t)x_stride * 2, 64, TILE);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tm_w, w, HEAD_DIM, (uint64_t)heads * HEAD_DIM, HEAD_DIM * 2, 64, TILE);
  if (rc) return rc;
  static thread_local int attr_set_dev = -1;
  int dev = 0;
  LOGO_CHECK_CUDA(cudaGetDevice(&dev));
  if (attr_set_dev != dev) {
    LOGO_CHECK_CUDA(cudaFuncSetAttribute(proj_rope_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PR_SMEM_BYTES));
    attr_set_dev = dev;
  }
  ProjArgs a{};
  a.x = (const __nv_bfloat16*)x;
  a.x_stride = x_stride;
  a.rows = rows;
  a.n_rows_ptr = n_rows;
  a.cos_t = (const __nv_bfloat16*)cos_t;
  a.sin_t = (const __nv_bfloat16*)sin_t;
  a.out = (__nv_bfloat16*)out;
  a.n_tokens = n_tokens;
  a.heads = heads;
  a.status = status;
  // enough CTAs to fill every SM three times over, each with a run of tiles long enough to amortise W
  const int n_tiles = (n_tokens + TILE - 1) / TILE;
  const int want_ctas = sm_count() * 3;
  int per = (n_tiles * heads + want_ctas - 1) / want_ctas;
  per = per < 1 ? 1 : (per > 8 ? 8 : per);
  a.tiles_per_cta = per;
  dim3 grid((n_tiles + per - 1) / per, heads);
  proj_rope_kernel<<<grid, PR_THREADS, PR_SMEM_BYTES, stream>>>(tm_x, tm_w, a);
  LOGO_CHECK_CUDA(cudaGetLastError());
  return LOGO_OK;
}
