// RMSNorm over rows of any width (the decoder-stack norms of the model use the same module as the
// per-head context norms), forward only, HBM-bound:
//
//   out = weight * bf16( x * rsqrt(mean(x^2) + eps) )
//
// with the roundings of the eager module: the normalised value is rounded to bf16 before the
// multiplication by the weight, and that product is one bf16 multiplication.
// One warp per row; a lane reads 16-byte chunks at stride 32 chunks. The row is read twice (sum of
// squares, then the scaling); the second read comes from L1 / L2 (a row is a few KB).
// Bytes per row: dim * 2 read + dim * 2 written.
#include "host_common.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>

namespace logo {

constexpr int RMS_THREADS = 256;

__global__ void __launch_bounds__(RMS_THREADS)
    rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                       __nv_bfloat16* __restrict__ out, long long rows, int dim, float eps) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = RMS_THREADS / 32;
  const int chunks = dim >> 3;   // 16-byte chunks per row
  const float inv_dim = 1.0f / (float)dim;
  for (long long row = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += (long long)gridDim.x * warps_per_block) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * dim);
    float ss = 0.f;
    for (int c = lane; c < chunks; c += 32) {
      const uint4 v = __ldg(xr + c);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(p[i]);
        ss = fmaf(f.x, f.x, ss);
        ss = fmaf(f.y, f.y, ss);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss * inv_dim + eps);
    uint4* orow = reinterpret_cast<uint4*>(out + row * dim);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    for (int c = lane; c < chunks; c += 32) {
      const uint4 v = __ldg(xr + c);
      const uint4 wv = __ldg(wr + c);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
      const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&wv);
      uint4 r;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(p[i]);
        const __nv_bfloat162 xh = __floats2bfloat162_rn(f.x * rstd, f.y * rstd);
        o2[i] = __hmul2_rn(q[i], xh);   // one rounding of the exact product = the eager bf16 multiply
      }
      __stcs(orow + c, r);
    }
  }
}

}  // namespace logo

extern "C" int logo_rmsnorm_fwd(const void* x, const void* weight, void* out, long long rows, int dim, float eps,
                                logo_stream_t stream) {
  using namespace logo;
  LOGO_REQUIRE(rows >= 0 && dim > 0 && dim % 8 == 0, LOGO_ERR_INVALID, "rmsnorm: dim must be a positive multiple of 8");
  if (rows == 0) return LOGO_OK;
  LOGO_REQUIRE(x && weight && out, LOGO_ERR_INVALID, "rmsnorm: NULL pointer");
  LOGO_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(weight) & 15) == 0,
               LOGO_ERR_INVALID, "rmsnorm: pointers must be 16-byte aligned");
  const long long want = (rows + (RMS_THREADS / 32) - 1) / (RMS_THREADS / 32);
  const int grid = (int)(want < (long long)sm_count() * 16 ? want : (long long)sm_count() * 16);
  rmsnorm_fwd_kernel<<<grid, RMS_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)weight, (__nv_bfloat16*)out, rows, dim, eps);
  LOGO_CHECK_CUDA(cudaGetLastError());
  return LOGO_OK;
}
