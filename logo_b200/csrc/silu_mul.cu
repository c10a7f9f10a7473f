// Gated activation of the model's MLP (logo/modules/mlp.py:25): out = silu(gate) * up, HBM-bound.
// Roundings of the eager bf16 graph: silu is evaluated in fp32 and rounded to bf16, the product is one
// bf16 multiplication. gate / up are rows of `dim` elements with their own row strides, so the two
// halves of a fused gate-up projection can be passed as views; out is packed.
// Bytes per element: 4 read + 2 written.
#include "host_common.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>

namespace logo {

__global__ void __launch_bounds__(256)
    silu_mul_kernel(const __nv_bfloat16* __restrict__ gate, long long gate_stride, const __nv_bfloat16* __restrict__ up,
                    long long up_stride, __nv_bfloat16* __restrict__ out, long long rows, int chunks_per_row) {
  const long long total = rows * chunks_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / chunks_per_row;
    const int c = (int)(i - row * chunks_per_row);
    const uint4 gv = __ldcs(reinterpret_cast<const uint4*>(gate + row * gate_stride) + c);
    const uint4 uv = __ldcs(reinterpret_cast<const uint4*>(up + row * up_stride) + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 r;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x = __bfloat1622float2(g2[k]);
      const __nv_bfloat162 s = __floats2bfloat162_rn(x.x / (1.0f + expf(-x.x)), x.y / (1.0f + expf(-x.y)));
      o2[k] = __hmul2_rn(s, u2[k]);
    }
    __stcs(reinterpret_cast<uint4*>(out + row * (long long)chunks_per_row * 8) + c, r);
  }
}

}  // namespace logo

extern "C" int logo_silu_mul(const void* gate, long long gate_stride, const void* up, long long up_stride, void* out,
                             long long rows, int dim, logo_stream_t stream) {
  using namespace logo;
  LOGO_REQUIRE(rows >= 0 && dim > 0 && dim % 8 == 0, LOGO_ERR_INVALID, "silu_mul: dim must be a positive multiple of 8");
  if (rows == 0) return LOGO_OK;
  LOGO_REQUIRE(gate && up && out, LOGO_ERR_INVALID, "silu_mul: NULL pointer");
  LOGO_REQUIRE(gate_stride % 8 == 0 && up_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(gate) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(up) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
               LOGO_ERR_INVALID, "silu_mul: rows must be 16-byte aligned");
  const long long total = rows * (dim / 8);
  const long long want = (total + 255) / 256;
  const int grid = (int)(want < (long long)sm_count() * 32 ? want : (long long)sm_count() * 32);
  silu_mul_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gate, gate_stride,
                                                          (const __nv_bfloat16*)up, up_stride, (__nv_bfloat16*)out,
                                                          rows, dim / 8);
  LOGO_CHECK_CUDA(cudaGetLastError());
  return LOGO_OK;
}
