// Rotary position embedding of a packed [n_tokens, heads, 128] bf16 tensor (HBM-bound).
//
//   out = bf16( bf16(x * cos) + bf16(rotate_half(x) * sin) ),  rotate_half(x) = cat(-x[64:], x[:64])
//
// i.e. the eager bf16 graph `(x * cos) + (rotate_half(x) * sin)` with each of its three roundings
// reproduced, in one pass over the tensor instead of six element-wise kernels and a concatenation.
// With `inverse != 0` the transposed rotation is applied (cat(y[64:], -y[:64]) in place of
// rotate_half): the gradient of the expression above with respect to x, rounded the way autograd
// rounds it.
//
// Layout: eight lanes own one 128-element head row; a lane loads the 16-byte chunk at column
// 8*l of the first half together with its partner at column 64 + 8*l, so both halves of a rotation
// pair sit in one thread. The input may be any view with contiguous 128-element rows (token and
// head strides are arguments: the per-head projection of the global branch comes out head-major);
// the output is packed. cos / sin are [n_tokens, 128] (any values: the two halves are read
// separately, nothing assumes cos[d] == cos[d + 64]).
// Bytes per token: heads * 256 read + heads * 256 written (+ 512 for cos / sin, L1-resident across
// the heads of a token).
#include "host_common.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>

namespace logo {

constexpr int ROPE_THREADS = 256;

// One thread: columns [8*l, 8*l+8) and [64 + 8*l, 64 + 8*l + 8) of one (token, head) row.
template <bool INVERSE>
__global__ void __launch_bounds__(ROPE_THREADS)
    rope_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                const __nv_bfloat16* __restrict__ cos_t, const __nv_bfloat16* __restrict__ sin_t, long long n_rows,
                int heads, long long x_stride_tok, long long x_stride_head) {
  const long long stride = (long long)gridDim.x * (ROPE_THREADS / 8);
  const int l = threadIdx.x & 7;
  for (long long row = (long long)blockIdx.x * (ROPE_THREADS / 8) + (threadIdx.x >> 3); row < n_rows; row += stride) {
    const long long tok = row / heads;
    const int head = (int)(row - tok * heads);
    const uint4* xr = reinterpret_cast<const uint4*>(x + tok * x_stride_tok + head * x_stride_head);
    const uint4* cr = reinterpret_cast<const uint4*>(cos_t + tok * 128);
    const uint4* sr = reinterpret_cast<const uint4*>(sin_t + tok * 128);
    const uint4 vx1 = __ldcs(xr + l), vx2 = __ldcs(xr + 8 + l);
    const uint4 vc1 = __ldg(cr + l), vc2 = __ldg(cr + 8 + l);
    const uint4 vs1 = __ldg(sr + l), vs2 = __ldg(sr + 8 + l);
    // Packed bf16 arithmetic: a bf16 x bf16 product is exact in fp32 and an fp32 sum of two bf16
    // values rounds to the same bf16 as their exact sum, so one rounding per packed instruction
    // reproduces the eager graph's convert / multiply / convert sequence bit for bit (`_rn` forms:
    // the plain ones may be contracted into a fused multiply-add, losing the product's rounding).
    const __nv_bfloat162* x1 = reinterpret_cast<const __nv_bfloat162*>(&vx1);
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&vx2);
    const __nv_bfloat162* c1 = reinterpret_cast<const __nv_bfloat162*>(&vc1);
    const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&vc2);
    const __nv_bfloat162* s1 = reinterpret_cast<const __nv_bfloat162*>(&vs1);
    const __nv_bfloat162* s2 = reinterpret_cast<const __nv_bfloat162*>(&vs2);
    uint4 w1, w2;
    __nv_bfloat162* o1 = reinterpret_cast<__nv_bfloat162*>(&w1);
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&w2);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (!INVERSE) {
        // first half: x1*cos1 + (-x2)*sin1 ; second half: x2*cos2 + x1*sin2
        o1[i] = __hadd2_rn(__hmul2_rn(x1[i], c1[i]), __hmul2_rn(__hneg2(x2[i]), s1[i]));
        o2[i] = __hadd2_rn(__hmul2_rn(x2[i], c2[i]), __hmul2_rn(x1[i], s2[i]));
      } else {
        // gradient: y*cos + rotate_half^T(y*sin), rotate_half^T(z) = cat(z[64:], -z[:64])
        o1[i] = __hadd2_rn(__hmul2_rn(x1[i], c1[i]), __hmul2_rn(x2[i], s2[i]));
        o2[i] = __hadd2_rn(__hmul2_rn(x2[i], c2[i]), __hneg2(__hmul2_rn(x1[i], s1[i])));
      }
    }
    uint4* orow = reinterpret_cast<uint4*>(out + row * 128);
    __stcs(orow + l, w1);
    __stcs(orow + 8 + l, w2);
  }
}

}  // namespace logo

extern "C" int logo_rope(const void* x, long long x_stride_tok, long long x_stride_head, void* out, const void* cos_t,
                         const void* sin_t, int n_tokens, int heads, int d, int inverse, logo_stream_t stream) {
  using namespace logo;
  LOGO_REQUIRE(d == 128, LOGO_ERR_UNSUPPORTED, "rope: head_dim must be 128");
  LOGO_REQUIRE(n_tokens >= 0 && heads > 0, LOGO_ERR_INVALID, "rope: bad sizes");
  if (n_tokens == 0) return LOGO_OK;
  LOGO_REQUIRE(x && out && cos_t && sin_t, LOGO_ERR_INVALID, "rope: NULL pointer");
  LOGO_REQUIRE(x_stride_tok % 8 == 0 && x_stride_head % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(out) & 15) == 0,
               LOGO_ERR_INVALID, "rope: rows must be 16-byte aligned (strides multiples of 8 elements)");
  const long long n_rows = (long long)n_tokens * heads;
  const long long want = (n_rows + (ROPE_THREADS / 8) - 1) / (ROPE_THREADS / 8);
  const int grid = (int)(want < (long long)sm_count() * 16 ? want : (long long)sm_count() * 16);
  cudaStream_t s = (cudaStream_t)stream;
  if (inverse)
    rope_kernel<true><<<grid, ROPE_THREADS, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out,
                                                    (const __nv_bfloat16*)cos_t, (const __nv_bfloat16*)sin_t, n_rows,
                                                    heads, x_stride_tok, x_stride_head);
  else
    rope_kernel<false><<<grid, ROPE_THREADS, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out,
                                                     (const __nv_bfloat16*)cos_t, (const __nv_bfloat16*)sin_t, n_rows,
                                                     heads, x_stride_tok, x_stride_head);
  LOGO_CHECK_CUDA(cudaGetLastError());
  return LOGO_OK;
}
