// Per-branch RMSNorm + gate mask + blend, forward and backward (HBM-bound, no tensor cores).
//
//   y_l = w_l * bf16(x_l * rsqrt(mean(x_l^2) + eps))       per (token, head) row of 128
//   y_g = w_g * bf16(x_g * rsqrt(mean(x_g^2) + eps))       only for tokens with gate >= thres
//   g   = gate >= thres ? gate : 0
//   out = (1 - g) * y_l + g * y_g
//
// Every intermediate is rounded to bf16 where the reference's eager bf16 graph rounds it, so
// for bf16 weights the forward result reproduces that graph's arithmetic.
// Rows of the global branch that are not selected are never read.
//
// Layout: 16 lanes own one 128-element row (8 contiguous bf16 = 16 bytes per lane), a warp
// walks the heads of one token two at a time.
// Bytes per token (forward): H*256 read (local) + H*256 read (global, selected tokens only)
// + H*256 written + sizeof(gate).
#include "host_common.cuh"
#include "ptx.cuh"

#include <cuda_fp16.h>

namespace logo {

constexpr int FUSE_THREADS = 256;
constexpr int FUSE_D = 128;
constexpr int FUSE_U = 4;   // head pairs whose loads are in flight together (forward)

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ float load_scalar_any(const void* p, int dtype) {
  if (dtype == LOGO_DTYPE_F32) return *static_cast<const float*>(p);
  if (dtype == LOGO_DTYPE_BF16) return __bfloat162float(*static_cast<const __nv_bfloat16*>(p));
  return __half2float(*static_cast<const __half*>(p));
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  v.x = pack_bf16x2(f[0], f[1]);
  v.y = pack_bf16x2(f[2], f[3]);
  v.z = pack_bf16x2(f[4], f[5]);
  v.w = pack_bf16x2(f[6], f[7]);
  return v;
}

__device__ __forceinline__ void load_weight8(const void* w, int w_dtype, int col, float (&f)[8]) {
  if (w == nullptr) {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = 1.f;
  } else if (w_dtype == LOGO_DTYPE_BF16) {
    unpack8(*reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(w) + col), f);
  } else {
    const float* p = static_cast<const float*>(w) + col;
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = p[i];
  }
}

// The eager graph does its bf16 element-wise arithmetic one operation at a time, each rounded to
// bf16. A bf16 x bf16 product is exact in fp32, and an fp32 sum of two bf16 values rounds to the same
// bf16 as the exact sum, so the packed bf16 instructions (one rounding of the exact result) give the
// graph's bits at a quarter of the instruction count of convert / multiply / convert. The `_rn`
// forms are required: the plain ones may be contracted into a fused multiply-add, which skips the
// rounding of the product.
__device__ __forceinline__ uint32_t bmul2(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t badd2(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r = __hadd2_rn(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bsplat2(float x) { return pack_bf16x2(x, x); }

// normalised row as packed bf16 (`hidden_states.to(input_dtype)`): four words for eight elements
__device__ __forceinline__ void normalise8_packed(const uint4& v, float eps, uint32_t (&xh)[4]) {
  float x[8];
  unpack8(v, x);
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
  ss += __shfl_xor_sync(0xffffffffu, ss, 8);
  ss += __shfl_xor_sync(0xffffffffu, ss, 4);
  ss += __shfl_xor_sync(0xffffffffu, ss, 2);
  ss += __shfl_xor_sync(0xffffffffu, ss, 1);
  const float rstd = rsqrtf(ss * (1.0f / FUSE_D) + eps);
#pragma unroll
  for (int i = 0; i < 4; ++i) xh[i] = pack_bf16x2(x[2 * i] * rstd, x[2 * i + 1] * rstd);
}

// sum over the 16 lanes that share a row
__device__ __forceinline__ float row_sum16(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 8);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  return x;
}

// normalised row, rounded to bf16 like `hidden_states.to(input_dtype)`; returns rstd
__device__ __forceinline__ float normalise8(const float (&x)[8], float eps, bool use_norm, float (&xh)[8]) {
  if (!use_norm) {
#pragma unroll
    for (int i = 0; i < 8; ++i) xh[i] = x[i];
    return 1.f;
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
  ss = row_sum16(ss);
  const float rstd = rsqrtf(ss * (1.0f / FUSE_D) + eps);
#pragma unroll
  for (int i = 0; i < 8; ++i) xh[i] = bf16_round(x[i] * rstd);
  return rstd;
}

__global__ void __launch_bounds__(FUSE_THREADS)
    fuse_fwd_kernel(const __nv_bfloat16* __restrict__ local, const __nv_bfloat16* __restrict__ glob,
                    const __nv_bfloat16* __restrict__ gate, const void* __restrict__ thres_ptr, int thres_dtype,
                    const void* __restrict__ w_local, const void* __restrict__ w_global, int w_dtype,
                    __nv_bfloat16* __restrict__ out, int n_tokens, int h, float eps, int use_norm) {
  const int lane = threadIdx.x & 31;
  const int sub = lane >> 4;          // which of the two heads handled together
  const int col = (lane & 15) * 8;
  const int warps_per_block = FUSE_THREADS / 32;
  const float thres = load_scalar_any(thres_ptr, thres_dtype);
  const bool bf16_w = (w_dtype == LOGO_DTYPE_BF16);

  float wl[8], wg[8];
  load_weight8(use_norm ? w_local : nullptr, w_dtype, col, wl);
  load_weight8(use_norm ? w_global : nullptr, w_dtype, col, wg);
  uint32_t wl2[4], wg2[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    wl2[i] = pack_bf16x2(wl[2 * i], wl[2 * i + 1]);
    wg2[i] = pack_bf16x2(wg[2 * i], wg[2 * i + 1]);
  }

  for (int tok = blockIdx.x * warps_per_block + (threadIdx.x >> 5); tok < n_tokens;
       tok += gridDim.x * warps_per_block) {
    const float gate_f = __bfloat162float(gate[tok]);
    const bool selected = gate_f >= thres;
    const float g = selected ? gate_f : 0.f;
    const float one_minus_g = bf16_round(1.f - g);
    const uint32_t g2 = bsplat2(g), omg2 = bsplat2(one_minus_g);
    // FUSE_U head pairs per iteration: all their loads are issued before the first reduction, which
    // is what keeps enough bytes in flight. The trip count is warp-uniform (the row sums shuffle).
    for (int hb = 0; hb < h; hb += 2 * FUSE_U) {
      uint4 lv[FUSE_U], gv[FUSE_U];
      size_t off[FUSE_U];
      bool act[FUSE_U];
#pragma unroll
      for (int u = 0; u < FUSE_U; ++u) {
        const int hh = hb + 2 * u + sub;
        act[u] = hh < h;
        off[u] = ((size_t)tok * h + (act[u] ? hh : 0)) * FUSE_D + col;
        lv[u] = __ldg(reinterpret_cast<const uint4*>(local + off[u]));
        if (selected) gv[u] = __ldg(reinterpret_cast<const uint4*>(glob + off[u]));
      }
      if (use_norm && bf16_w) {
        // bf16 weights (the layer's own dtype): everything after the normalisation is packed bf16
#pragma unroll
        for (int u = 0; u < FUSE_U; ++u) {
          uint32_t xh[4], yl[4];
          normalise8_packed(lv[u], eps, xh);
#pragma unroll
          for (int i = 0; i < 4; ++i) yl[i] = bmul2(wl2[i], xh[i]);
          if (selected) {
            uint32_t yg[4];
            normalise8_packed(gv[u], eps, xh);
#pragma unroll
            for (int i = 0; i < 4; ++i) yg[i] = bmul2(wg2[i], xh[i]);
#pragma unroll
            for (int i = 0; i < 4; ++i) yl[i] = badd2(bmul2(omg2, yl[i]), bmul2(g2, yg[i]));
          }
          if (act[u]) *reinterpret_cast<uint4*>(out + off[u]) = make_uint4(yl[0], yl[1], yl[2], yl[3]);
        }
        continue;
      }
#pragma unroll
      for (int u = 0; u < FUSE_U; ++u) {
        float x[8], xh[8], yl[8], res[8];
        unpack8(lv[u], x);
        normalise8(x, eps, use_norm != 0, xh);
#pragma unroll
        for (int i = 0; i < 8; ++i) yl[i] = (use_norm && bf16_w) ? bf16_round(wl[i] * xh[i]) : wl[i] * xh[i];
        if (selected) {
          float yg[8];
          unpack8(gv[u], x);
          normalise8(x, eps, use_norm != 0, xh);
#pragma unroll
          for (int i = 0; i < 8; ++i) yg[i] = (use_norm && bf16_w) ? bf16_round(wg[i] * xh[i]) : wg[i] * xh[i];
#pragma unroll
          for (int i = 0; i < 8; ++i) res[i] = bf16_round(one_minus_g * yl[i]) + bf16_round(g * yg[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) res[i] = yl[i];
        }
        if (act[u]) *reinterpret_cast<uint4*>(out + off[u]) = pack8(res);
      }
    }
  }
}

// Backward. Each warp owns tokens; the weight gradients are accumulated per thread, reduced
// per block in a fixed order and written as block partials; fuse_bwd_finish_kernel sums them.
__global__ void __launch_bounds__(FUSE_THREADS, 3)   // three blocks per SM: the kernel is latency-bound
    fuse_bwd_kernel(const __nv_bfloat16* __restrict__ d_out, const __nv_bfloat16* __restrict__ local,
                    const __nv_bfloat16* __restrict__ glob, const __nv_bfloat16* __restrict__ gate,
                    const void* __restrict__ thres_ptr, int thres_dtype, const void* __restrict__ w_local,
                    const void* __restrict__ w_global, int w_dtype, __nv_bfloat16* __restrict__ d_local,
                    __nv_bfloat16* __restrict__ d_glob, __nv_bfloat16* __restrict__ d_gate,
                    float* __restrict__ partials, int n_tokens, int h, float eps, int use_norm) {
  __shared__ float s_part[FUSE_THREADS / 16][2][FUSE_D];
  const int lane = threadIdx.x & 31;
  const int sub = lane >> 4;
  const int col = (lane & 15) * 8;
  const int warps_per_block = FUSE_THREADS / 32;
  const float thres = load_scalar_any(thres_ptr, thres_dtype);

  float wl[8], wg[8], dwl[8], dwg[8];
  load_weight8(use_norm ? w_local : nullptr, w_dtype, col, wl);
  load_weight8(use_norm ? w_global : nullptr, w_dtype, col, wg);
#pragma unroll
  for (int i = 0; i < 8; ++i) dwl[i] = dwg[i] = 0.f;

  for (int tok = blockIdx.x * warps_per_block + (threadIdx.x >> 5); tok < n_tokens;
       tok += gridDim.x * warps_per_block) {
    const float gate_f = __bfloat162float(gate[tok]);
    const bool selected = gate_f >= thres;
    const float g = selected ? gate_f : 0.f;
    const float one_minus_g = 1.f - g;
    float dgate = 0.f;
#pragma unroll 2
    for (int hb = 0; hb < h; hb += 2) {
      const int hh = hb + sub;
      const bool act = hh < h;
      const size_t off = ((size_t)tok * h + (act ? hh : 0)) * FUSE_D + col;
      float go[8], x[8], xh[8];
      // all three loads of the row are issued before the first reduction
      const uint4 go_v = __ldg(reinterpret_cast<const uint4*>(d_out + off));
      const uint4 lo_v = __ldg(reinterpret_cast<const uint4*>(local + off));
      uint4 gl_v = make_uint4(0, 0, 0, 0);
      if (selected) gl_v = __ldg(reinterpret_cast<const uint4*>(glob + off));
      unpack8(go_v, go);
      if (!act) {
#pragma unroll
        for (int i = 0; i < 8; ++i) go[i] = 0.f;
      }

      // local branch
      unpack8(lo_v, x);
      const float rstd_l = normalise8(x, eps, use_norm != 0, xh);
      float dxh[8], dot = 0.f, res[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float dy = one_minus_g * go[i];
        dwl[i] = fmaf(dy, xh[i], dwl[i]);
        dxh[i] = dy * wl[i];
        dot = fmaf(dxh[i], xh[i], dot);
        dgate -= go[i] * wl[i] * xh[i];
      }
      if (use_norm) {
        dot = row_sum16(dot) * (1.0f / FUSE_D);
#pragma unroll
        for (int i = 0; i < 8; ++i) res[i] = rstd_l * (dxh[i] - xh[i] * dot);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) res[i] = dxh[i];
      }
      if (act) *reinterpret_cast<uint4*>(d_local + off) = pack8(res);

      // global branch
      if (selected) {
        unpack8(gl_v, x);
        const float rstd_g = normalise8(x, eps, use_norm != 0, xh);
        dot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float dy = g * go[i];
          dwg[i] = fmaf(dy, xh[i], dwg[i]);
          dxh[i] = dy * wg[i];
          dot = fmaf(dxh[i], xh[i], dot);
          dgate += go[i] * wg[i] * xh[i];
        }
        if (use_norm) {
          dot = row_sum16(dot) * (1.0f / FUSE_D);
#pragma unroll
          for (int i = 0; i < 8; ++i) res[i] = rstd_g * (dxh[i] - xh[i] * dot);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) res[i] = dxh[i];
        }
        if (act) *reinterpret_cast<uint4*>(d_glob + off) = pack8(res);
      } else if (act) {
        *reinterpret_cast<uint4*>(d_glob + off) = make_uint4(0, 0, 0, 0);
      }
    }
    // d gate: sum over every head and column of the token; zero where the gate was masked
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dgate += __shfl_xor_sync(0xffffffffu, dgate, o);
    if (lane == 0) d_gate[tok] = __float2bfloat16_rn(selected ? dgate : 0.f);
  }

  // fixed-order block reduction of the weight gradients
  const int hw = threadIdx.x >> 4;  // half-warp index, 0..15
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    s_part[hw][0][col + i] = dwl[i];
    s_part[hw][1][col + i] = dwg[i];
  }
  __syncthreads();
  {
    const int which = threadIdx.x >> 7, c = threadIdx.x & 127;
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < FUSE_THREADS / 16; ++k) acc += s_part[k][which][c];
    partials[((size_t)blockIdx.x * 2 + which) * FUSE_D + c] = acc;
  }
}

// Sums the block partials in a fixed order: 4 slices of the block list per column in parallel, then
// the 4 slice sums in order (deterministic, and 4x shorter than one thread per column walking the list).
__global__ void __launch_bounds__(1024)
    fuse_bwd_finish_kernel(const float* __restrict__ partials, int nblocks, void* d_w_local, void* d_w_global,
                           int w_dtype) {
  __shared__ float s_acc[4][2 * FUSE_D];
  const int slice = threadIdx.x >> 8, wc = threadIdx.x & 255;   // wc = which * 128 + column
  const int per = (nblocks + 3) / 4;
  const int b0 = slice * per, b1 = min(b0 + per, nblocks);
  float acc = 0.f;
  int b = b0;
  for (; b + 8 <= b1; b += 8) {   // eight loads in flight, added in list order
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = __ldg(partials + (size_t)(b + k) * 2 * FUSE_D + wc);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc += v[k];
  }
  for (; b < b1; ++b) acc += __ldg(partials + (size_t)b * 2 * FUSE_D + wc);
  s_acc[slice][wc] = acc;
  __syncthreads();
  if (slice == 0) {
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) tot += s_acc[k][wc];
    void* dst = (wc >> 7) == 0 ? d_w_local : d_w_global;
    if (!dst) return;
    const int c = wc & 127;
    if (w_dtype == LOGO_DTYPE_BF16)
      static_cast<__nv_bfloat16*>(dst)[c] = __float2bfloat16_rn(tot);
    else
      static_cast<float*>(dst)[c] = tot;
  }
}

static int fuse_grid(int n_tokens) {
  const int warps_per_block = FUSE_THREADS / 32;
  const int want = (n_tokens + warps_per_block - 1) / warps_per_block;
  const int cap = sm_count() * 8;
  return want < 1 ? 1 : (want < cap ? want : cap);
}

static int check_fuse(const void* local, const void* glob, const void* gate, int gate_dtype, const void* thres,
                      int thres_dtype, const void* w_local, const void* w_global, int w_dtype, int n_tokens, int h,
                      int d, int use_norm) {
  LOGO_REQUIRE(d == FUSE_D, LOGO_ERR_UNSUPPORTED, "head_dim %d is not supported (only 128)", d);
  LOGO_REQUIRE(n_tokens >= 0 && h > 0, LOGO_ERR_INVALID, "n_tokens must be >= 0 and h > 0");
  LOGO_REQUIRE(gate_dtype == LOGO_DTYPE_BF16, LOGO_ERR_UNSUPPORTED, "the gate must be bf16 like the activations");
  LOGO_REQUIRE(thres_dtype >= LOGO_DTYPE_BF16 && thres_dtype <= LOGO_DTYPE_F16, LOGO_ERR_INVALID,
               "unknown threshold dtype %d", thres_dtype);
  LOGO_REQUIRE(n_tokens == 0 || (local && glob && gate && thres), LOGO_ERR_INVALID,
               "local, glob, gate and thres must not be NULL");
  if (use_norm) {
    LOGO_REQUIRE(w_local && w_global, LOGO_ERR_INVALID, "norm weights must not be NULL when use_norm is set");
    LOGO_REQUIRE(w_dtype == LOGO_DTYPE_BF16 || w_dtype == LOGO_DTYPE_F32, LOGO_ERR_INVALID,
                 "norm weights must be bf16 or fp32");
    LOGO_REQUIRE(aligned16(w_local) && aligned16(w_global), LOGO_ERR_INVALID, "norm weights must be 16-byte aligned");
  }
  LOGO_REQUIRE(aligned16(local) && aligned16(glob), LOGO_ERR_INVALID, "local and glob must be 16-byte aligned");
  return LOGO_OK;
}

}  // namespace logo

extern "C" int logo_fuse_fwd(const void* local, const void* glob, const void* gate, int gate_dtype, const void* thres,
                             int thres_dtype, const void* w_local, const void* w_global, int w_dtype, void* out,
                             int n_tokens, int h, int d, float eps, int use_norm, logo_stream_t stream) {
  using namespace logo;
  int rc = check_fuse(local, glob, gate, gate_dtype, thres, thres_dtype, w_local, w_global, w_dtype, n_tokens, h, d,
                      use_norm);
  if (rc) return rc;
  if (n_tokens == 0) return LOGO_OK;
  LOGO_REQUIRE(out && aligned16(out), LOGO_ERR_INVALID, "out must be a 16-byte aligned pointer");
  fuse_fwd_kernel<<<fuse_grid(n_tokens), FUSE_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)local, (const __nv_bfloat16*)glob, (const __nv_bfloat16*)gate, thres, thres_dtype, w_local,
      w_global, w_dtype, (__nv_bfloat16*)out, n_tokens, h, eps, use_norm);
  LOGO_CHECK_CUDA(cudaGetLastError());
  return LOGO_OK;
}

extern "C" size_t logo_fuse_bwd_workspace_bytes(int n_tokens) {
  if (n_tokens < 0) n_tokens = 0;
  return (size_t)logo::fuse_grid(n_tokens) * 2 * logo::FUSE_D * sizeof(float);
}

extern "C" int logo_fuse_bwd(const void* d_out, const void* local, const void* glob, const void* gate, int gate_dtype,
                             const void* thres, int thres_dtype, const void* w_local, const void* w_global,
                             int w_dtype, void* d_local, void* d_glob, void* d_gate, void* d_w_local,
                             void* d_w_global, int n_tokens, int h, int d, float eps, int use_norm, void* workspace,
                             size_t workspace_bytes, logo_stream_t stream_) {
  using namespace logo;
  cudaStream_t stream = (cudaStream_t)stream_;
  int rc = check_fuse(local, glob, gate, gate_dtype, thres, thres_dtype, w_local, w_global, w_dtype, n_tokens, h, d,
                      use_norm);
  if (rc) return rc;
  const int grid = fuse_grid(n_tokens);
  const size_t need = (size_t)grid * 2 * FUSE_D * sizeof(float);
  LOGO_REQUIRE(workspace && workspace_bytes >= need, LOGO_ERR_WORKSPACE, "fuse backward workspace too small: need %zu",
               need);
  LOGO_REQUIRE(n_tokens == 0 || (d_out && d_local && d_glob && d_gate), LOGO_ERR_INVALID,
               "gradient pointers must not be NULL");
  LOGO_REQUIRE(aligned16(d_out) && aligned16(d_local) && aligned16(d_glob), LOGO_ERR_INVALID,
               "gradient tensors must be 16-byte aligned");
  if (n_tokens == 0) {
    LOGO_CHECK_CUDA(cudaMemsetAsync(workspace, 0, need, stream));
  } else {
    fuse_bwd_kernel<<<grid, FUSE_THREADS, 0, stream>>>(
        (const __nv_bfloat16*)d_out, (const __nv_bfloat16*)local, (const __nv_bfloat16*)glob,
        (const __nv_bfloat16*)gate, thres, thres_dtype, w_local, w_global, w_dtype, (__nv_bfloat16*)d_local,
        (__nv_bfloat16*)d_glob, (__nv_bfloat16*)d_gate, static_cast<float*>(workspace), n_tokens, h, eps, use_norm);
    LOGO_CHECK_CUDA(cudaGetLastError());
  }
  if (use_norm && (d_w_local || d_w_global)) {
    fuse_bwd_finish_kernel<<<1, 1024, 0, stream>>>(static_cast<const float*>(workspace), grid, d_w_local, d_w_global,
                                                  w_dtype);
    LOGO_CHECK_CUDA(cudaGetLastError());
  }
  return LOGO_OK;
}
