// Decode-time attention over the KV cache and the in-place cache append (HBM-bound).
//
// Cache layout (bf16, head-major so that KV-head sharding is a slice):
//   global branch: k_cache, v_cache [B, H, t_max, 128]; token p of sequence b at row p
//   local branch : k_ring,  v_ring  [B, H, ring, 128];  token p at row p % ring, ring = window + 1
//
// decode_attn_kernel: grid (splits + 1, H, B). CTAs with blockIdx.x < splits stream one
// chunk of DECODE_CHUNK cached keys of an ACTIVE sequence (gate >= thres, evaluated on the
// device -- inactive sequences cost nothing) and write an un-normalised partial
// (max, sum, acc[128]); the CTA with blockIdx.x == splits does the local branch over the
// ring. 16 lanes own one key row (16 bytes per lane), so every load instruction of a warp
// covers two full 256-byte rows. decode_combine_kernel merges the partials.
//
// Bytes per step and layer: sum over active sequences of 2 * ctx * H * 256 (global K and V)
// + sum over all sequences of 2 * min(ctx, ring) * H * 256 (local) + O(B * HQ * 128).
#include "host_common.cuh"
#include "ptx.cuh"

#include <cuda_fp16.h>

namespace logo {

constexpr int DEC_THREADS = 256;
constexpr int DEC_D = 128;
constexpr int DECODE_CHUNK = 1024;
constexpr int DEC_PART = DEC_D + 4;  // floats per partial: max, sum, 2 pad, acc[128]

__device__ __forceinline__ float dec_scalar(const void* p, int dtype, int i) {
  if (dtype == LOGO_DTYPE_F32) return static_cast<const float*>(p)[i];
  if (dtype == LOGO_DTYPE_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ void dec_unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ float sum16(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 8);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  return x;
}

struct DecodeArgs {
  const __nv_bfloat16* q_local;
  const __nv_bfloat16* q_global;
  const __nv_bfloat16* k_ring;
  const __nv_bfloat16* v_ring;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int32_t* ctx_lens;
  const void* gate;
  const void* thres;
  int gate_dtype, thres_dtype;
  __nv_bfloat16* o_local;
  __nv_bfloat16* o_global;
  float* partials;  // [B, HQ, splits, DEC_PART]
  int batch, hq, h, ring, t_max, splits;
  float scale_log2;
  int* status;
};

template <int G>
__global__ void __launch_bounds__(DEC_THREADS)
    decode_attn_kernel(const DecodeArgs a) {
  __shared__ float s_m[G][DEC_THREADS / 16];
  __shared__ float s_l[G][DEC_THREADS / 16];
  __shared__ float s_acc[G][DEC_THREADS / 16][DEC_D];

  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const bool is_local = (split == a.splits);
  const int tid = threadIdx.x;
  const int hw = tid >> 4;              // half-warp 0..15
  const int col = (tid & 15) * 8;

  int n = __ldg(a.ctx_lens + b);
  if (n < 0 || n > a.t_max) {
    if (tid == 0 && a.status) atomicCAS(a.status, 0, (int)DEV_BAD_INDEX);
    n = max(0, min(n, a.t_max));
  }
  int k_begin, k_end;
  const __nv_bfloat16 *kbase, *vbase, *qbase;
  if (is_local) {
    k_begin = 0;
    k_end = min(n, a.ring);
    kbase = a.k_ring + ((size_t)b * a.h + kvh) * a.ring * DEC_D;
    vbase = a.v_ring + ((size_t)b * a.h + kvh) * a.ring * DEC_D;
    qbase = a.q_local;
  } else {
    const bool active = dec_scalar(a.gate, a.gate_dtype, b) >= dec_scalar(a.thres, a.thres_dtype, 0);
    k_begin = split * DECODE_CHUNK;
    k_end = min(n, k_begin + DECODE_CHUNK);
    if (!active || k_begin >= k_end) return;
    kbase = a.k_cache + ((size_t)b * a.h + kvh) * a.t_max * DEC_D;
    vbase = a.v_cache + ((size_t)b * a.h + kvh) * a.t_max * DEC_D;
    qbase = a.q_global;
  }

  float q[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float t[8];
    dec_unpack8(__ldg(reinterpret_cast<const uint4*>(qbase + ((size_t)b * a.hq + kvh * G + g) * DEC_D + col)), t);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[g][i] = t[i] * a.scale_log2;
  }
  float m[G], l[G], acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  }

  constexpr int UNROLL = 4;
  constexpr int HW = DEC_THREADS / 16;
  // The trip count is uniform across the CTA: the 16-lane reductions shuffle over the full warp.
  for (int k0 = k_begin; k0 < k_end; k0 += HW * UNROLL) {
    uint4 kv[UNROLL], vv[UNROLL];
    bool ok[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int key = k0 + u * HW + hw;
      ok[u] = key < k_end;
      const size_t off = (size_t)(ok[u] ? key : k_begin) * DEC_D + col;
      kv[u] = __ldg(reinterpret_cast<const uint4*>(kbase + off));
      vv[u] = __ldg(reinterpret_cast<const uint4*>(vbase + off));
    }
    float kf[UNROLL][8];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) dec_unpack8(kv[u], kf[u]);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) d = fmaf(q[g][i], kf[u][i], d);
        d = sum16(d);
        s[u] = ok[u] ? d : -INFINITY;
      }
      float m_new = m[g];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) m_new = fmaxf(m_new, s[u]);
      if (m_new > -INFINITY) {
        const float alpha = fast_exp2(m[g] - m_new);
        l[g] *= alpha;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] *= alpha;
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const float p = fast_exp2(s[u] - m_new);
          l[g] += p;
          float vf[8];
          dec_unpack8(vv[u], vf);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(p, vf[i], acc[g][i]);
        }
        m[g] = m_new;
      }
    }
  }

  // ---- merge the 16 half-warps ----
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if ((tid & 15) == 0) {
      s_m[g][hw] = m[g];
      s_l[g][hw] = l[g];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) s_acc[g][hw][col + i] = acc[g][i];
  }
  __syncthreads();
  for (int idx = tid; idx < G * DEC_D; idx += DEC_THREADS) {
    const int g = idx / DEC_D, c = idx % DEC_D;
    float M = -INFINITY;
#pragma unroll
    for (int k = 0; k < HW; ++k) M = fmaxf(M, s_m[g][k]);
    float L = 0.f, o = 0.f;
#pragma unroll
    for (int k = 0; k < HW; ++k) {
      const float wgt = (s_m[g][k] == -INFINITY) ? 0.f : fast_exp2(s_m[g][k] - M);
      L = fmaf(wgt, s_l[g][k], L);
      o = fmaf(wgt, s_acc[g][k][c], o);
    }
    const int hq_idx = kvh * G + g;
    if (is_local) {
      a.o_local[((size_t)b * a.hq + hq_idx) * DEC_D + c] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
    } else {
      float* part = a.partials + (((size_t)b * a.hq + hq_idx) * a.splits + split) * DEC_PART;
      part[4 + c] = o;
      if (c == 0) {
        part[0] = M;
        part[1] = L;
      }
    }
  }
}

// grid (HQ, B), 128 threads: merges the split partials of the global branch
__global__ void __launch_bounds__(DEC_D)
    decode_combine_kernel(const DecodeArgs a) {
  const int hq_idx = blockIdx.x, b = blockIdx.y, c = threadIdx.x;
  __nv_bfloat16* dst = a.o_global + ((size_t)b * a.hq + hq_idx) * DEC_D + c;
  const bool active = dec_scalar(a.gate, a.gate_dtype, b) >= dec_scalar(a.thres, a.thres_dtype, 0);
  const int n = max(0, min(__ldg(a.ctx_lens + b), a.t_max));
  const int used = (n + DECODE_CHUNK - 1) / DECODE_CHUNK;
  if (!active || used == 0) {
    *dst = __float2bfloat16_rn(0.f);
    return;
  }
  const float* part = a.partials + ((size_t)b * a.hq + hq_idx) * a.splits * DEC_PART;
  float M = -INFINITY;
  for (int s = 0; s < used; ++s) M = fmaxf(M, part[(size_t)s * DEC_PART]);
  float L = 0.f, o = 0.f;
  for (int s = 0; s < used; ++s) {
    const float wgt = fast_exp2(part[(size_t)s * DEC_PART] - M);
    L = fmaf(wgt, part[(size_t)s * DEC_PART + 1], L);
    o = fmaf(wgt, part[(size_t)s * DEC_PART + 4 + c], o);
  }
  *dst = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
}

// ---------------------------------------------------------------------------------------
// cache append: new tokens [B, t_new, H, 128] (element strides given) -> ring and full cache
// ---------------------------------------------------------------------------------------
struct AppendArgs {
  const __nv_bfloat16* k_local;
  const __nv_bfloat16* v_local;
  const __nv_bfloat16* k_global;
  const __nv_bfloat16* v_global;
  long long sb, st, sh;   // element strides of the four inputs (batch, token, head)
  __nv_bfloat16* k_ring;
  __nv_bfloat16* v_ring;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  const int32_t* start_lens;
  int start, batch, t_new, h, ring, t_max;
  int* status;
};

__global__ void __launch_bounds__(256)
    cache_append_kernel(const AppendArgs a) {
  const int lane16 = threadIdx.x & 15;
  const long long rows = (long long)a.batch * a.t_new * a.h;
  for (long long r = (long long)blockIdx.x * 16 + (threadIdx.x >> 4); r < rows; r += (long long)gridDim.x * 16) {
    const int hh = (int)(r % a.h);
    const int t = (int)((r / a.h) % a.t_new);
    const int b = (int)(r / ((long long)a.h * a.t_new));
    const int pos = (a.start_lens ? __ldg(a.start_lens + b) : a.start) + t;
    const size_t src = (size_t)(b * a.sb + t * a.st + hh * a.sh) + lane16 * 8;
    if (pos < 0 || pos >= a.t_max) {
      if (lane16 == 0 && a.status) atomicCAS(a.status, 0, (int)DEV_BAD_INDEX);
      continue;
    }
    if (a.k_cache) {
      const size_t dst = (((size_t)b * a.h + hh) * a.t_max + pos) * DEC_D + lane16 * 8;
      *reinterpret_cast<uint4*>(a.k_cache + dst) = __ldg(reinterpret_cast<const uint4*>(a.k_global + src));
      *reinterpret_cast<uint4*>(a.v_cache + dst) = __ldg(reinterpret_cast<const uint4*>(a.v_global + src));
    }
    if (a.k_ring && t >= a.t_new - a.ring) {   // older tokens would be overwritten by later ones
      const size_t dst = (((size_t)b * a.h + hh) * a.ring + (pos % a.ring)) * DEC_D + lane16 * 8;
      *reinterpret_cast<uint4*>(a.k_ring + dst) = __ldg(reinterpret_cast<const uint4*>(a.k_local + src));
      *reinterpret_cast<uint4*>(a.v_ring + dst) = __ldg(reinterpret_cast<const uint4*>(a.v_local + src));
    }
  }
}

static int decode_splits(int max_ctx) { return max_ctx <= 0 ? 1 : (max_ctx + DECODE_CHUNK - 1) / DECODE_CHUNK; }

}  // namespace logo

extern "C" size_t logo_decode_workspace_bytes(int batch, int hq, int max_ctx) {
  if (batch <= 0 || hq <= 0) return 256;
  return (size_t)batch * hq * logo::decode_splits(max_ctx) * logo::DEC_PART * sizeof(float) + 256;
}

extern "C" int logo_decode_attn(const void* q_local, const void* q_global, const void* k_ring, const void* v_ring,
                                int ring, const void* k_cache, const void* v_cache, int t_max,
                                const int32_t* ctx_lens, const void* gate, int gate_dtype, const void* thres,
                                int thres_dtype, void* o_local, void* o_global, int batch, int hq, int h, int d,
                                int max_ctx, float scale, void* workspace, size_t workspace_bytes, int32_t* status,
                                logo_stream_t stream_) {
  using namespace logo;
  cudaStream_t stream = (cudaStream_t)stream_;
  LOGO_REQUIRE(d == DEC_D, LOGO_ERR_UNSUPPORTED, "head_dim %d is not supported (only 128)", d);
  LOGO_REQUIRE(batch >= 0 && hq > 0 && h > 0 && hq % h == 0, LOGO_ERR_INVALID, "bad batch / head counts");
  const int G = hq / h;
  LOGO_REQUIRE(G == 1 || G == 2 || G == 4, LOGO_ERR_UNSUPPORTED, "GQA group size %d is not supported", G);
  LOGO_REQUIRE(ring > 0 && t_max > 0 && max_ctx >= 0 && max_ctx <= t_max, LOGO_ERR_INVALID,
               "need ring > 0, t_max > 0 and 0 <= max_ctx <= t_max");
  if (batch == 0) return LOGO_OK;
  LOGO_REQUIRE(q_local && q_global && k_ring && v_ring && k_cache && v_cache && ctx_lens && gate && thres && o_local &&
                   o_global,
               LOGO_ERR_INVALID, "decode pointers must not be NULL");
  LOGO_REQUIRE(aligned16(q_local) && aligned16(q_global) && aligned16(k_ring) && aligned16(v_ring) &&
                   aligned16(k_cache) && aligned16(v_cache),
               LOGO_ERR_INVALID, "decode tensors must be 16-byte aligned");
  LOGO_REQUIRE(gate_dtype >= LOGO_DTYPE_BF16 && gate_dtype <= LOGO_DTYPE_F16 && thres_dtype >= LOGO_DTYPE_BF16 &&
                   thres_dtype <= LOGO_DTYPE_F16,
               LOGO_ERR_INVALID, "gate and threshold must be bf16, fp16 or fp32");
  LOGO_REQUIRE(workspace && workspace_bytes >= logo_decode_workspace_bytes(batch, hq, max_ctx), LOGO_ERR_WORKSPACE,
               "decode workspace too small: need %zu bytes", logo_decode_workspace_bytes(batch, hq, max_ctx));
  DecodeArgs a{};
  a.q_local = (const __nv_bfloat16*)q_local;
  a.q_global = (const __nv_bfloat16*)q_global;
  a.k_ring = (const __nv_bfloat16*)k_ring;
  a.v_ring = (const __nv_bfloat16*)v_ring;
  a.k_cache = (const __nv_bfloat16*)k_cache;
  a.v_cache = (const __nv_bfloat16*)v_cache;
  a.ctx_lens = ctx_lens;
  a.gate = gate;
  a.thres = thres;
  a.gate_dtype = gate_dtype;
  a.thres_dtype = thres_dtype;
  a.o_local = (__nv_bfloat16*)o_local;
  a.o_global = (__nv_bfloat16*)o_global;
  a.partials = static_cast<float*>(workspace);
  a.batch = batch;
  a.hq = hq;
  a.h = h;
  a.ring = ring;
  a.t_max = t_max;
  a.splits = decode_splits(max_ctx);
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  const dim3 grid(a.splits + 1, h, batch);
  switch (G) {
    case 1: decode_attn_kernel<1><<<grid, DEC_THREADS, 0, stream>>>(a); break;
    case 2: decode_attn_kernel<2><<<grid, DEC_THREADS, 0, stream>>>(a); break;
    default: decode_attn_kernel<4><<<grid, DEC_THREADS, 0, stream>>>(a); break;
  }
  LOGO_CHECK_CUDA(cudaGetLastError());
  decode_combine_kernel<<<dim3(hq, batch), DEC_D, 0, stream>>>(a);
  LOGO_CHECK_CUDA(cudaGetLastError());
  return LOGO_OK;
}

extern "C" int logo_cache_append(const void* k_local, const void* v_local, const void* k_global, const void* v_global,
                                 long long stride_b, long long stride_t, long long stride_h, void* k_ring,
                                 void* v_ring, int ring, void* k_cache, void* v_cache, int t_max,
                                 const int32_t* start_lens, int start, int batch, int t_new, int h, int d,
                                 int32_t* status, logo_stream_t stream) {
  using namespace logo;
  LOGO_REQUIRE(d == DEC_D, LOGO_ERR_UNSUPPORTED, "head_dim %d is not supported (only 128)", d);
  LOGO_REQUIRE(batch >= 0 && t_new >= 0 && h > 0, LOGO_ERR_INVALID, "bad batch / token / head counts");
  if (batch == 0 || t_new == 0) return LOGO_OK;
  LOGO_REQUIRE((k_ring == nullptr) == (v_ring == nullptr) && (k_cache == nullptr) == (v_cache == nullptr),
               LOGO_ERR_INVALID, "ring and cache pointers must come in k/v pairs");
  LOGO_REQUIRE(!k_ring || (k_local && v_local && ring > 0), LOGO_ERR_INVALID, "local states and ring size required");
  LOGO_REQUIRE(!k_cache || (k_global && v_global && t_max > 0), LOGO_ERR_INVALID, "global states and t_max required");
  LOGO_REQUIRE((stride_b % 8) == 0 && (stride_t % 8) == 0 && (stride_h % 8) == 0, LOGO_ERR_INVALID,
               "input strides must be multiples of 8 elements (16 bytes)");
  LOGO_REQUIRE(aligned16(k_local) && aligned16(v_local) && aligned16(k_global) && aligned16(v_global) &&
                   aligned16(k_ring) && aligned16(v_ring) && aligned16(k_cache) && aligned16(v_cache),
               LOGO_ERR_INVALID, "cache tensors must be 16-byte aligned");
  AppendArgs a{};
  a.k_local = (const __nv_bfloat16*)k_local;
  a.v_local = (const __nv_bfloat16*)v_local;
  a.k_global = (const __nv_bfloat16*)k_global;
  a.v_global = (const __nv_bfloat16*)v_global;
  a.sb = stride_b;
  a.st = stride_t;
  a.sh = stride_h;
  a.k_ring = (__nv_bfloat16*)k_ring;
  a.v_ring = (__nv_bfloat16*)v_ring;
  a.k_cache = (__nv_bfloat16*)k_cache;
  a.v_cache = (__nv_bfloat16*)v_cache;
  a.start_lens = start_lens;
  a.start = start;
  a.batch = batch;
  a.t_new = t_new;
  a.h = h;
  a.ring = ring;
  a.t_max = k_cache ? t_max : 0x7fffffff;
  a.status = status;
  const long long rows = (long long)batch * t_new * h;
  long long blocks = (rows + 15) / 16;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  cache_append_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(a);
  LOGO_CHECK_CUDA(cudaGetLastError());
  return LOGO_OK;
}
