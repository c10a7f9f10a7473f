// Token cross-entropy over lm_head logits with the model's packed-sequence label shift.
//
// Two kernels:
//   shift_labels_kernel: target of token i = labels[i + 1], except for the last token of every
//       packed sequence (and for labels equal to ignore_index), which get ignore_index -- the
//       `shift_labels[cu_seqlens[1:-1] - 1] = -100` of the reference's loss;
//   ce_rows_kernel: one CTA per row of bf16 logits: log-sum-exp in fp32 (first pass), loss =
//       lse - logit[target]; optionally a second pass (the row is still in L2) overwrites the
//       logits with the gradient (softmax - onehot) * scale as bf16, so the caller can feed it
//       straight to the two lm_head gradient products without materialising fp32 logits.
// Bytes per row (HBM): vocab * 2 read + vocab * 2 written.
#include "host_common.cuh"

namespace logo {

constexpr int CE_THREADS = 256;

__global__ void __launch_bounds__(256)
    shift_labels_kernel(const int64_t* __restrict__ labels, const int32_t* __restrict__ cu, int n_seq, int n_tokens,
                        long long ignore_index, int64_t* __restrict__ targets, int* __restrict__ n_valid) {
  int valid = 0;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_tokens; i += gridDim.x * blockDim.x) {
    // sequence that owns token i: largest s with cu[s] <= i
    int lo = 0, hi = n_seq;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (__ldg(cu + mid) <= i) lo = mid; else hi = mid;
    }
    const int end = __ldg(cu + lo + 1);
    long long t = ignore_index;
    if (i + 1 < end) t = __ldg(labels + i + 1);
    targets[i] = t;
    valid += (t != ignore_index);
  }
  valid = __reduce_add_sync(0xffffffffu, valid);
  if ((threadIdx.x & 31) == 0 && valid) atomicAdd(n_valid, valid);
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&x)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(p[i]);
    x[2 * i] = f.x;
    x[2 * i + 1] = f.y;
  }
}

// logits: rows of `vocab` bf16 at `row_stride` elements; vocab % 8 == 0 and rows 16-byte aligned.
// n_valid: device scalar, number of rows whose target is not ignore_index (gradient scale = upstream / n_valid).
template <bool WRITE_GRAD>
__global__ void __launch_bounds__(CE_THREADS)
    ce_rows_kernel(__nv_bfloat16* __restrict__ logits, long long row_stride, const int64_t* __restrict__ targets,
                   long long ignore_index, float* __restrict__ row_loss, const int* __restrict__ n_valid, float upstream,
                   int vocab, int* status) {
  __shared__ float s_m[CE_THREADS / 32], s_s[CE_THREADS / 32];
  const int row = blockIdx.x, tid = threadIdx.x;
  __nv_bfloat16* x = logits + (size_t)row * row_stride;
  const long long t = __ldg(targets + row);
  const int chunks = vocab >> 3;
  if (t == ignore_index || t < 0 || t >= vocab) {
    if (t != ignore_index && tid == 0 && status) atomicCAS(status, 0, 2 /* DEV_BAD_INDEX */);
    if (tid == 0) row_loss[row] = 0.f;
    if (WRITE_GRAD)
      for (int c = tid; c < chunks; c += CE_THREADS) reinterpret_cast<uint4*>(x)[c] = make_uint4(0, 0, 0, 0);
    return;
  }
  constexpr float LOG2E = 1.4426950408889634f;
  float m = -INFINITY, s = 0.f;   // running maximum and sum of 2^((x - m) * log2e)
  for (int c = tid; c < chunks; c += CE_THREADS) {
    float v[8];
    unpack8(reinterpret_cast<const uint4*>(x)[c], v);
    float cm = v[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) cm = fmaxf(cm, v[i]);
    const float m_new = fmaxf(m, cm);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += exp2f((v[i] - m_new) * LOG2E);
    s = s * exp2f((m - m_new) * LOG2E) + acc;
    m = m_new;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, off), s2 = __shfl_xor_sync(0xffffffffu, s, off);
    const float mn = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * exp2f((m - mn) * LOG2E)) + (m2 == -INFINITY ? 0.f : s2 * exp2f((m2 - mn) * LOG2E));
    m = mn;
  }
  if ((tid & 31) == 0) {
    s_m[tid >> 5] = m;
    s_s[tid >> 5] = s;
  }
  __syncthreads();
  m = s_m[0];
  s = s_s[0];
#pragma unroll
  for (int w = 1; w < CE_THREADS / 32; ++w) {
    const float m2 = s_m[w], s2 = s_s[w];
    const float mn = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * exp2f((m - mn) * LOG2E)) + (m2 == -INFINITY ? 0.f : s2 * exp2f((m2 - mn) * LOG2E));
    m = mn;
  }
  const float lse = m + logf(s);
  if (tid == 0) row_loss[row] = lse - __bfloat162float(x[t]);
  if (WRITE_GRAD) {
    const int nv = max(__ldg(n_valid), 1);
    const float scale = upstream / (float)nv;
    const float lse2 = lse * LOG2E;
    const int t_chunk = (int)(t >> 3), t_lane = (int)(t & 7);
    for (int c = tid; c < chunks; c += CE_THREADS) {
      float v[8];
      unpack8(reinterpret_cast<const uint4*>(x)[c], v);
      uint32_t out[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float g0 = exp2f(v[2 * i] * LOG2E - lse2), g1 = exp2f(v[2 * i + 1] * LOG2E - lse2);
        if (c == t_chunk) {
          if (2 * i == t_lane) g0 -= 1.f;
          if (2 * i + 1 == t_lane) g1 -= 1.f;
        }
        const __nv_bfloat162 p = __floats2bfloat162_rn(g0 * scale, g1 * scale);
        out[i] = *reinterpret_cast<const uint32_t*>(&p);
      }
      reinterpret_cast<uint4*>(x)[c] = make_uint4(out[0], out[1], out[2], out[3]);
    }
  }
}

}  // namespace logo

extern "C" int logo_shift_labels(const int64_t* labels, const int32_t* cu_seqlens, int n_seq, int n_tokens,
                                 long long ignore_index, int64_t* targets, int32_t* n_valid, logo_stream_t stream_) {
  using namespace logo;
  cudaStream_t stream = (cudaStream_t)stream_;
  LOGO_REQUIRE(n_tokens >= 0 && n_seq >= 0, LOGO_ERR_INVALID, "n_tokens and n_seq must be non-negative");
  LOGO_REQUIRE(n_valid != nullptr, LOGO_ERR_INVALID, "n_valid must not be NULL");
  LOGO_CHECK_CUDA(cudaMemsetAsync(n_valid, 0, sizeof(int32_t), stream));
  if (n_tokens == 0) return LOGO_OK;
  LOGO_REQUIRE(labels && cu_seqlens && targets && n_seq > 0, LOGO_ERR_INVALID,
               "labels, cu_seqlens and targets must not be NULL");
  const int grid = min((n_tokens + 255) / 256, sm_count() * 8);
  shift_labels_kernel<<<grid, 256, 0, stream>>>(labels, cu_seqlens, n_seq, n_tokens, ignore_index, targets, n_valid);
  LOGO_CHECK_CUDA(cudaGetLastError());
  return LOGO_OK;
}

extern "C" int logo_ce_rows(void* logits, long long row_stride, const int64_t* targets, long long ignore_index,
                            float* row_loss, const int32_t* n_valid, float upstream, int rows, int vocab,
                            int write_grad, int32_t* status, logo_stream_t stream_) {
  using namespace logo;
  cudaStream_t stream = (cudaStream_t)stream_;
  LOGO_REQUIRE(rows >= 0 && vocab > 0, LOGO_ERR_INVALID, "rows must be non-negative and vocab positive");
  if (rows == 0) return LOGO_OK;
  LOGO_REQUIRE(logits && targets && row_loss, LOGO_ERR_INVALID, "logits, targets and row_loss must not be NULL");
  LOGO_REQUIRE(!write_grad || n_valid, LOGO_ERR_INVALID, "n_valid is needed to scale the gradient");
  LOGO_REQUIRE(vocab % 8 == 0 && row_stride % 8 == 0 && row_stride >= vocab && aligned16(logits), LOGO_ERR_UNSUPPORTED,
               "vocab (%d) and the row stride must be multiples of 8 and the logits 16-byte aligned", vocab);
  if (write_grad)
    ce_rows_kernel<true><<<rows, CE_THREADS, 0, stream>>>((__nv_bfloat16*)logits, row_stride, targets, ignore_index,
                                                         row_loss, n_valid, upstream, vocab, status);
  else
    ce_rows_kernel<false><<<rows, CE_THREADS, 0, stream>>>((__nv_bfloat16*)logits, row_stride, targets, ignore_index,
                                                          row_loss, n_valid, upstream, vocab, status);
  LOGO_CHECK_CUDA(cudaGetLastError());
  return LOGO_OK;
}
