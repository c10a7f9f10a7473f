// Definitions shared by the backward attention kernels (the two-kernel path of attn_bwd.cu and the
// single-pass kernel of attn_bwd_fused.cu): argument block, the element-wise helpers that turn
// score tiles into probabilities and dS, and the decoding of a (key tile, kv head) work item.
#pragma once

#include "attn_common.cuh"
#include "host_common.cuh"

namespace logo {

struct BwdArgs {
  const int64_t* q_idx;       // null: identity (local branch)
  const int32_t* sq_ptr;      // [1] number of selected rows (with q_idx)
  const int32_t* pos_ids;
  const int32_t* cu_q;
  const int32_t* cu_k;
  const int32_t* tile_off_q;  // [n_seq+1] prefix of 128-row query tiles
  const int32_t* n_qtiles;
  const int32_t* tile_off_k;  // [n_seq+1] prefix of 128-key tiles
  const int32_t* n_ktiles;
  int* counter_dq;            // [1] zeroed before the launch: next unclaimed item of the dQ kernel
  int* counter_dkv;           // [1] same for the dK/dV kernel
  const float* lse_sel;       // [hq][cap] head-major, compact rows
  const float* delta_sel;     // [hq][cap]
  int cap;
  __nv_bfloat16* dq;          // [n_tokens, hq, 128]
  __nv_bfloat16* dk;          // [n_tokens, h, 128]
  __nv_bfloat16* dv;
  int n_seq, n_tokens, hq, h, window;
  float scale, scale_log2;
  int* status;
};

constexpr int BWD_THREADS = 320;      // dK/dV kernel: 8 element-wise warps + producer + MMA
constexpr int DQ_EW_WARPS = 16;        // dQ kernel: 16 element-wise warps (four per scheduler), 32 columns each
constexpr int DQ_THREADS = (DQ_EW_WARPS + 2) * 32;
constexpr int BWD_SMEM_BYTES = 6 * TILE_BYTES + 1024;

__device__ __forceinline__ int bwd_row_position(const BwdArgs& a, int bos_q, int r) {
  return a.q_idx ? __ldg(a.pos_ids + bos_q + r) : r;
}


// r[i] <- bits of p = 2^(s*c - lse) for 32 scores of one row; keys outside [key_lo, key_hi] give 0.
// MASK is a template parameter so that the unmasked (by far most frequent) instance is branch-free:
// 0 no mask, 1 causal only (one comparison per element), 2 causal + window.
template <int MASK>
__device__ __forceinline__ void prob_chunk_row_t(uint32_t (&r)[32], float c, float lse, int k0, int key_hi, int key_lo) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float pv = fast_exp2(fmaf(__uint_as_float(r[i]), c, -lse));
    if (MASK == 1) pv = (k0 + i <= key_hi) ? pv : 0.f;
    if (MASK == 2) pv = (k0 + i <= key_hi && k0 + i >= key_lo) ? pv : 0.f;
    r[i] = __float_as_uint(pv);
  }
}

__device__ __forceinline__ void prob_chunk_row(uint32_t (&r)[32], float c, float lse, bool masked, int k0, int key_hi,
                                               int key_lo) {
  if (!masked) prob_chunk_row_t<0>(r, c, lse, k0, key_hi, key_lo);
  else if (key_lo == INT32_MIN) prob_chunk_row_t<1>(r, c, lse, k0, key_hi, key_lo);
  else prob_chunk_row_t<2>(r, c, lse, k0, key_hi, key_lo);
}

// pk[i] <- bf16x2 of p * (dp - delta) for 32 elements of one row
__device__ __forceinline__ void ds_pack_chunk_row(const uint32_t (&p)[32], const uint32_t (&dp)[32], float delta,
                                                  uint32_t* pk) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float d0 = __uint_as_float(p[2 * i]) * (__uint_as_float(dp[2 * i]) - delta);
    const float d1 = __uint_as_float(p[2 * i + 1]) * (__uint_as_float(dp[2 * i + 1]) - delta);
    pk[i] = pack_bf16x2(d0, d1);
  }
}

// Column-wise variants for the transposed tiles of the dK/dV kernel: lse / delta / position differ per
// column and come from shared memory (16-byte broadcast loads). MASK as above; an invalid key row
// (past the end of the sequence) is passed as key_pos = INT32_MAX, which no query position reaches.
template <int MASK>
__device__ __forceinline__ void prob_chunk_col_t(uint32_t (&r)[32], float c, const float* __restrict__ lse_s,
                                                 const int* __restrict__ pos_s, int key_pos, int window) {
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const float4 l4 = *reinterpret_cast<const float4*>(lse_s + 4 * g);
    const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
    int pv4[4] = {0, 0, 0, 0};
    if (MASK != 0) {
      const int4 q4 = *reinterpret_cast<const int4*>(pos_s + 4 * g);
      pv4[0] = q4.x;
      pv4[1] = q4.y;
      pv4[2] = q4.z;
      pv4[3] = q4.w;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float pv = fast_exp2(fmaf(__uint_as_float(r[4 * g + e]), c, -lv[e]));
      if (MASK == 1) pv = (key_pos <= pv4[e]) ? pv : 0.f;
      if (MASK == 2) pv = (key_pos <= pv4[e] && key_pos >= pv4[e] - window) ? pv : 0.f;
      r[4 * g + e] = __float_as_uint(pv);
    }
  }
}

__device__ __forceinline__ void prob_chunk_col(uint32_t (&r)[32], float c, const float* __restrict__ lse_s,
                                               const int* __restrict__ pos_s, bool masked, bool key_valid,
                                               int key_pos, int window) {
  const int kp = key_valid ? key_pos : INT32_MAX;
  if (!masked) prob_chunk_col_t<0>(r, c, lse_s, pos_s, kp, window);
  else if (window == 0) prob_chunk_col_t<1>(r, c, lse_s, pos_s, kp, window);
  else prob_chunk_col_t<2>(r, c, lse_s, pos_s, kp, window);
}

__device__ __forceinline__ void ds_pack_chunk_col(const uint32_t (&p)[32], const uint32_t (&dp)[32],
                                                  const float* __restrict__ delta_s, uint32_t* pk) {
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const float4 d4 = *reinterpret_cast<const float4*>(delta_s + 4 * g);
    const float d0 = __uint_as_float(p[4 * g]) * (__uint_as_float(dp[4 * g]) - d4.x);
    const float d1 = __uint_as_float(p[4 * g + 1]) * (__uint_as_float(dp[4 * g + 1]) - d4.y);
    const float d2 = __uint_as_float(p[4 * g + 2]) * (__uint_as_float(dp[4 * g + 2]) - d4.z);
    const float d3 = __uint_as_float(p[4 * g + 3]) * (__uint_as_float(dp[4 * g + 3]) - d4.w);
    pk[2 * g] = pack_bf16x2(d0, d1);
    pk[2 * g + 1] = pack_bf16x2(d2, d3);
  }
}

// Variants for score / dP tiles that already carry the row vectors (the single-pass kernel adds
// -lse / c to S^T and -delta to dP^T on the tensor core): p = 2^(s c), dS = p dp. Positions are only
// read on masked tiles.
template <int MASK>
__device__ __forceinline__ void prob_chunk_biased_t(uint32_t (&r)[32], float c, const int* __restrict__ pos_s, int key_pos,
                                                    int window) {
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    int pv4[4] = {0, 0, 0, 0};
    if (MASK != 0) {
      const int4 q4 = *reinterpret_cast<const int4*>(pos_s + 4 * g);
      pv4[0] = q4.x;
      pv4[1] = q4.y;
      pv4[2] = q4.z;
      pv4[3] = q4.w;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float pv = fast_exp2(__uint_as_float(r[4 * g + e]) * c);
      if (MASK == 1) pv = (key_pos <= pv4[e]) ? pv : 0.f;
      if (MASK == 2) pv = (key_pos <= pv4[e] && key_pos >= pv4[e] - window) ? pv : 0.f;
      r[4 * g + e] = __float_as_uint(pv);
    }
  }
}

__device__ __forceinline__ void prob_chunk_biased(uint32_t (&r)[32], float c, const int* __restrict__ pos_s, bool masked,
                                                  bool key_valid, int key_pos, int window) {
  const int kp = key_valid ? key_pos : INT32_MAX;
  if (!masked) prob_chunk_biased_t<0>(r, c, pos_s, kp, window);
  else if (window == 0) prob_chunk_biased_t<1>(r, c, pos_s, kp, window);
  else prob_chunk_biased_t<2>(r, c, pos_s, kp, window);
}

__device__ __forceinline__ void ds_pack_chunk_biased(const uint32_t (&p)[32], const uint32_t (&dp)[32], uint32_t* pk) {
#pragma unroll
  for (int i = 0; i < 16; ++i)
    pk[i] = pack_bf16x2(__uint_as_float(p[2 * i]) * __uint_as_float(dp[2 * i]),
                        __uint_as_float(p[2 * i + 1]) * __uint_as_float(dp[2 * i + 1]));
}

__device__ __forceinline__ void pack_chunk(const uint32_t (&p)[32], uint32_t* pk) {
#pragma unroll
  for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(__uint_as_float(p[2 * i]), __uint_as_float(p[2 * i + 1]));
}

struct DkvItem {
  int kvh, bos_q, bos_k, nsel, len_k, kv_start, i0, i_end;
};

// first index in [0, n) with pos[idx] >= x (pos ascending)
__device__ __forceinline__ int lower_bound_pos(const int32_t* __restrict__ pos, int n, int x) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(pos + mid) < x) lo = mid + 1; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ void dkv_decode_item(const BwdArgs& a, int w, DkvItem& it) {
  const int tile_g = w / a.h;
  it.kvh = w % a.h;
  const int seq = find_sequence(a.tile_off_k, a.n_seq, tile_g);
  const int tile_l = tile_g - __ldg(a.tile_off_k + seq);
  it.bos_q = __ldg(a.cu_q + seq);
  it.nsel = max(__ldg(a.cu_q + seq + 1) - it.bos_q, 0);
  it.bos_k = __ldg(a.cu_k + seq);
  it.len_k = __ldg(a.cu_k + seq + 1) - it.bos_k;
  it.kv_start = tile_l * TILE;
  int first, last;  // compacted rows [first, last) can see some key of this tile
  if (a.q_idx) {
    const int32_t* pos = a.pos_ids + it.bos_q;
    first = lower_bound_pos(pos, it.nsel, it.kv_start);
    last = a.window > 0 ? lower_bound_pos(pos, it.nsel, it.kv_start + TILE + a.window) : it.nsel;
  } else {
    first = min(it.kv_start, it.nsel);
    last = a.window > 0 ? min(it.nsel, it.kv_start + TILE + a.window) : it.nsel;
  }
  it.i0 = first / TILE;
  it.i_end = (last + TILE - 1) / TILE;
  if (last <= first) it.i_end = it.i0;
}

// Single-pass backward (attn_bwd_fused.cu): dK, dV and dQ from one evaluation of S and dP per
// (query tile, key tile) pair. dQ is accumulated with fp32 reductions into `dq_acc`
// ([rows][hq][128], zeroed by the preprocess kernel) and converted by bwd_dq_finish_kernel.
int launch_attn_bwd_fused(const CUtensorMap& tm_q, const CUtensorMap& tm_do, const CUtensorMap& tm_k,
                          const CUtensorMap& tm_v, const BwdArgs& a, float* dq_acc, const __nv_bfloat16* vec_split,
                          const int32_t* sq_ptr, cudaStream_t stream);

}  // namespace logo
