// Forward attention for both LoGo branches on tcgen05 tensor cores.
//
//   global branch: query-sparse causal attention -- only the rows listed in q_idx are
//                  computed; K/V of every token of the sequence stay visible;
//   local branch : every row, keys [pos - window, pos].
//
// A work item is a pair of query tiles (2 x 128 compacted rows of one sequence and one head);
// the kernel is persistent (one CTA per SM claims items from a global counter through the record
// ring of attn_common.cuh). Twenty warps:
//   warps 0-7 / 8-15 : softmax groups for query tile 0 / 1, two threads per row: warps 0-3 (8-11) take
//                      keys 0-63 of the score tile and output columns 0-63, warps 4-7 (12-15) the other
//                      half; the two threads of a row exchange their maxima through shared memory
//   warp 16          : claims / decodes items, TMA producer of the 128-key K and V tiles (2-stage rings)
//   warp 17          : issues tcgen05.mma (whole warp walks the loop, an elected lane issues)
//   warps 18-19      : global branch: zero the output rows of the tokens the selection leaves out
// A tile's softmax sits on the chain scores -> softmax -> P*V -> next scores (P overwrites S); with one
// thread per row that step took about 2500 clocks against 1024 clocks of tensor-pipe work per tile, so
// the tiles' softmax phases overlapped and shared the special-function unit. Halving the row work per
// thread shortens the chain.
// Tensor memory (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each. The bf16
// probabilities of each column half overwrite the first 32 columns of that half's scores (so the
// two threads of a row never touch each other's columns) and are the A operand of the P*V
// product straight from tensor memory; V is consumed as an MN-major B operand so
// the [keys][128] tile is used as it lies in memory.
// Softmax runs in base 2 with a lazily updated row maximum: the running maximum is only
// raised (and O rescaled in tensor memory) when a row's new maximum exceeds it by more
// than 2^8, so most key tiles need no correction pass.
//
// Algorithmic work per work item: 4 * 128 * sum over its rows of (visible keys) FLOPs.
#include "attn_common.cuh"
#include "host_common.cuh"

namespace logo {

constexpr int FWD_SM_WARPS = 16;   // softmax warps: 2 tiles x 2 column halves x 4 row quarters
constexpr int FWD_THREADS = (FWD_SM_WARPS + 4) * 32;   // + producer, MMA issuer, two spare warps
constexpr int FWD_STAGES = 2;
constexpr int FWD_SMEM_BYTES = 2 * TILE_BYTES + 2 * FWD_STAGES * TILE_BYTES + 1024;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units
constexpr int FWD_MAX_ORDERED_SEQ = 16;    // up to this many sequences the work list is ordered by cost across sequences

struct FwdItem {
  int hq, kvh, bos_q, bos_k, row0;
  int nrows[2], min_pos[2], max_pos[2], jb[2], je[2];
  int JB, JE;
};

__device__ __forceinline__ void fwd_decode_item(const AttnArgs& a, int w, int total_pairs, FwdItem& it) {
  it.hq = w % a.hq;
  it.kvh = it.hq / (a.hq / a.h);
  int seq, pair_l;
  if (a.n_seq <= FWD_MAX_ORDERED_SEQ) {
    // Heaviest first over ALL sequences: the cost of a pair grows with its index p inside its sequence, so
    // the list goes by p, highest first, taking pair p of every sequence that has one (walking the sequences
    // one after the other would leave the heavy pairs of the last-walked sequence for the end of the
    // launch). g(L) = sum over sequences of max(pairs - L, 0) is the number of items with p >= L.
    const int k = w / a.hq;
    int np[FWD_MAX_ORDERED_SEQ];
    int max_np = 0;
#pragma unroll
    for (int s = 0; s < FWD_MAX_ORDERED_SEQ; ++s) {
      np[s] = s < a.n_seq ? __ldg(a.tile_off + s + 1) - __ldg(a.tile_off + s) : 0;
      max_np = max(max_np, np[s]);
    }
    auto at_or_above = [&](int L) {
      int g = 0;
#pragma unroll
      for (int s = 0; s < FWD_MAX_ORDERED_SEQ; ++s) g += max(np[s] - L, 0);
      return g;
    };
    int lo = 0, hi = max(max_np - 1, 0);   // smallest L with at_or_above(L + 1) <= k: the level of item k
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (at_or_above(mid + 1) <= k) hi = mid; else lo = mid + 1;
    }
    const int j = k - at_or_above(lo + 1);   // the j-th sequence with more than `lo` pairs
    seq = 0;
    int c = 0;
#pragma unroll
    for (int s = 0; s < FWD_MAX_ORDERED_SEQ; ++s) {
      if (np[s] > lo) {
        if (c == j) seq = s;
        ++c;
      }
    }
    pair_l = min(lo, max(np[seq] - 1, 0));
  } else {
    const int pair_g = total_pairs - 1 - w / a.hq;
    seq = find_sequence(a.tile_off, a.n_seq, pair_g);
    pair_l = pair_g - __ldg(a.tile_off + seq);
  }
  it.bos_q = __ldg(a.cu_q + seq);
  const int nsel = __ldg(a.cu_q + seq + 1) - it.bos_q;
  it.bos_k = __ldg(a.cu_k + seq);
  const int len_k = __ldg(a.cu_k + seq + 1) - it.bos_k;
  it.row0 = pair_l * 2 * TILE;
  it.JB = 0x7fffffff;
  it.JE = 0;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r0 = it.row0 + t * TILE;
    const int n = min(max(nsel - r0, 0), TILE);
    it.nrows[t] = n;
    it.min_pos[t] = it.max_pos[t] = 0;
    it.jb[t] = it.je[t] = 0;
    if (n > 0) {
      int lo = row_position(a, it.bos_q, r0);
      int hi = row_position(a, it.bos_q, r0 + n - 1);
      if (lo < 0 || hi >= len_k || lo > hi) {  // corrupted metadata: stay inside the sequence
        if (a.status) atomicCAS(a.status, 0, (int)DEV_BAD_INDEX);
        lo = max(min(lo, len_k - 1), 0);
        hi = max(min(hi, len_k - 1), lo);
      }
      it.min_pos[t] = lo;
      it.max_pos[t] = hi;
      it.je[t] = hi / TILE + 1;
      it.jb[t] = a.window > 0 ? max(lo - a.window, 0) / TILE : 0;
      it.JB = min(it.JB, it.jb[t]);
      it.JE = max(it.JE, it.je[t]);
    }
  }
  if (it.JE == 0) it.JB = 0;
}

__device__ __forceinline__ bool tile_active(const FwdItem& it, int t, int j) {
  return it.nrows[t] > 0 && j >= it.jb[t] && j < it.je[t];
}

// keys outside [key_lo, key_hi] get a score of -inf; WINDOWED = false: causal only, key_lo is ignored
template <bool WINDOWED>
__device__ __forceinline__ void mask_chunk_t(uint32_t (&r)[32], int k0, int key_hi, int key_lo) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int key = k0 + i;
    const bool ok = WINDOWED ? (key <= key_hi && key >= key_lo) : (key <= key_hi);
    if (!ok) r[i] = 0xff800000u;
  }
}

__device__ __forceinline__ void mask_chunk(uint32_t (&r)[32], int k0, int key_hi, int key_lo) {
  if (key_lo == INT32_MIN) mask_chunk_t<false>(r, k0, key_hi, key_lo);
  else mask_chunk_t<true>(r, k0, key_hi, key_lo);
}

__device__ __forceinline__ float max_chunk(const uint32_t (&r)[32]) {
  float m[4];
#pragma unroll
  for (int c4 = 0; c4 < 4; ++c4) {
    const uint32_t* v = r + 8 * c4;
    float x = fmax3(__uint_as_float(v[0]), __uint_as_float(v[1]), __uint_as_float(v[2]));
    x = fmax3(x, __uint_as_float(v[3]), __uint_as_float(v[4]));
    x = fmax3(x, __uint_as_float(v[5]), __uint_as_float(v[6]));
    m[c4] = fmaxf(x, __uint_as_float(v[7]));
  }
  return fmaxf(fmax3(m[0], m[1], m[2]), m[3]);
}

// p = 2^(s*c - mc) for 32 scores, packed to 16 bf16x2 words; the fp32 values are summed into l0 / l1
__device__ __forceinline__ void exp_pack_chunk(const uint32_t (&r)[32], float c, float mc, uint32_t (&pk)[16],
                                               float& l0, float& l1) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float p0 = fast_exp2(fmaf(__uint_as_float(r[2 * i]), c, -mc));
    const float p1 = fast_exp2(fmaf(__uint_as_float(r[2 * i + 1]), c, -mc));
    l0 += p0;
    l1 += p1;
    pk[i] = pack_bf16x2(p0, p1);
  }
}

// One softmax group (256 threads, `idx` = thread index inside it) copies the query rows of its
// tile into 128-byte swizzled shared memory. All eight index loads, then all eight row loads,
// are issued back to back (no branch between them), so the copy costs two memory round trips.
__device__ __forceinline__ void gather_query_tile(const AttnArgs& a, const FwdItem& it, int t, int idx, uint8_t* sQt) {
  const int nrows = it.nrows[t];
  const int r_base = it.row0 + t * TILE;
  const int ch = idx & 15;  // 16-byte chunk of the 256-byte row
  uint32_t tok[8];   // token indices fit 31 bits (n_tokens is an int)
  uint32_t ok_mask = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 16 + (idx >> 4);
    const long long tk = row_token(a, it.bos_q, it.bos_k, r_base + min(r, nrows - 1));
    const bool ok = tk >= 0 && tk < a.n_tokens;
    ok_mask |= (uint32_t)ok << i;
    tok[i] = ok ? (uint32_t)tk : 0u;
  }
  uint4 vals[8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
    vals[i] = __ldg(reinterpret_cast<const uint4*>(a.q + ((size_t)tok[i] * a.hq + it.hq) * HEAD_DIM) + ch);
  if (ok_mask != 0xffu && a.status) atomicCAS(a.status, 0, (int)DEV_BAD_INDEX);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 16 + (idx >> 4);
    const bool keep = (r < nrows) && ((ok_mask >> i) & 1u);
    uint4 v = vals[i];
    if (!keep) v = make_uint4(0, 0, 0, 0);
    *reinterpret_cast<uint4*>(sQt + (ch >> 3) * BLK_BYTES + sw128_offset((uint32_t)r, (uint32_t)(ch & 7) * 8)) = v;
  }
  fence_proxy_async_smem();
}

// A [32 rows][16 columns] bf16 patch (8 packed words per lane, lane == row) goes through a warp-private
// 1 KB buffer and out with two lanes per row: one store instruction covers 16 rows x 32 contiguous
// bytes (whole sectors). 16-byte chunks are XOR-swizzled by (row / 4) so neither pass has bank conflicts.
//   my_row_off : element offset of (this lane's row, first column of the patch), or -1 to skip the row
__device__ __forceinline__ void store_patch_32x16(uint8_t* stage, const uint32_t* pk, __nv_bfloat16* base,
                                                  long long my_row_off, int lane) {
  uint8_t* wr = stage + lane * 32;
#pragma unroll
  for (int c = 0; c < 2; ++c)
    *reinterpret_cast<uint4*>(wr + (((c ^ (lane >> 2)) & 1) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
  __syncwarp();
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int r = 16 * k + (lane >> 1), c = lane & 1;
    const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 32 + (((c ^ (r >> 2)) & 1) << 4));
    const long long off = __shfl_sync(0xffffffffu, my_row_off, r);
    if (off >= 0) *reinterpret_cast<uint4*>(base + off + c * 8) = v;
  }
  __syncwarp();
}

__global__ void __launch_bounds__(FWD_THREADS, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                    const AttnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + 2 * TILE_BYTES;
  uint8_t* sV = sK + FWD_STAGES * TILE_BYTES;

  __shared__ uint64_t k_full[FWD_STAGES], k_empty[FWD_STAGES], v_full[FWD_STAGES], v_empty[FWD_STAGES];
  __shared__ uint64_t q_ready[2], s_full[2], p_ready[2], o_done[2];
  __shared__ __align__(16) uint8_t s_stage[FWD_SM_WARPS][1024];   // per-warp staging of the epilogue stores
  __shared__ float s_xch[2][FWD_SM_WARPS][32];   // row maxima / row sums handed to the row's other thread
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ int s_items[ITEM_RING * ITEM_WORDS];
  __shared__ uint64_t item_full[ITEM_RING], item_empty[ITEM_RING];
  const ItemRing ring{s_items, item_full, item_empty};

  const int tid = threadIdx.x;
  const int warp = uniform_warp_idx();
  const int lane = tid & 31;
  AbortState ab{&abort_flag, a.status};

  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < FWD_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&q_ready[t], FWD_SM_WARPS / 2);   // one arrival per warp
      mbar_init(&s_full[t], 1);
      mbar_init(&p_ready[t], FWD_SM_WARPS / 2);
      mbar_init(&o_done[t], 1);
    }
    ring_init(ring, FWD_SM_WARPS + 1);   // the softmax warps + the MMA warp
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  const int total_pairs = __ldg(a.n_tiles);
  const long long total_items = (long long)total_pairs * a.hq;

  if (warp < FWD_SM_WARPS) {
    // =====================================================================================
    // softmax groups
    // =====================================================================================
    const int t = warp >> 3;              // query tile of this group
    const int h = (warp >> 2) & 1;        // column half: keys / output columns [64 h, 64 h + 64)
    const int row = (warp & 3) * 32 + lane;   // row inside the tile == TMEM lane (a warp reaches lanes 32 * (warp % 4) ..)
    const int idx = tid & 255;            // thread index inside the tile's group
    const int pair_bar = 1 + (warp & 3) + 4 * t;   // named barrier of the two warps that share these rows
    const int partner = warp ^ 4;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + (uint32_t)t * 128u + lane_off + (uint32_t)h * 64u;   // this half's scores
    const uint32_t tP = tS;   // this half's probabilities (bf16, 32 columns) overwrite the start of its own scores
    const uint32_t tO = tmem + 256u + (uint32_t)t * 128u + lane_off + (uint32_t)h * 64u;
    uint8_t* sQt = sQ + t * TILE_BYTES;
    const float c = a.scale_log2;
    uint32_t n_steps = 0;   // (tile, key-step) pairs processed so far == S / P / O barrier phases
    uint32_t n_xch = 0;     // exchanges with the row's other thread so far (slot parity)

    // hands `mine` to the row's other thread and returns its value; every thread of both warps calls it
    auto exchange = [&](float mine) -> float {
      const uint32_t slot = n_xch++ & 1u;
      s_xch[slot][warp][lane] = mine;
      named_barrier_sync(pair_bar, 64);
      return s_xch[slot][partner][lane];
    };

    // Items are walked one ahead: as soon as the last score tile of an item has been read, the
    // rows of the NEXT item are copied into shared memory (Q is free by then), so the tensor pipe
    // computes its first scores while this group still writes the current item's output.
    uint32_t n_ring = 0;
    FwdItem it;
    long long w = ring_pop(ring, n_ring, it, ab);
    if (w >= 0) {
      if (it.nrows[t] > 0) {
        gather_query_tile(a, it, t, idx, sQt);
        tc_fence_before();
        mbar_arrive_warp(&q_ready[t]);
      }
    }
    while (w >= 0) {
      const int nrows = it.nrows[t];
      FwdItem it_next;
      long long w_next;
      if (nrows == 0) {
        w_next = ring_pop(ring, n_ring + 1, it_next, ab);
        if (w_next >= 0) {
          if (it_next.nrows[t] > 0) {
            gather_query_tile(a, it_next, t, idx, sQt);
            tc_fence_before();
            mbar_arrive_warp(&q_ready[t]);
          }
        }
        ring_release(ring, n_ring);
        it = it_next;
        w = w_next;
        ++n_ring;
        continue;
      }
      const int r_base = it.row0 + t * TILE;

      const int my_r = min(row, nrows - 1);
      const int my_pos = row_position(a, it.bos_q, r_base + my_r);
      const int min_pos = it.min_pos[t], max_pos = it.max_pos[t];
      float m_run = -INFINITY;
      float l_run = 0.f;   // this half's share of the row sum

      for (int j = it.jb[t]; j < it.je[t]; ++j) {
        const bool first = (j == it.jb[t]);
        const bool masked = (j * TILE + TILE - 1 > min_pos) || (a.window > 0 && j * TILE < max_pos - a.window);
        const int key_hi = my_pos;                                      // keys <= key_hi are visible
        const int key_lo = a.window > 0 ? my_pos - a.window : INT32_MIN;  // keys >= key_lo are visible

        mbar_wait(&s_full[t], n_steps & 1u, ab);
        tc_fence_after();

        // ---- this half of the score row (64 fp32): maximum first; the second 32 columns are read again
        //      for the exponentials instead of being held (96 registers per thread at this block size) ----
        uint32_t s0[32];
        float mx_half;
        {
          uint32_t s1[32];
          tmem_ld32(tS, s0);
          tmem_ld32(tS + 32, s1);
          tmem_ld_wait();
          if (masked) {
            mask_chunk(s0, j * TILE + h * 64, key_hi, key_lo);
            mask_chunk(s1, j * TILE + h * 64 + 32, key_hi, key_lo);
          }
          mx_half = fmaxf(max_chunk(s0), max_chunk(s1));
        }
        const float mx = fmaxf(mx_half, exchange(mx_half));   // row maximum over both halves

        // ---- running maximum, lazy rescale of O (both threads of a row take the same decision) ----
        if (first) {
          m_run = mx;
        } else {
          const float m_new = fmaxf(m_run, mx);
          const bool need = (m_new > m_run) && ((m_new - m_run) * c > RESCALE_THRESHOLD || m_run == -INFINITY);
          if (__any_sync(0xffffffffu, need)) {
            // the previous P*V of this tile must have landed before O is touched
            mbar_wait(&o_done[t], (n_steps - 1u) & 1u, ab);
            tc_fence_after();
            float alpha = 1.f;
            if (need) {
              alpha = (m_run == -INFINITY) ? 0.f : fast_exp2((m_run - m_new) * c);
              m_run = m_new;
              l_run *= alpha;
            }
#pragma unroll 1
            for (int chk = 0; chk < 2; ++chk) {
              uint32_t r[32];
              tmem_ld32(tO + chk * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st32(tO + chk * 32, r);
            }
            tmem_st_wait();
          }
        }

        // ---- probabilities -> bf16 in tensor memory (over S), row sum ----
        const float mc = (m_run == -INFINITY) ? 0.f : m_run * c;
        float l0 = 0.f, l1 = 0.f;
        {
          uint32_t pk[16];
          exp_pack_chunk(s0, c, mc, pk, l0, l1);
          tmem_ld32(tS + 32, s0);   // columns 32-63 again (the store below only touches columns 0-15)
          tmem_ld_wait();
          tmem_st16(tP, pk);
          if (masked) mask_chunk(s0, j * TILE + h * 64 + 32, key_hi, key_lo);
          exp_pack_chunk(s0, c, mc, pk, l0, l1);
          tmem_st16(tP + 16, pk);
        }
        l_run += l0 + l1;
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive_warp(&p_ready[t]);
        ++n_steps;
      }

      // ---- epilogue: O / l -> bf16 rows of the output, log-sum-exp ----
      const bool row_valid = row < nrows;
      const long long tok = row_valid ? row_token(a, it.bos_q, it.bos_k, r_base + row) : -1;
      const bool store = row_valid && tok >= 0 && tok < a.n_tokens;
      const float l_row = l_run + exchange(l_run);
      const float inv_l = 1.f / l_row;
      __nv_bfloat16* orow = a.o + ((size_t)(store ? tok : 0) * a.hq + it.hq) * HEAD_DIM + h * 64;
      float* lse_out = (store && a.lse && h == 0) ? a.lse + (size_t)tok * a.hq + it.hq : nullptr;

      w_next = ring_pop(ring, n_ring + 1, it_next, ab);
      if (w_next >= 0) {
        if (it_next.nrows[t] > 0) {
          gather_query_tile(a, it_next, t, idx, sQt);
          tc_fence_before();
          mbar_arrive_warp(&q_ready[t]);
        }
      }

      mbar_wait(&o_done[t], (n_steps - 1u) & 1u, ab);
      tc_fence_after();
      const long long row_off = store ? (long long)(orow - a.o) : -1;
#pragma unroll 1
      for (int chk = 0; chk < 2; ++chk) {
        uint32_t r[32], pk[16];
        tmem_ld32(tO + chk * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i)
          pk[i] = pack_bf16x2(__uint_as_float(r[2 * i]) * inv_l, __uint_as_float(r[2 * i + 1]) * inv_l);
        store_patch_32x16(s_stage[warp], pk, a.o, row_off >= 0 ? row_off + chk * 32 : -1, lane);
        store_patch_32x16(s_stage[warp], pk + 8, a.o, row_off >= 0 ? row_off + chk * 32 + 16 : -1, lane);
      }
      if (lse_out) *lse_out = m_run * c + log2f(l_row);
      tc_fence_before();
      ring_release(ring, n_ring);
      it = it_next;
      w = w_next;
      ++n_ring;
    }
  } else if (warp == FWD_SM_WARPS) {
    // =====================================================================================
    // TMA producer
    // =====================================================================================
    if (lane == 0) {
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      uint32_t kv_iter = 0, n_pub = 0;
      FwdItem it, it_ahead;
      long long w_last = -1;
      // claim + decode + publish one record; false once the list is exhausted (end marker published)
      auto next_item = [&](FwdItem& dst) -> bool {
        const long long w = ring_claim(a.work_counter, total_items, ab);
        if (w >= 0) fwd_decode_item(a, (int)w, total_pairs, dst);
        ring_publish(ring, n_pub++, w, dst, ab);
        w_last = w;
        return w >= 0;
      };
      bool have = next_item(it);
      while (have) {
        // Look one item ahead (decode and publish it before this item's loads) while the list is long;
        // near its end claim late, so that no CTA sits on an item another CTA could already run.
        const bool ahead = (total_items - w_last) > 6ll * gridDim.x;
        bool have_ahead = ahead ? next_item(it_ahead) : false;
        const int x = it.kvh * HEAD_DIM;
        for (int j = it.JB; j < it.JE; ++j, ++kv_iter) {
          const uint32_t st = kv_iter % FWD_STAGES;
          const uint32_t ph = (kv_iter / FWD_STAGES) & 1u;
          const int y = it.bos_k + j * TILE;
          mbar_wait(&k_empty[st], ph ^ 1u, ab);
          mbar_arrive_expect_tx(&k_full[st], TILE_BYTES);
          tma_load_2d(sK + st * TILE_BYTES, &tm_k, &k_full[st], x, y);
          tma_load_2d(sK + st * TILE_BYTES + BLK_BYTES, &tm_k, &k_full[st], x + 64, y);
          mbar_wait(&v_empty[st], ph ^ 1u, ab);
          mbar_arrive_expect_tx(&v_full[st], TILE_BYTES);
          tma_load_2d(sV + st * TILE_BYTES, &tm_v, &v_full[st], x, y);
          tma_load_2d(sV + st * TILE_BYTES + BLK_BYTES, &tm_v, &v_full[st], x + 64, y);
        }
        if (!ahead) have_ahead = next_item(it_ahead);
        it = it_ahead;
        have = have_ahead;
      }
      // On an aborted run copies may still be in flight: give them a bounded time to land
      // before the CTA's shared memory is released.
      if (abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp > FWD_SM_WARPS + 1) {
    // =====================================================================================
    // spare warps: the output rows of unselected tokens are zero (HBM traffic that hides under the products)
    // =====================================================================================
    if (a.zero_sq && a.q_idx) {
      const int sq = min(max(__ldg(a.zero_sq), 0), a.n_tokens);
      zero_unselected_rows_part(reinterpret_cast<uint4*>(a.o), a.q_idx, sq, a.n_tokens, a.hq * HEAD_DIM / 8,
                                blockIdx.x * 2 + (warp - (FWD_SM_WARPS + 2)), gridDim.x * 2, lane);
    }
  } else {
    // =====================================================================================
    // MMA issuer: the whole warp walks this code, an elected lane issues (see umma_ss)
    // =====================================================================================
    {
      const uint32_t idesc_qk = umma_idesc_bf16(TILE, TILE, 0, 0);
      const uint32_t idesc_pv = umma_idesc_bf16(TILE, HEAD_DIM, 0, 1);
      const uint32_t q_base = smem_u32(sQ), k_base = smem_u32(sK), v_base = smem_u32(sV);
      uint32_t kv_iter = 0;
      uint32_t n_p[2] = {0, 0};      // P barriers consumed per tile
      uint32_t n_items[2] = {0, 0};  // items per tile

      auto issue_s = [&](int t, uint32_t st) {
        umma_tile_k128<false, false>(tmem + (uint32_t)t * 128u, umma_desc_sw128(q_base + (uint32_t)t * TILE_BYTES, 0, 1024),
                                     umma_desc_sw128(k_base + st * TILE_BYTES, 0, 1024), idesc_qk, 0u);
        umma_commit(&s_full[t]);
      };
      auto issue_pv = [&](int t, uint32_t st, bool acc) {
        umma_tile_k128<true, true, 2>(tmem + 256u + (uint32_t)t * 128u, tmem + (uint32_t)t * 128u,
                                   umma_desc_sw128(v_base + st * TILE_BYTES, BLK_BYTES, 1024), idesc_pv, acc ? 1u : 0u);
        umma_commit(&o_done[t]);
      };

      for (uint32_t n_ring = 0;; ++n_ring) {
        FwdItem it;
        const long long w = ring_pop(ring, n_ring, it, ab);
        if (w < 0) break;
        if (it.JE <= it.JB) {
          ring_release(ring, n_ring);
          continue;
        }
        for (int t = 0; t < 2; ++t) {
          if (it.nrows[t] > 0) {
            mbar_wait(&q_ready[t], n_items[t] & 1u, ab);
            ++n_items[t];
          }
        }
        tc_fence_after();
        bool started[2] = {false, false};

        // scores of the first key tile
        {
          const uint32_t st = kv_iter % FWD_STAGES, ph = (kv_iter / FWD_STAGES) & 1u;
          mbar_wait(&k_full[st], ph, ab);
          tc_fence_after();
          for (int t = 0; t < 2; ++t)
            if (tile_active(it, t, it.JB)) issue_s(t, st);
          umma_commit(&k_empty[st]);
        }
        for (int j = it.JB; j < it.JE; ++j, ++kv_iter) {
          const uint32_t st = kv_iter % FWD_STAGES, ph = (kv_iter / FWD_STAGES) & 1u;
          const uint32_t st_n = (kv_iter + 1) % FWD_STAGES, ph_n = ((kv_iter + 1) / FWD_STAGES) & 1u;
          const bool has_next = (j + 1 < it.JE);
          mbar_wait(&v_full[st], ph, ab);
          for (int t = 0; t < 2; ++t) {
            if (tile_active(it, t, j)) {
              mbar_wait(&p_ready[t], n_p[t] & 1u, ab);
              ++n_p[t];
              tc_fence_after();
              issue_pv(t, st, started[t]);
              started[t] = true;
            }
            if (t == 1) umma_commit(&v_empty[st]);
            if (has_next) {
              if (t == 0) {
                mbar_wait(&k_full[st_n], ph_n, ab);
                tc_fence_after();
              }
              if (tile_active(it, t, j + 1)) issue_s(t, st_n);
              if (t == 1) umma_commit(&k_empty[st_n]);
            }
          }
        }
        ring_release(ring, n_ring);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

static int launch_attn_fwd(const AttnArgs& a, cudaStream_t stream) {
  CUtensorMap tm_k, tm_v;
  const uint64_t row_bytes = (uint64_t)a.h * HEAD_DIM * sizeof(__nv_bfloat16);
  int rc = make_tmap_2d_bf16(&tm_k, a.k, (uint64_t)a.h * HEAD_DIM, (uint64_t)a.n_tokens, row_bytes, 64, TILE);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tm_v, a.v, (uint64_t)a.h * HEAD_DIM, (uint64_t)a.n_tokens, row_bytes, 64, TILE);
  if (rc) return rc;
  static thread_local int attr_set_dev = -1;
  int dev = 0;
  LOGO_CHECK_CUDA(cudaGetDevice(&dev));
  if (attr_set_dev != dev) {
    LOGO_CHECK_CUDA(cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM_BYTES));
    attr_set_dev = dev;
  }
  const int grid = sm_count();
  LOGO_CHECK_CUDA(cudaMemsetAsync(a.work_counter, 0, sizeof(int), stream));
  prof_begin(PROF_ATTN_FWD, stream);
  attn_fwd_kernel<<<grid, FWD_THREADS, FWD_SMEM_BYTES, stream>>>(tm_k, tm_v, a);
  prof_end(PROF_ATTN_FWD, stream);
  LOGO_CHECK_CUDA(cudaGetLastError());
  return LOGO_OK;
}

static int check_attn_common(const void* q, const void* k, const void* v, const void* o, int n_tokens, int n_seq,
                             int hq, int h, int d) {
  LOGO_REQUIRE(d == HEAD_DIM, LOGO_ERR_UNSUPPORTED, "head_dim %d is not supported (only 128)", d);
  LOGO_REQUIRE(hq > 0 && h > 0 && hq % h == 0, LOGO_ERR_INVALID, "hq (%d) must be a positive multiple of h (%d)", hq, h);
  LOGO_REQUIRE(n_tokens >= 0 && n_seq >= 0, LOGO_ERR_INVALID, "n_tokens and n_seq must be non-negative");
  LOGO_REQUIRE(n_tokens == 0 || (q && k && v && o), LOGO_ERR_INVALID, "q, k, v and the output must not be NULL");
  LOGO_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o), LOGO_ERR_INVALID,
               "q, k, v and the output must be 16-byte aligned");
  return LOGO_OK;
}

}  // namespace logo

extern "C" int logo_sq_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int64_t* q_idx,
                                const int32_t* pos_ids, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                const int32_t* tile_off, int32_t* meta, int n_seq, int n_tokens, int hq, int h,
                                int d, float scale, int zero_fill, int32_t* status, logo_stream_t stream_) {
  using namespace logo;
  cudaStream_t stream = (cudaStream_t)stream_;
  int rc = check_attn_common(q, k, v, o, n_tokens, n_seq, hq, h, d);
  if (rc) return rc;
  if (n_tokens == 0 || n_seq == 0) return LOGO_OK;
  LOGO_REQUIRE(q_idx && pos_ids && cu_seqlens_q && cu_seqlens_k && tile_off && meta, LOGO_ERR_INVALID,
               "selection metadata pointers must not be NULL");
  AttnArgs a{};
  a.q = (const __nv_bfloat16*)q;
  a.k = (const __nv_bfloat16*)k;
  a.v = (const __nv_bfloat16*)v;
  a.o = (__nv_bfloat16*)o;
  a.lse = lse;
  a.q_idx = q_idx;
  a.pos_ids = pos_ids;
  a.cu_q = cu_seqlens_q;
  a.cu_k = cu_seqlens_k;
  a.tile_off = tile_off;  // row 0: selected-row pairs
  a.n_tiles = meta + 1;
  a.work_counter = meta + LOGO_META_COUNTER_SQ_FWD;
  a.n_seq = n_seq;
  a.n_tokens = n_tokens;
  a.hq = hq;
  a.h = h;
  a.window = 0;
  a.zero_sq = zero_fill ? meta : nullptr;   // meta[0] = number of selected rows
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  return launch_attn_fwd(a, stream);
}

extern "C" int logo_swa_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                            const int32_t* cu_seqlens, const int32_t* tile_off, int32_t* meta, int n_seq,
                            int n_tokens, int hq, int h, int d, int window, float scale, int32_t* status,
                            logo_stream_t stream_) {
  using namespace logo;
  cudaStream_t stream = (cudaStream_t)stream_;
  int rc = check_attn_common(q, k, v, o, n_tokens, n_seq, hq, h, d);
  if (rc) return rc;
  LOGO_REQUIRE(window > 0, LOGO_ERR_INVALID, "window must be positive, got %d", window);
  if (n_tokens == 0 || n_seq == 0) return LOGO_OK;
  LOGO_REQUIRE(cu_seqlens && tile_off && meta, LOGO_ERR_INVALID, "cu_seqlens, tile_off and meta must not be NULL");
  AttnArgs a{};
  a.q = (const __nv_bfloat16*)q;
  a.k = (const __nv_bfloat16*)k;
  a.v = (const __nv_bfloat16*)v;
  a.o = (__nv_bfloat16*)o;
  a.lse = lse;
  a.q_idx = nullptr;
  a.pos_ids = nullptr;
  a.cu_q = cu_seqlens;
  a.cu_k = cu_seqlens;
  a.tile_off = tile_off + 2 * (n_seq + 1);  // row 2: all-row pairs
  a.n_tiles = meta + 3;
  a.work_counter = meta + LOGO_META_COUNTER_SWA_FWD;
  a.n_seq = n_seq;
  a.n_tokens = n_tokens;
  a.hq = hq;
  a.h = h;
  a.window = window;
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  return launch_attn_fwd(a, stream);
}
