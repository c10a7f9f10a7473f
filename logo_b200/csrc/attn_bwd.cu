// Backward attention for both LoGo branches on tcgen05 tensor cores.
//
// Three kernels:
//   1. bwd_preprocess_kernel: delta = sum_d o * dO per (row, head); for the query-sparse
//      branch it also packs the selected rows of Q and dO into contiguous buffers so the
//      two GEMM kernels can stream them with TMA, and transposes lse to head-major.
//   2. attn_bwd_dq_kernel: work item = (128-row query tile, head); streams K/V tiles.
//        S = Q K^T, dP = dO V^T, dS = P o (dP - delta), dQ += dS K
//   3. attn_bwd_dkv_kernel: work item = (128-key tile, kv head); streams Q/dO tiles of every
//      query head of the group (the GQA reduction happens in the accumulators).
//        S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q
// Both GEMM kernels are persistent (one CTA per SM claims items from a global counter through
// the record ring of attn_common.cuh). The element-wise warps split a 128x128 tile by TMEM lane
// quarter (w % 4) and column range: eight warps x 64 columns in the dK/dV kernel, sixteen warps
// x 32 columns in the dQ kernel; one further warp is the TMA producer and one issues the MMAs.
// P / dS are written back to tensor memory as bf16 INSIDE the columns their warp read (so no
// warp touches another warp's columns) and consumed as the A operand of the next product; the
// tile that supplies the B operand of that product ([rows][128] as it lies in memory) is read
// through an MN-major descriptor.
//
// Algorithmic work: 2.5x the forward FLOPs (5 products against 2); S is recomputed in both
// GEMM kernels, so 7 products execute.
#include "attn_bwd_common.cuh"

#include <atomic>

namespace logo {

// ---------------------------------------------------------------------------------------
// 1. preprocess
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
    bwd_preprocess_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ o,
                          const __nv_bfloat16* __restrict__ d_o, const float* __restrict__ lse,
                          const int64_t* __restrict__ q_idx, const int32_t* __restrict__ sq_ptr,
                          __nv_bfloat16* __restrict__ q_sel, __nv_bfloat16* __restrict__ do_sel,
                          float* __restrict__ lse_sel, float* __restrict__ delta_sel, float* __restrict__ dq_acc,
                          __nv_bfloat16* __restrict__ vec_split, float inv_scale_log2, int cap, int n_tokens, int hq,
                          int* status) {
  const bool gathered = (q_idx != nullptr);
  const int sq = gathered ? min(max(__ldg(sq_ptr), 0), n_tokens) : n_tokens;
  const int rows_total = gathered ? min(sq + TILE, cap) : sq;
  const int lane = threadIdx.x & 31;
  const int sub = lane >> 4;            // which of the two heads a warp handles at a time
  const int col = (lane & 15) * 8;      // 16 lanes x 16 bytes cover one 128-element row
  const int warps_per_block = blockDim.x >> 5;
  constexpr int U = 4;                  // head pairs in flight: all their loads are issued before the first reduction
  for (int r = blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < rows_total; r += gridDim.x * warps_per_block) {
    if (r < sq) {
      long long tok = gathered ? __ldg(q_idx + r) : (long long)r;
      if (tok < 0 || tok >= n_tokens) {
        if (lane == 0 && status) atomicCAS(status, 0, (int)DEV_BAD_INDEX);
        tok = 0;
      }
      for (int hb = 0; hb < hq; hb += 2 * U) {
        uint4 ov[U], dv[U], qv[U];
        float lv[U];
        bool act[U];
        int hh[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          hh[u] = hb + 2 * u + sub;
          act[u] = hh[u] < hq;
          const size_t src = ((size_t)tok * hq + (act[u] ? hh[u] : 0)) * HEAD_DIM + col;
          ov[u] = __ldg(reinterpret_cast<const uint4*>(o + src));
          dv[u] = __ldg(reinterpret_cast<const uint4*>(d_o + src));
          if (gathered) qv[u] = __ldg(reinterpret_cast<const uint4*>(q + src));
          lv[u] = __ldg(lse + (size_t)tok * hq + (act[u] ? hh[u] : 0));
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&ov[u]);
          const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dv[u]);
          float acc = 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 of = __bfloat1622float2(o2[i]);
            const float2 df = __bfloat1622float2(d2[i]);
            acc = fmaf(of.x, df.x, acc);
            acc = fmaf(of.y, df.y, acc);
          }
#pragma unroll
          for (int off = 8; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
          if (act[u]) {
            if ((lane & 15) == 0) {
              delta_sel[(size_t)hh[u] * cap + r] = acc;
              lse_sel[(size_t)hh[u] * cap + r] = lv[u];
              if (vec_split) {
                // -lse / c and -delta as three bf16 terms each (24 bits): the single-pass kernel adds them to
                // its score and dP tiles with a tensor-core k-step
                const float x = -lv[u] * inv_scale_log2, y = -acc;
                const __nv_bfloat16 x0 = __float2bfloat16_rn(x);
                const __nv_bfloat16 x1 = __float2bfloat16_rn(x - __bfloat162float(x0));
                const __nv_bfloat16 x2 = __float2bfloat16_rn(x - __bfloat162float(x0) - __bfloat162float(x1));
                const __nv_bfloat16 y0 = __float2bfloat16_rn(y);
                const __nv_bfloat16 y1 = __float2bfloat16_rn(y - __bfloat162float(y0));
                const __nv_bfloat16 y2 = __float2bfloat16_rn(y - __bfloat162float(y0) - __bfloat162float(y1));
                auto pair = [](__nv_bfloat16 lo, __nv_bfloat16 hi) {
                  return (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
                };
                uint4* dst = reinterpret_cast<uint4*>(vec_split + ((size_t)r * hq + hh[u]) * 16);
                dst[0] = make_uint4(pair(x0, x1), pair(x2, y0), pair(y1, y2), 0u);
                dst[1] = make_uint4(0u, 0u, 0u, 0u);
              }
            }
            if (gathered) {
              const size_t dst = ((size_t)r * hq + hh[u]) * HEAD_DIM + col;
              *reinterpret_cast<uint4*>(q_sel + dst) = qv[u];
              *reinterpret_cast<uint4*>(do_sel + dst) = dv[u];
            }
            if (dq_acc) {   // the single-pass backward adds into this row: it must start at zero
              float4* z = reinterpret_cast<float4*>(dq_acc + ((size_t)r * hq + hh[u]) * HEAD_DIM + col);
              z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
              z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
          }
        }
      }
    } else {
      // padding rows behind the last selected row: tiles may read them, keep them finite
      for (int hb = 0; hb < hq; hb += 2) {
        const int h1 = hb + sub;
        if (h1 < hq) {
          const size_t dst = ((size_t)r * hq + h1) * HEAD_DIM + col;
          *reinterpret_cast<uint4*>(q_sel + dst) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(do_sel + dst) = make_uint4(0, 0, 0, 0);
          if ((lane & 15) == 0) {
            delta_sel[(size_t)h1 * cap + r] = 0.f;
            lse_sel[(size_t)h1 * cap + r] = 0.f;
            if (vec_split) {
              uint4* dst = reinterpret_cast<uint4*>(vec_split + ((size_t)r * hq + h1) * 16);
              dst[0] = make_uint4(0u, 0u, 0u, 0u);
              dst[1] = make_uint4(0u, 0u, 0u, 0u);
            }
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// 2. dQ
// ---------------------------------------------------------------------------------------
struct DqItem {
  int hq, kvh, bos_q, bos_k, r_base, nrows, min_pos, max_pos, jb, je;
};

__device__ __forceinline__ void dq_decode_item(const BwdArgs& a, int w, int total_tiles, DqItem& it) {
  const int tile_g = total_tiles - 1 - w / a.hq;
  it.hq = w % a.hq;
  it.kvh = it.hq / (a.hq / a.h);
  const int seq = find_sequence(a.tile_off_q, a.n_seq, tile_g);
  const int tile_l = tile_g - __ldg(a.tile_off_q + seq);
  it.bos_q = __ldg(a.cu_q + seq);
  const int nsel = __ldg(a.cu_q + seq + 1) - it.bos_q;
  it.bos_k = __ldg(a.cu_k + seq);
  const int len_k = __ldg(a.cu_k + seq + 1) - it.bos_k;
  it.r_base = tile_l * TILE;
  it.nrows = min(max(nsel - it.r_base, 0), TILE);
  it.min_pos = it.max_pos = 0;
  it.jb = it.je = 0;
  if (it.nrows > 0) {
    int lo = bwd_row_position(a, it.bos_q, it.r_base);
    int hi = bwd_row_position(a, it.bos_q, it.r_base + it.nrows - 1);
    if (lo < 0 || hi >= len_k || lo > hi) {
      if (a.status) atomicCAS(a.status, 0, (int)DEV_BAD_INDEX);
      lo = max(min(lo, len_k - 1), 0);
      hi = max(min(hi, len_k - 1), lo);
    }
    it.min_pos = lo;
    it.max_pos = hi;
    it.je = hi / TILE + 1;
    it.jb = a.window > 0 ? max(lo - a.window, 0) / TILE : 0;
  }
}

__global__ void __launch_bounds__(DQ_THREADS, 1)
    attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                       const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                       const BwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + TILE_BYTES;
  uint8_t* sK = smem + 2 * TILE_BYTES;   // 2 stages
  uint8_t* sV = smem + 4 * TILE_BYTES;   // 2 stages

  __shared__ uint64_t qdo_full, qdo_free, k_full[2], k_empty[2], v_full[2], v_empty[2];
  __shared__ uint64_t s_full[2], dp_full, ds_ready, acc_done;
  __shared__ __align__(16) uint8_t s_stage[8][2048];   // per-warp staging of the epilogue stores
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ int s_items[ITEM_RING * ITEM_WORDS];
  __shared__ uint64_t item_full[ITEM_RING], item_empty[ITEM_RING];
  const ItemRing ring{s_items, item_full, item_empty};

  const int tid = threadIdx.x, warp = uniform_warp_idx(), lane = tid & 31;
  AbortState ab{&abort_flag, a.status};

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&qdo_full, 1);
    mbar_init(&qdo_free, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
    }
    mbar_init(&dp_full, 1);
    mbar_init(&ds_ready, DQ_EW_WARPS);   // one arrival per warp
    mbar_init(&acc_done, 1);
    ring_init(ring, DQ_EW_WARPS + 1);
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
  const uint32_t TM_S = tmem, TM_DP = tmem + 256u, TM_DQ = tmem + 384u;

  const int total_tiles = __ldg(a.n_qtiles);
  const long long total_items = (long long)total_tiles * a.hq;

  if (warp < DQ_EW_WARPS) {
    // Sixteen element-wise warps: warp w works on the 32 rows of lane quarter w % 4 and the 32 key
    // columns [32 * (w / 4), +32). Four warps per scheduler keep its pipes fed while one of them waits
    // on tensor memory or a barrier; with eight warps (64 columns each) the instruction stream of a
    // warp was the bottleneck.
    const int quad = warp & 3, part = warp >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const int col0 = part * 32;
    const float c = a.scale_log2;
    uint32_t idx = 0;      // key steps processed so far (all items)
    uint32_t n_items = 0;

    for (uint32_t n_ring = 0;; ++n_ring) {
      DqItem it;
      const long long w = ring_pop(ring, n_ring, it, ab);
      if (w < 0) break;
      if (it.nrows == 0) {
        ring_release(ring, n_ring);
        continue;
      }
      const int rowv = min(row, it.nrows - 1);
      const int my_pos = bwd_row_position(a, it.bos_q, it.r_base + rowv);
      const size_t sidx = (size_t)it.hq * a.cap + it.bos_q + it.r_base + rowv;
      const float lse_r = __ldg(a.lse_sel + sidx);
      const float delta_r = __ldg(a.delta_sel + sidx);
      const int key_hi = my_pos;
      const int key_lo = a.window > 0 ? my_pos - a.window : INT32_MIN;

      for (int j = it.jb; j < it.je; ++j, ++idx) {
        const bool masked =
            (j * TILE + TILE - 1 > it.min_pos) || (a.window > 0 && j * TILE < it.max_pos - a.window);
        const uint32_t tS = TM_S + (idx & 1u) * 128u + lane_off + (uint32_t)col0;
        uint32_t p0[32];
        mbar_wait(&s_full[idx & 1u], (idx >> 1) & 1u, ab);
        tc_fence_after();
        tmem_ld32(tS, p0);
        tmem_ld_wait();
        prob_chunk_row(p0, c, lse_r, masked, j * TILE + col0, key_hi, key_lo);
        mbar_wait(&dp_full, idx & 1u, ab);
        tc_fence_after();
        uint32_t pk[16];
        {
          uint32_t d0[32];
          tmem_ld32(TM_DP + lane_off + (uint32_t)col0, d0);
          tmem_ld_wait();
          ds_pack_chunk_row(p0, d0, delta_r, pk);
        }
        // dS (bf16) goes into the first 16 of the 32 dP columns this warp has just read: no other warp
        // reads or writes them, so no barrier is needed before the overwrite
        tmem_st16(TM_DP + lane_off + (uint32_t)col0, pk);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive_warp(&ds_ready);
      }

      // ---- epilogue: dQ * scale -> bf16 rows ----
      mbar_wait(&acc_done, n_items & 1u, ab);
      tc_fence_after();
      ++n_items;
      long long tok = -1;
      if (row < it.nrows)
        tok = a.q_idx ? __ldg(a.q_idx + it.bos_q + it.r_base + row) : (long long)(it.bos_k + it.r_base + row);
      const bool store = tok >= 0 && tok < a.n_tokens;
      const long long row_off = store ? (long long)(((size_t)tok * a.hq + it.hq) * HEAD_DIM + col0) : -1;
      {
        uint32_t r[32], pk[16];
        tmem_ld32(TM_DQ + lane_off + (uint32_t)col0, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i)
          pk[i] = pack_bf16x2(__uint_as_float(r[2 * i]) * a.scale, __uint_as_float(r[2 * i + 1]) * a.scale);
        // eight staging buffers for sixteen warps: two rounds
        if (part < 2) store_patch_32x32(s_stage[warp], pk, a.dq, row_off, lane);
        named_barrier_sync(1, DQ_EW_WARPS * 32);
        if (part >= 2) store_patch_32x32(s_stage[warp - 8], pk, a.dq, row_off, lane);
      }
      tc_fence_before();
      ring_release(ring, n_ring);
    }
  } else if (warp == DQ_EW_WARPS) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_do);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      uint32_t kv_iter = 0, n_items = 0, n_pub = 0;
      DqItem it, it_ahead;
      long long w_last = -1;
      auto next_item = [&](DqItem& dst) -> bool {
        const long long w = ring_claim(a.counter_dq, total_items, ab);
        if (w >= 0) dq_decode_item(a, (int)w, total_tiles, dst);
        ring_publish(ring, n_pub++, w, dst, ab);
        w_last = w;
        return w >= 0;
      };
      bool have = next_item(it);
      while (have) {
        if (it.nrows > 0) {
          const int xq = it.hq * HEAD_DIM, yq = it.bos_q + it.r_base;
          mbar_wait(&qdo_free, (n_items & 1u) ^ 1u, ab);
          mbar_arrive_expect_tx(&qdo_full, 2 * TILE_BYTES);
          tma_load_2d(sQ, &tm_q, &qdo_full, xq, yq);
          tma_load_2d(sQ + BLK_BYTES, &tm_q, &qdo_full, xq + 64, yq);
          tma_load_2d(sDO, &tm_do, &qdo_full, xq, yq);
          tma_load_2d(sDO + BLK_BYTES, &tm_do, &qdo_full, xq + 64, yq);
          ++n_items;
        }
        // Look one item ahead (decode and publish it before this item's K/V stream) while the list is long;
        // near its end claim late, so that no CTA sits on an item another CTA could already run.
        const bool ahead = (total_items - w_last) > 6ll * gridDim.x;
        bool have_ahead = ahead ? next_item(it_ahead) : false;
        const int x = it.kvh * HEAD_DIM;
        for (int j = it.jb; it.nrows > 0 && j < it.je; ++j, ++kv_iter) {
          const uint32_t st = kv_iter & 1u, ph = (kv_iter >> 1) & 1u;
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
      if (abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else {
    {   // MMA issuer: the whole warp walks this code, an elected lane issues (see umma_ss)
      const uint32_t idesc_kk = umma_idesc_bf16(TILE, TILE, 0, 0);       // both operands K-major
      const uint32_t idesc_mn = umma_idesc_bf16(TILE, HEAD_DIM, 0, 1);   // B operand MN-major
      const uint32_t q_base = smem_u32(sQ), do_base = smem_u32(sDO), k_base = smem_u32(sK), v_base = smem_u32(sV);
      uint32_t kv_iter = 0, n_items = 0;

      auto issue_kk = [&](uint32_t d_tmem, uint32_t a_base, uint32_t b_base) {
        umma_tile_k128<false, false>(d_tmem, umma_desc_sw128(a_base, 0, 1024), umma_desc_sw128(b_base, 0, 1024),
                                     idesc_kk, 0u);
      };
      auto issue_ts = [&](uint32_t d_tmem, uint32_t a_tmem, uint32_t b_base, bool acc) {
        umma_tile_k128<true, true, 4>(d_tmem, a_tmem, umma_desc_sw128(b_base, BLK_BYTES, 1024), idesc_mn,
                                      acc ? 1u : 0u);
      };

      for (uint32_t n_ring = 0;; ++n_ring) {
        DqItem it;
        const long long w = ring_pop(ring, n_ring, it, ab);
        if (w < 0) break;
        if (it.nrows == 0) {
          ring_release(ring, n_ring);
          continue;
        }
        mbar_wait(&qdo_full, n_items & 1u, ab);
        ++n_items;
        tc_fence_after();
        // Issue order. dQ(j) and dP(j+1) go out the moment dS(j) is ready (they are the dependency
        // chain of the element-wise warps); the scores run two key tiles ahead into the S buffer the
        // warps finished reading a step earlier, so a K tile that is still in flight delays nothing.
        const int n_kt = it.je - it.jb;
        {
          const uint32_t st = kv_iter & 1u, ph = (kv_iter >> 1) & 1u;
          mbar_wait(&k_full[st], ph, ab);
          tc_fence_after();
          issue_kk(TM_S + st * 128u, q_base, k_base + st * TILE_BYTES);
          umma_commit(&s_full[st]);
          mbar_wait(&v_full[st], ph, ab);
          tc_fence_after();
          issue_kk(TM_DP, do_base, v_base + st * TILE_BYTES);
          umma_commit(&dp_full);
          umma_commit(&v_empty[st]);
          if (n_kt > 1) {
            const uint32_t nx = kv_iter + 1u, st_n = nx & 1u, ph_n = (nx >> 1) & 1u;
            mbar_wait(&k_full[st_n], ph_n, ab);
            tc_fence_after();
            issue_kk(TM_S + st_n * 128u, q_base, k_base + st_n * TILE_BYTES);
            umma_commit(&s_full[st_n]);
          }
        }
        for (int j = it.jb; j < it.je; ++j, ++kv_iter) {
          const uint32_t st = kv_iter & 1u;
          const uint32_t nx = kv_iter + 1u, st_n = nx & 1u, ph_n = (nx >> 1) & 1u;
          const uint32_t nx2 = kv_iter + 2u, ph_n2 = (nx2 >> 1) & 1u;   // same stage / S buffer as step j
          const bool has_next = (j + 1 < it.je), has_next2 = (j + 2 < it.je);
          mbar_wait(&ds_ready, kv_iter & 1u, ab);
          tc_fence_after();
          issue_ts(TM_DQ, TM_DP, k_base + st * TILE_BYTES, j > it.jb);
          umma_commit(&k_empty[st]);
          if (has_next) {
            mbar_wait(&v_full[st_n], ph_n, ab);
            tc_fence_after();
            issue_kk(TM_DP, do_base, v_base + st_n * TILE_BYTES);
            umma_commit(&dp_full);
            umma_commit(&v_empty[st_n]);
          }
          if (has_next2) {
            mbar_wait(&k_full[st], ph_n2, ab);
            tc_fence_after();
            issue_kk(TM_S + st * 128u, q_base, k_base + st * TILE_BYTES);
            umma_commit(&s_full[st]);
          }
          // every product that reads Q / dO has been issued: the next item's tiles may come in
          // while the remaining dQ products and the epilogue run
          if (has_next ? !has_next2 : n_kt == 1) umma_commit(&qdo_free);
        }
        umma_commit(&acc_done);
        ring_release(ring, n_ring);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------------------
// 3. dK / dV
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(BWD_THREADS, 1)
    attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                        const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                        const BwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE_BYTES;
  uint8_t* sQ = smem + 2 * TILE_BYTES;    // 2 stages
  uint8_t* sDO = smem + 4 * TILE_BYTES;   // 2 stages

  __shared__ uint64_t kv_full, kv_free, q_full[2], q_empty[2], do_full[2], do_empty[2];
  __shared__ uint64_t st_full, dpt_full, p_ready, ds_ready, acc_done;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ __align__(16) float s_lse[2][TILE];
  __shared__ __align__(16) float s_delta[2][TILE];
  __shared__ __align__(16) int s_pos[2][TILE];
  __shared__ __align__(16) uint8_t s_stage[8][2048];   // per-warp staging of the epilogue stores
  __shared__ int s_items[ITEM_RING * ITEM_WORDS];
  __shared__ uint64_t item_full[ITEM_RING], item_empty[ITEM_RING];
  const ItemRing ring{s_items, item_full, item_empty};

  const int tid = threadIdx.x, warp = uniform_warp_idx(), lane = tid & 31;
  AbortState ab{&abort_flag, a.status};

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&kv_full, 1);
    mbar_init(&kv_free, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
      mbar_init(&do_full[s], 1);
      mbar_init(&do_empty[s], 1);
    }
    mbar_init(&st_full, 1);
    mbar_init(&dpt_full, 1);
    mbar_init(&p_ready, 8);    // one arrival per warp
    mbar_init(&ds_ready, 8);
    mbar_init(&acc_done, 1);
    ring_init(ring, 9);
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
  const uint32_t TM_ST = tmem, TM_DPT = tmem + 128u, TM_DK = tmem + 256u, TM_DV = tmem + 384u;

  const int total_tiles = __ldg(a.n_ktiles);
  const long long total_items = (long long)total_tiles * a.h;
  const int G = a.hq / a.h;

  if (warp < 8) {
    const int quad = warp & 3, half = warp >> 2;
    const int row = quad * 32 + lane;   // key inside the tile
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const int col0 = half * 64;
    const float c = a.scale_log2;
    uint32_t idx = 0, n_items = 0;

    // Loads lse / delta / pos of query tile `i` of head `hq` into registers. The loads are issued
    // unconditionally from a clamped row (no select on a loaded value before it is needed, which
    // would expose the memory round trip); rows past the end are replaced when the values are used.
    const int vrow = tid & (TILE - 1);
    auto fetch_vec = [&](const DkvItem& it, int hq, int i, float& l, float& d, int& p) -> bool {
      const int r = i * TILE + vrow;
      const int rc = min(r, it.nsel - 1);
      const size_t sidx = (size_t)hq * a.cap + it.bos_q + rc;
      l = __ldg(a.lse_sel + sidx);
      d = __ldg(a.delta_sel + sidx);
      p = bwd_row_position(a, it.bos_q, rc);
      return r < it.nsel;
    };

    // Items are walked one ahead: during the last step of an item the next record is popped and its
    // first-step vectors start travelling to shared memory, so the next item begins without a
    // memory round trip.
    uint32_t n_ring = 0;
    DkvItem it;
    long long w = ring_pop(ring, n_ring, it, ab);
    bool vec_ready = false;   // the first-step vectors of `it` are already in s_*[idx & 1]
    while (w >= 0) {
      DkvItem it_next;
      long long w_next = -1;
      bool vec_next = false;
      const int nq = it.i_end - it.i0;
      const int key_pos = it.kv_start + row;
      const bool key_valid = key_pos < it.len_k;
      __nv_bfloat16* dk_row = a.dk + ((size_t)(it.bos_k + (key_valid ? key_pos : 0)) * a.h + it.kvh) * HEAD_DIM + col0;
      __nv_bfloat16* dv_row = a.dv + ((size_t)(it.bos_k + (key_valid ? key_pos : 0)) * a.h + it.kvh) * HEAD_DIM + col0;
      if (nq <= 0) {
        // no query can see this key tile: the gradients are zero
        if (key_valid) {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            reinterpret_cast<uint4*>(dk_row)[g] = make_uint4(0, 0, 0, 0);
            reinterpret_cast<uint4*>(dv_row)[g] = make_uint4(0, 0, 0, 0);
          }
        }
        w_next = ring_pop(ring, n_ring + 1, it_next, ab);
        ring_release(ring, n_ring);
        it = it_next;
        w = w_next;
        vec_ready = false;
        ++n_ring;
        continue;
      }
      const int n_steps = nq * G;
      const bool partial_keys = it.kv_start + TILE > it.len_k;

      // vectors of the first step, unless the previous item already fetched them
      if (!vec_ready) {
        float l, d;
        int p;
        const bool ok = fetch_vec(it, it.kvh * G, it.i0, l, d, p);
        if (tid < TILE) {
          s_lse[idx & 1u][tid] = ok ? l : 0.f;
          s_delta[idx & 1u][tid] = ok ? d : 0.f;
          s_pos[idx & 1u][tid] = ok ? p : -1;
        }
        named_barrier_sync(3, 256);
      }

      int g_nx = 0, i_nx = 0;   // (head of the group, query tile) of step s + 1, advanced without a division
      for (int s = 0; s < n_steps; ++s, ++idx) {
        if (++i_nx == nq) {
          i_nx = 0;
          ++g_nx;
        }
        const uint32_t vb = idx & 1u;
        // prefetch the vectors of the next step
        // the vectors of the next step travel global -> shared asynchronously (the buffer they land
        // in was last read before barrier 2 of the previous step)
        const bool has_next = (s + 1 < n_steps);
        bool next_ok = true;
        if (!has_next) {
          w_next = ring_pop(ring, n_ring + 1, it_next, ab);
          vec_next = (w_next >= 0) && (it_next.i_end > it_next.i0);
        }
        if ((has_next || vec_next) && tid < TILE) {
          const DkvItem& src = has_next ? it : it_next;
          const int hq_nx = src.kvh * G + (has_next ? g_nx : 0);
          const int r = (src.i0 + (has_next ? i_nx : 0)) * TILE + tid;
          const int rc = min(r, src.nsel - 1);
          next_ok = r < src.nsel;
          const size_t sidx = (size_t)hq_nx * a.cap + src.bos_q + rc;
          cp_async_4(&s_lse[vb ^ 1u][tid], a.lse_sel + sidx);
          cp_async_4(&s_delta[vb ^ 1u][tid], a.delta_sel + sidx);
          if (a.q_idx) cp_async_4(&s_pos[vb ^ 1u][tid], a.pos_ids + src.bos_q + rc);
          else s_pos[vb ^ 1u][tid] = next_ok ? r : -1;
        }

        const int pos_first = s_pos[vb][0], pos_last = s_pos[vb][TILE - 1];
        const bool masked = partial_keys || pos_last < 0 || pos_first < it.kv_start + TILE - 1 ||
                            (a.window > 0 && pos_last > it.kv_start + a.window);
        uint32_t p0[32], p1[32];
        mbar_wait(&st_full, idx & 1u, ab);
        tc_fence_after();
        tmem_ld32(TM_ST + lane_off + (uint32_t)col0, p0);
        tmem_ld32(TM_ST + lane_off + (uint32_t)col0 + 32, p1);
        tmem_ld_wait();
        prob_chunk_col(p0, c, &s_lse[vb][col0], &s_pos[vb][col0], masked, key_valid, key_pos, a.window);
        prob_chunk_col(p1, c, &s_lse[vb][col0 + 32], &s_pos[vb][col0 + 32], masked, key_valid, key_pos, a.window);
        {
          uint32_t pk[32];
          pack_chunk(p0, pk);
          pack_chunk(p1, pk + 16);
          // P^T (bf16) overwrites the first 32 of the 64 S^T columns this warp has just read: private
          // to the warp, no barrier needed
          tmem_st32(TM_ST + lane_off + (uint32_t)col0, pk);
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive_warp(&p_ready);
        }
        mbar_wait(&dpt_full, idx & 1u, ab);
        tc_fence_after();
        {
          uint32_t pk[32];
          {
            uint32_t d0[32], d1[32];
            tmem_ld32(TM_DPT + lane_off + (uint32_t)col0, d0);
            tmem_ld32(TM_DPT + lane_off + (uint32_t)col0 + 32, d1);
            tmem_ld_wait();
            ds_pack_chunk_col(p0, d0, &s_delta[vb][col0], pk);
            ds_pack_chunk_col(p1, d1, &s_delta[vb][col0 + 32], pk + 16);
          }
          if ((has_next || vec_next) && tid < TILE) {
            cp_async_wait_all();
            if (!next_ok) s_pos[vb ^ 1u][tid] = -1;   // rows past the end of the sequence see no key
          }
          named_barrier_sync(2, 256);   // vector buffers: this step.s reads done, next step.s values visible
          tmem_st32(TM_DPT + lane_off + (uint32_t)col0, pk);
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive_warp(&ds_ready);
        }
      }

      // ---- epilogue ----
      mbar_wait(&acc_done, n_items & 1u, ab);
      tc_fence_after();
      ++n_items;
      {
        const long long row_off =
            key_valid ? (long long)(((size_t)(it.bos_k + key_pos) * a.h + it.kvh) * HEAD_DIM + col0) : -1;
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          const uint32_t base = (which == 0 ? TM_DK : TM_DV) + lane_off + (uint32_t)col0;
          const float mul = (which == 0) ? a.scale : 1.f;
#pragma unroll
          for (int chk = 0; chk < 2; ++chk) {
            uint32_t r[32], pk[16];
            tmem_ld32(base + chk * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i)
              pk[i] = pack_bf16x2(__uint_as_float(r[2 * i]) * mul, __uint_as_float(r[2 * i + 1]) * mul);
            store_patch_32x32(s_stage[warp], pk, which == 0 ? a.dk : a.dv, row_off >= 0 ? row_off + chk * 32 : -1, lane);
          }
        }
      }
      tc_fence_before();
      ring_release(ring, n_ring);
      it = it_next;
      w = w_next;
      vec_ready = vec_next;
      ++n_ring;
    }
  } else if (warp == 8) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_do);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      uint32_t q_iter = 0, n_items = 0, n_pub = 0;
      DkvItem it, it_ahead;
      long long w_last = -1;
      auto next_item = [&](DkvItem& dst) -> bool {
        const long long w = ring_claim(a.counter_dkv, total_items, ab);
        if (w >= 0) dkv_decode_item(a, (int)w, dst);
        ring_publish(ring, n_pub++, w, dst, ab);
        w_last = w;
        return w >= 0;
      };
      bool have = next_item(it);
      while (have) {
        const int nq = max(it.i_end - it.i0, 0);
        if (nq > 0) {
          const int xk = it.kvh * HEAD_DIM, yk = it.bos_k + it.kv_start;
          mbar_wait(&kv_free, (n_items & 1u) ^ 1u, ab);
          mbar_arrive_expect_tx(&kv_full, 2 * TILE_BYTES);
          tma_load_2d(sK, &tm_k, &kv_full, xk, yk);
          tma_load_2d(sK + BLK_BYTES, &tm_k, &kv_full, xk + 64, yk);
          tma_load_2d(sV, &tm_v, &kv_full, xk, yk);
          tma_load_2d(sV + BLK_BYTES, &tm_v, &kv_full, xk + 64, yk);
          ++n_items;
        }
        // Look one item ahead (decode and publish it before this item's Q/dO stream) while the list is long;
        // near its end claim late, so that no CTA sits on an item another CTA could already run.
        const bool ahead = (total_items - w_last) > 6ll * gridDim.x;
        bool have_ahead = ahead ? next_item(it_ahead) : false;
        int g = 0, i = it.i0;   // query head of the group, query tile
        for (int s = 0; s < nq * G; ++s, ++q_iter, ++i) {
          if (i == it.i_end) {
            i = it.i0;
            ++g;
          }
          const uint32_t st = q_iter & 1u, ph = (q_iter >> 1) & 1u;
          const int x = (it.kvh * G + g) * HEAD_DIM, y = it.bos_q + i * TILE;
          mbar_wait(&q_empty[st], ph ^ 1u, ab);
          mbar_arrive_expect_tx(&q_full[st], TILE_BYTES);
          tma_load_2d(sQ + st * TILE_BYTES, &tm_q, &q_full[st], x, y);
          tma_load_2d(sQ + st * TILE_BYTES + BLK_BYTES, &tm_q, &q_full[st], x + 64, y);
          mbar_wait(&do_empty[st], ph ^ 1u, ab);
          mbar_arrive_expect_tx(&do_full[st], TILE_BYTES);
          tma_load_2d(sDO + st * TILE_BYTES, &tm_do, &do_full[st], x, y);
          tma_load_2d(sDO + st * TILE_BYTES + BLK_BYTES, &tm_do, &do_full[st], x + 64, y);
        }
        if (!ahead) have_ahead = next_item(it_ahead);
        it = it_ahead;
        have = have_ahead;
      }
      if (abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else {
    {   // MMA issuer: the whole warp walks this code, an elected lane issues (see umma_ss)
      const uint32_t idesc_kk = umma_idesc_bf16(TILE, TILE, 0, 0);
      const uint32_t idesc_mn = umma_idesc_bf16(TILE, HEAD_DIM, 0, 1);
      const uint32_t k_base = smem_u32(sK), v_base = smem_u32(sV), q_base = smem_u32(sQ), do_base = smem_u32(sDO);
      uint32_t q_iter = 0, n_items = 0;

      auto issue_kk = [&](uint32_t d_tmem, uint32_t a_base, uint32_t b_base) {
        umma_tile_k128<false, false>(d_tmem, umma_desc_sw128(a_base, 0, 1024), umma_desc_sw128(b_base, 0, 1024),
                                     idesc_kk, 0u);
      };
      auto issue_ts = [&](uint32_t d_tmem, uint32_t a_tmem, uint32_t b_base, bool acc) {
        umma_tile_k128<true, true, 2>(d_tmem, a_tmem, umma_desc_sw128(b_base, BLK_BYTES, 1024), idesc_mn,
                                         acc ? 1u : 0u);
      };

      for (uint32_t n_ring = 0;; ++n_ring) {
        DkvItem it;
        const long long w = ring_pop(ring, n_ring, it, ab);
        if (w < 0) break;
        const int nq = it.i_end - it.i0;
        if (nq <= 0) {
          ring_release(ring, n_ring);
          continue;
        }
        const int n_steps = nq * G;
        mbar_wait(&kv_full, n_items & 1u, ab);
        ++n_items;
        tc_fence_after();
        {
          const uint32_t st = q_iter & 1u, ph = (q_iter >> 1) & 1u;
          mbar_wait(&q_full[st], ph, ab);
          tc_fence_after();
          issue_kk(TM_ST, k_base, q_base + st * TILE_BYTES);
          umma_commit(&st_full);
          mbar_wait(&do_full[st], ph, ab);
          tc_fence_after();
          issue_kk(TM_DPT, v_base, do_base + st * TILE_BYTES);
          umma_commit(&dpt_full);
        }
        for (int s = 0; s < n_steps; ++s, ++q_iter) {
          const uint32_t st = q_iter & 1u;
          const uint32_t nx = q_iter + 1u, st_n = nx & 1u, ph_n = (nx >> 1) & 1u;
          const bool has_next = (s + 1 < n_steps);
          // every product that reads K / V has been issued: the next item's tiles may come in while
          // this item's last two accumulations and its epilogue run
          if (!has_next) umma_commit(&kv_free);
          mbar_wait(&p_ready, q_iter & 1u, ab);
          tc_fence_after();
          issue_ts(TM_DV, TM_ST, do_base + st * TILE_BYTES, s > 0);
          umma_commit(&do_empty[st]);
          if (has_next) {
            mbar_wait(&q_full[st_n], ph_n, ab);
            tc_fence_after();
            issue_kk(TM_ST, k_base, q_base + st_n * TILE_BYTES);
            umma_commit(&st_full);
          }
          mbar_wait(&ds_ready, q_iter & 1u, ab);
          tc_fence_after();
          issue_ts(TM_DK, TM_DPT, q_base + st * TILE_BYTES, s > 0);
          umma_commit(&q_empty[st]);
          if (has_next) {
            mbar_wait(&do_full[st_n], ph_n, ab);
            tc_fence_after();
            issue_kk(TM_DPT, v_base, do_base + st_n * TILE_BYTES);
            umma_commit(&dpt_full);
          }
        }
        umma_commit(&acc_done);
        ring_release(ring, n_ring);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
struct BwdWorkspace {
  __nv_bfloat16* q_sel;
  __nv_bfloat16* do_sel;
  float* lse_sel;
  float* delta_sel;
  float* dq_acc;      // [cap][hq][128] fp32 accumulator of the single-pass backward
  __nv_bfloat16* vec_split;   // [cap][hq][16]: -lse / c and -delta as three bf16 terms each (single-pass backward)
  int cap;
  size_t bytes;
};

static BwdWorkspace bwd_workspace_layout(void* base, int n_tokens, int hq, bool gathered) {
  BwdWorkspace w{};
  w.cap = gathered ? n_tokens + TILE : n_tokens;
  w.cap = (w.cap + 3) & ~3;
  uint8_t* p = static_cast<uint8_t*>(base);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    uint8_t* r = p ? p + off : nullptr;
    off += (bytes + 255) & ~size_t(255);
    return r;
  };
  if (gathered) {
    w.q_sel = reinterpret_cast<__nv_bfloat16*>(take((size_t)w.cap * hq * HEAD_DIM * 2));
    w.do_sel = reinterpret_cast<__nv_bfloat16*>(take((size_t)w.cap * hq * HEAD_DIM * 2));
  }
  w.lse_sel = reinterpret_cast<float*>(take((size_t)w.cap * hq * 4));
  w.delta_sel = reinterpret_cast<float*>(take((size_t)w.cap * hq * 4));
  w.dq_acc = reinterpret_cast<float*>(take((size_t)w.cap * hq * HEAD_DIM * 4));
  w.vec_split = reinterpret_cast<__nv_bfloat16*>(take((size_t)w.cap * hq * 16 * 2));
  w.bytes = off;
  return w;
}

// Which backward runs, per branch (0 = global / query-sparse, 1 = local / window):
// 0 single pass (five tile products, dQ by fp32 reductions), 1 two kernels (seven products, every
// output accumulated in a fixed order).
static std::atomic<int> g_bwd_mode[2] = {{0}, {1}};

static int launch_attn_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse,
                           const void* d_o, void* dq, void* dk, void* dv, const int64_t* q_idx,
                           const int32_t* pos_ids, const int32_t* cu_q, const int32_t* cu_k, const int32_t* tile_off_q,
                           const int32_t* n_qtiles, const int32_t* tile_off_k, const int32_t* n_ktiles,
                           const int32_t* sq_ptr, int* counter_dq, int* counter_dkv, int n_seq, int n_tokens, int hq, int h, int window, float scale,
                           void* workspace, size_t workspace_bytes, int32_t* status, cudaStream_t stream) {
  const bool gathered = (q_idx != nullptr);
  BwdWorkspace ws = bwd_workspace_layout(workspace, n_tokens, hq, gathered);
  LOGO_REQUIRE(workspace && workspace_bytes >= ws.bytes, LOGO_ERR_WORKSPACE,
               "attention backward workspace too small: need %zu bytes", ws.bytes);
  LOGO_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, LOGO_ERR_INVALID,
               "attention backward workspace must be 256-byte aligned");

  const bool fused = g_bwd_mode[gathered ? 0 : 1].load(std::memory_order_relaxed) == 0;
  if (gathered && !fused) {   // dQ of unselected rows is zero (the single-pass kernel writes the zeros itself)
    const int rc0 = launch_zero_unselected_rows(dq, q_idx, sq_ptr, n_tokens,
                                                (size_t)hq * HEAD_DIM * sizeof(__nv_bfloat16), stream);
    if (rc0) return rc0;
  }

  const int sms = sm_count();
  prof_begin(PROF_BWD_PRE, stream);
  bwd_preprocess_kernel<<<sms * 4, 256, 0, stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, lse, q_idx, sq_ptr, ws.q_sel,
      ws.do_sel, ws.lse_sel, ws.delta_sel, fused ? ws.dq_acc : nullptr, fused ? ws.vec_split : nullptr,
      1.f / (scale * 1.4426950408889634f), ws.cap, n_tokens, hq, status);
  prof_end(PROF_BWD_PRE, stream);
  LOGO_CHECK_CUDA(cudaGetLastError());

  CUtensorMap tm_q, tm_do, tm_k, tm_v;
  const uint64_t q_row_bytes = (uint64_t)hq * HEAD_DIM * 2, kv_row_bytes = (uint64_t)h * HEAD_DIM * 2;
  const void* q_src = gathered ? (const void*)ws.q_sel : q;
  const void* do_src = gathered ? (const void*)ws.do_sel : d_o;
  const uint64_t q_rows = gathered ? (uint64_t)ws.cap : (uint64_t)n_tokens;
  int rc;
  if ((rc = make_tmap_2d_bf16(&tm_q, q_src, (uint64_t)hq * HEAD_DIM, q_rows, q_row_bytes, 64, TILE))) return rc;
  if ((rc = make_tmap_2d_bf16(&tm_do, do_src, (uint64_t)hq * HEAD_DIM, q_rows, q_row_bytes, 64, TILE))) return rc;
  if ((rc = make_tmap_2d_bf16(&tm_k, k, (uint64_t)h * HEAD_DIM, (uint64_t)n_tokens, kv_row_bytes, 64, TILE))) return rc;
  if ((rc = make_tmap_2d_bf16(&tm_v, v, (uint64_t)h * HEAD_DIM, (uint64_t)n_tokens, kv_row_bytes, 64, TILE))) return rc;

  BwdArgs a{};
  a.q_idx = q_idx;
  a.sq_ptr = sq_ptr;
  a.pos_ids = pos_ids;
  a.cu_q = cu_q;
  a.cu_k = cu_k;
  a.tile_off_q = tile_off_q;
  a.n_qtiles = n_qtiles;
  a.tile_off_k = tile_off_k;
  a.n_ktiles = n_ktiles;
  a.counter_dq = counter_dq;
  a.counter_dkv = counter_dkv;
  a.lse_sel = ws.lse_sel;
  a.delta_sel = ws.delta_sel;
  a.cap = ws.cap;
  a.dq = (__nv_bfloat16*)dq;
  a.dk = (__nv_bfloat16*)dk;
  a.dv = (__nv_bfloat16*)dv;
  a.n_seq = n_seq;
  a.n_tokens = n_tokens;
  a.hq = hq;
  a.h = h;
  a.window = window;
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;

  if (fused) return launch_attn_bwd_fused(tm_q, tm_do, tm_k, tm_v, a, ws.dq_acc, ws.vec_split, sq_ptr, stream);

  static thread_local int attr_set_dev = -1;
  int dev = 0;
  LOGO_CHECK_CUDA(cudaGetDevice(&dev));
  if (attr_set_dev != dev) {
    LOGO_CHECK_CUDA(
        cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM_BYTES));
    LOGO_CHECK_CUDA(
        cudaFuncSetAttribute(attn_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM_BYTES));
    attr_set_dev = dev;
  }
  LOGO_CHECK_CUDA(cudaMemsetAsync(counter_dq, 0, sizeof(int), stream));
  LOGO_CHECK_CUDA(cudaMemsetAsync(counter_dkv, 0, sizeof(int), stream));
  prof_begin(PROF_BWD_DKV, stream);
  attn_bwd_dkv_kernel<<<sms, BWD_THREADS, BWD_SMEM_BYTES, stream>>>(tm_q, tm_do, tm_k, tm_v, a);
  prof_end(PROF_BWD_DKV, stream);
  LOGO_CHECK_CUDA(cudaGetLastError());
  prof_begin(PROF_BWD_DQ, stream);
  attn_bwd_dq_kernel<<<sms, DQ_THREADS, BWD_SMEM_BYTES, stream>>>(tm_q, tm_do, tm_k, tm_v, a);
  prof_end(PROF_BWD_DQ, stream);
  LOGO_CHECK_CUDA(cudaGetLastError());
  return LOGO_OK;
}

}  // namespace logo

extern "C" int logo_set_backward_mode(int branch, int mode) {
  using namespace logo;
  LOGO_REQUIRE(branch == 0 || branch == 1, LOGO_ERR_INVALID, "branch must be 0 (global) or 1 (local), got %d", branch);
  LOGO_REQUIRE(mode == 0 || mode == 1, LOGO_ERR_INVALID, "mode must be 0 (single pass) or 1 (two kernels), got %d", mode);
  g_bwd_mode[branch].store(mode, std::memory_order_relaxed);
  return LOGO_OK;
}

extern "C" int logo_get_backward_mode(int branch) {
  return (branch == 0 || branch == 1) ? logo::g_bwd_mode[branch].load(std::memory_order_relaxed) : -1;
}

extern "C" size_t logo_attn_bwd_workspace_bytes(int n_tokens, int hq, int gathered) {
  if (n_tokens < 0 || hq <= 0) return 0;
  return logo::bwd_workspace_layout(nullptr, n_tokens, hq, gathered != 0).bytes;
}

extern "C" int logo_sq_attn_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse,
                                const void* d_o, void* dq, void* dk, void* dv, const int64_t* q_idx,
                                const int32_t* pos_ids, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                const int32_t* tile_off, int32_t* meta, void* workspace, size_t workspace_bytes,
                                int n_seq, int n_tokens, int hq, int h, int d, float scale, int32_t* status,
                                logo_stream_t stream) {
  using namespace logo;
  LOGO_REQUIRE(d == HEAD_DIM, LOGO_ERR_UNSUPPORTED, "head_dim %d is not supported (only 128)", d);
  LOGO_REQUIRE(hq > 0 && h > 0 && hq % h == 0, LOGO_ERR_INVALID, "hq (%d) must be a positive multiple of h (%d)", hq, h);
  LOGO_REQUIRE(n_tokens >= 0 && n_seq >= 0, LOGO_ERR_INVALID, "n_tokens and n_seq must be non-negative");
  if (n_tokens == 0 || n_seq == 0) return LOGO_OK;
  LOGO_REQUIRE(q && k && v && o && lse && d_o && dq && dk && dv, LOGO_ERR_INVALID, "tensor pointers must not be NULL");
  LOGO_REQUIRE(q_idx && pos_ids && cu_seqlens_q && cu_seqlens_k && tile_off && meta, LOGO_ERR_INVALID,
               "selection metadata pointers must not be NULL");
  LOGO_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o) && aligned16(d_o) && aligned16(dq) &&
                   aligned16(dk) && aligned16(dv),
               LOGO_ERR_INVALID, "tensors must be 16-byte aligned");
  return launch_attn_bwd(q, k, v, o, lse, d_o, dq, dk, dv, q_idx, pos_ids, cu_seqlens_q, cu_seqlens_k,
                         tile_off + 3 * (n_seq + 1), meta + 4, tile_off + (n_seq + 1), meta + 2, meta,
                         meta + LOGO_META_COUNTER_SQ_DQ, meta + LOGO_META_COUNTER_SQ_DKV, n_seq, n_tokens, hq, h, 0, scale, workspace, workspace_bytes, status, (cudaStream_t)stream);
}

extern "C" int logo_swa_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse,
                            const void* d_o, void* dq, void* dk, void* dv, const int32_t* cu_seqlens,
                            const int32_t* tile_off, int32_t* meta, void* workspace, size_t workspace_bytes,
                            int n_seq, int n_tokens, int hq, int h, int d, int window, float scale, int32_t* status,
                            logo_stream_t stream) {
  using namespace logo;
  LOGO_REQUIRE(d == HEAD_DIM, LOGO_ERR_UNSUPPORTED, "head_dim %d is not supported (only 128)", d);
  LOGO_REQUIRE(hq > 0 && h > 0 && hq % h == 0, LOGO_ERR_INVALID, "hq (%d) must be a positive multiple of h (%d)", hq, h);
  LOGO_REQUIRE(window > 0, LOGO_ERR_INVALID, "window must be positive, got %d", window);
  LOGO_REQUIRE(n_tokens >= 0 && n_seq >= 0, LOGO_ERR_INVALID, "n_tokens and n_seq must be non-negative");
  if (n_tokens == 0 || n_seq == 0) return LOGO_OK;
  LOGO_REQUIRE(q && k && v && o && lse && d_o && dq && dk && dv, LOGO_ERR_INVALID, "tensor pointers must not be NULL");
  LOGO_REQUIRE(cu_seqlens && tile_off && meta, LOGO_ERR_INVALID, "cu_seqlens, tile_off and meta must not be NULL");
  LOGO_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o) && aligned16(d_o) && aligned16(dq) &&
                   aligned16(dk) && aligned16(dv),
               LOGO_ERR_INVALID, "tensors must be 16-byte aligned");
  // identity selection: query tiles == key tiles (row 1 of tile_off, meta[2])
  return launch_attn_bwd(q, k, v, o, lse, d_o, dq, dk, dv, nullptr, nullptr, cu_seqlens, cu_seqlens,
                         tile_off + (n_seq + 1), meta + 2, tile_off + (n_seq + 1), meta + 2, nullptr,
                         meta + LOGO_META_COUNTER_SWA_DQ, meta + LOGO_META_COUNTER_SWA_DKV, n_seq, n_tokens, hq, h, window,
                         scale, workspace, workspace_bytes, status, (cudaStream_t)stream);
}
