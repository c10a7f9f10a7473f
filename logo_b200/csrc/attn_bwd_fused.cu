// Single-pass backward attention: dK, dV and dQ from ONE evaluation of S and dP per
// (query tile, key tile) pair, five tile products instead of the seven of the two-kernel path.
//
// Work item = (128-key tile, kv head); the CTA keeps the K / V tile in shared memory and the
// dK / dV accumulators in tensor memory and streams the Q / dO tiles of every query head of
// the group that can see the key tile. Per step (one query tile):
//     S^T  = K Q^T - lse / c  -> TMEM X           (both operands K-major in shared memory; the row
//     dP^T = V dO^T - delta   -> TMEM Y            vectors are added by a ninth k-step, see below)
//     P^T  = exp2(S^T c) masked, bf16             -> written into X (the A operand of dV)
//     dV  += P^T dO                               (A from TMEM, B = dO tile read MN-major)
//     dS^T = P^T o dP^T, bf16                     -> written to SHARED memory as a [key][query]
//                                                    tile, into the dO stage dV has finished with
//     dK  += dS^T Q                               (A = the dS^T tile K-major, B = Q tile MN-major)
//     dQ^T = K^T dS^T         -> TMEM Y           (A = the K tile read MN-major, B = dS^T MN-major)
// lse and delta are per query row, i.e. per COLUMN of the transposed tiles: every thread of the
// element-wise warps would need all 64 values of its columns, 16-byte broadcast loads that cost the
// shared-memory pipe one wavefront per 4 bytes per warp (a quarter of its thread traffic, and the
// pipe is what bounds this kernel). Instead the preprocess kernel writes -lse / c and -delta of every
// (row, head) as three bf16 terms each (24 bits) into a [rows][heads][16] array; the tile of a step
// comes in by TMA with the Q tile (32-byte swizzle) and is the B operand of one more k-step whose A
// operand is a constant tile of ones in the matching columns: exact products, fp32 sums.
// dQ^T of the step (rows = head dimension, columns = query rows) is read out of Y by four
// dedicated warps; each lays its 32 head-dimension columns down as fp32 [query][32] pieces, 32 query
// rows at a time, in its own double-buffered part of the 32 KB staging tile X and adds them to an
// fp32 accumulator in global memory by bulk tensor reductions of its own (cp.reduce.async.bulk: the
// reduction runs in L2; per-thread red.global.add was measured 2.5x slower, bound by the SM's
// atomic issue rate; waiting for each reduction before staging the next piece cost 3000 clocks a step).
// bwd_dq_finish_kernel scales, converts and scatters the accumulator to the token rows afterwards.
// Tensor memory is full (X, Y, dK, dV = 512 columns): dQ^T shares Y with dP^T, so the next
// dP^T waits until the read-out warps hold the previous dQ^T in registers.
//
// Warp roles (512 threads = four warpgroups): 0-7 element-wise (lane quarter w % 4, 64 query
// columns each), 8-11 dQ read-out (one per lane quarter), 12 TMA producer + work claiming, 13 MMA
// issue, 14-15 zero the dQ rows of the tokens the selection leaves out (HBM traffic that hides under
// the products). The kernel starts with 128 registers per thread; the element-wise warpgroups
// raise their share to 160 with setmaxnreg (they keep a 64-column fp32 P row and a dP chunk live),
// the read-out warpgroup takes 144 (a whole 128-column row of dQ^T in registers, so that Y is released
// after one round of loads) and the last one drops to 48: every scheduler holds one warp of each
// warpgroup, 160 + 160 + 144 + 48 = 512 registers per lane = its whole register file.
//
// The order in which key tiles reach a dQ row is not fixed, so dQ can differ between runs in
// the last bit of its fp32 sum (dK and dV are accumulated in a fixed order and are reproducible).
#include "attn_bwd_common.cuh"

namespace logo {

constexpr int FUSED_EW_WARPS = 8;
constexpr int FUSED_DQ_WARPS = 4;
constexpr int FUSED_THREADS = 512;

__device__ __forceinline__ void reg_inc_ew() { asm volatile("setmaxnreg.inc.sync.aligned.u32 160;"); }
__device__ __forceinline__ void reg_dec_dq() { asm volatile("setmaxnreg.inc.sync.aligned.u32 144;"); }
__device__ __forceinline__ void reg_dec_misc() { asm volatile("setmaxnreg.dec.sync.aligned.u32 48;"); }

// Shared memory (all of it dynamic, so that the 1024-byte alignment the swizzled tiles need costs no
// padding): seven 32 KB tiles, then the per-step vectors, barriers and the work-item ring.
struct FusedSmem {
  static constexpr uint32_t K = 0, V = TILE_BYTES, Q = 2 * TILE_BYTES, DO = 4 * TILE_BYTES, X = 6 * TILE_BYTES;
  static constexpr uint32_t X_BYTES = 24576;                 // four read-out warps x three 2 KB buffers
  static constexpr uint32_t VEC_BYTES = TILE * 32;           // one [128][16] bf16 tile, 32-byte swizzle
  static constexpr uint32_t VEC = X + X_BYTES;               // 2 stages, loaded with the Q tile
  static constexpr uint32_t ONES_BYTES = 256;                // a [128][16] tile of identical rows (see sOnes)
  static constexpr uint32_t ONES = VEC + 2 * VEC_BYTES;      // two of them
  static constexpr uint32_t POS = ONES + 2 * ONES_BYTES;
  static constexpr uint32_t BARS = POS + TILE * 4;          // 8-byte aligned
  static constexpr uint32_t N_BARS = 21 + 2 * ITEM_RING;
  static constexpr uint32_t ITEMS = BARS + N_BARS * 8;
  static constexpr uint32_t MISC = ITEMS + ITEM_RING * ITEM_WORDS * 4;   // tmem slot, abort flag
  static constexpr uint32_t BYTES = MISC + 16;
};
static_assert(FusedSmem::BYTES <= 232448, "the single-pass backward does not fit the 227 KB of shared memory");

__global__ void __launch_bounds__(FUSED_THREADS, 1)
    attn_bwd_fused_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                          const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                          const __grid_constant__ CUtensorMap tm_dq, const __grid_constant__ CUtensorMap tm_vec,
                          const BwdArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem + FusedSmem::K;
  uint8_t* sV = smem + FusedSmem::V;
  uint8_t* sQ = smem + FusedSmem::Q;      // 2 stages
  uint8_t* sDO = smem + FusedSmem::DO;    // 2 stages; stage s & 1 holds dS^T of step s once dV(s) is done
  // X: pieces of a step's dQ tile on their way to the bulk reductions; at the end of an item the
  // staging of the dK / dV stores
  uint8_t* sX = smem + FusedSmem::X;
  // -lse / c and -delta of the step's 128 query rows travel as three bf16 terms each in columns 0-2 and
  // 3-5 of a [128][16] tile (the B operand of a ninth k-step); the matching A tiles hold ones in those
  // columns for every key row, so the tensor core adds the row vectors to S^T and dP^T (exact products,
  // fp32 sums) and the element-wise warps never load them. All rows of an A tile being equal, it is
  // stored as two 128-byte core matrices without swizzle and a zero distance between 8-row groups.
  uint8_t* sOnes = smem + FusedSmem::ONES;
  uint8_t* sVec = smem + FusedSmem::VEC;
  int* s_pos = reinterpret_cast<int*>(smem + FusedSmem::POS);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FusedSmem::BARS);
  uint64_t &k_full = bars[0], &k_free = bars[1], &v_full = bars[19], &v_free = bars[20], *q_full = bars + 2, *q_empty = bars + 4, *do_full = bars + 6,
           *do_empty = bars + 8, &st_full = bars[10], &dpt_full = bars[11], &p_ready = bars[12], &ds_ready = bars[13],
           &dq_full = bars[14], &dv_done = bars[15], &dq_read = bars[16], &acc_read = bars[17], &acc_done = bars[18];
  const ItemRing ring{reinterpret_cast<int*>(smem + FusedSmem::ITEMS), bars + 21, bars + 21 + ITEM_RING};
  uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(smem + FusedSmem::MISC);
  int& abort_flag = *reinterpret_cast<int*>(smem + FusedSmem::MISC + 4);

  const int tid = threadIdx.x, warp = uniform_warp_idx(), lane = tid & 31;
  AbortState ab{&abort_flag, a.status};

  // the tile layouts (TMA 128-byte swizzle, UMMA descriptors) assume a 1024-byte aligned base
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (tid == 0 && a.status) atomicCAS(a.status, 0, (int)DEV_BAD_INDEX);
    return;
  }

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&k_full, 1);
    mbar_init(&k_free, 1);
    mbar_init(&v_full, 1);
    mbar_init(&v_free, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
      mbar_init(&do_full[s], 1);
      mbar_init(&do_empty[s], 1);
    }
    mbar_init(&st_full, 1);
    mbar_init(&dpt_full, 1);
    mbar_init(&p_ready, FUSED_EW_WARPS);    // one arrival per warp
    mbar_init(&ds_ready, FUSED_EW_WARPS);
    mbar_init(&dq_full, 1);
    mbar_init(&dv_done, 1);
    mbar_init(&dq_read, FUSED_DQ_WARPS);
    mbar_init(&acc_read, FUSED_DQ_WARPS);   // one arrival per read-out warp
    mbar_init(&acc_done, 1);
    ring_init(ring, FUSED_EW_WARPS + FUSED_DQ_WARPS + 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_slot, 512);
    tmem_relinquish();
  }
  if (tid < 32) {
    // tile 0: ones in columns 0-2 (adds -lse / c to S^T), tile 1: ones in columns 3-5 (adds -delta to dP^T);
    // per tile 8 rows x 16 bytes for columns 0-7, then 8 rows of zeros for columns 8-15
    const int tile = tid >> 4, r = tid & 15;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < 8) v = tile == 0 ? make_uint4(0x3F803F80u, 0x00003F80u, 0u, 0u) : make_uint4(0u, 0x3F800000u, 0x3F803F80u, 0u);
    reinterpret_cast<uint4*>(sOnes + tile * FusedSmem::ONES_BYTES)[r] = v;
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t TM_X = tmem, TM_Y = tmem + 128u, TM_DK = tmem + 256u, TM_DV = tmem + 384u;

  const int total_tiles = __ldg(a.n_ktiles);
  const long long total_items = (long long)total_tiles * a.h;
  const int G = a.hq / a.h;

  if (warp < FUSED_EW_WARPS) {
    // ================= element-wise warps =================
    reg_inc_ew();
    const int quad = warp & 3, half = warp >> 2;
    const int row = quad * 32 + lane;   // key inside the tile
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const int col0 = half * 64;
    const float c = a.scale_log2;
    uint32_t idx = 0;

    // position of row `tid` of query tile `i`: loaded from a clamped row into a register (threads
    // 0-127), stored to the shared vector between two steps (lse and delta reach the tiles through the
    // tensor core, see sVec)
    auto fetch_pos = [&](const DkvItem& it, int i) -> int {
      const int r = i * TILE + (tid & (TILE - 1));
      const int rc = min(r, it.nsel - 1);
      const int p = bwd_row_position(a, it.bos_q, rc);
      return r >= it.nsel ? -1 : p;   // rows past the end of the sequence see no key
    };

    uint32_t n_ring = 0;
    DkvItem it;
    long long w = ring_pop(ring, n_ring, it, ab);
    bool vec_ready = false;   // the first-step vectors of `it` are already in the shared vectors
    while (w >= 0) {
      DkvItem it_next;
      long long w_next = -1;
      bool vec_next = false;
      const int nq = it.i_end - it.i0;
      const int key_pos = it.kv_start + row;
      const bool key_valid = key_pos < it.len_k;
      if (nq <= 0) {
        // no query can see this key tile: the gradients are zero
        if (key_valid) {
          __nv_bfloat16* dk_row = a.dk + ((size_t)(it.bos_k + key_pos) * a.h + it.kvh) * HEAD_DIM + col0;
          __nv_bfloat16* dv_row = a.dv + ((size_t)(it.bos_k + key_pos) * a.h + it.kvh) * HEAD_DIM + col0;
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

      if (!vec_ready) {
        if (tid < TILE) s_pos[tid] = fetch_pos(it, it.i0);
        named_barrier_sync(3, 256);
      }

      int g_nx = 0, i_nx = 0;   // (head of the group, query tile) of step s + 1
      for (int s = 0; s < n_steps; ++s, ++idx) {
        if (++i_nx == nq) {
          i_nx = 0;
          ++g_nx;
        }
        // the vectors of the next step (of the next item after the last step) start travelling now
        const bool has_next = (s + 1 < n_steps);
        if (!has_next) {
          w_next = ring_pop(ring, n_ring + 1, it_next, ab);
          vec_next = (w_next >= 0) && (it_next.i_end > it_next.i0);
        }
        int p_nx = -1;
        if ((has_next || vec_next) && tid < TILE)
          p_nx = has_next ? fetch_pos(it, it.i0 + i_nx) : fetch_pos(it_next, it_next.i0);

        const int pos_first = s_pos[0], pos_last = s_pos[TILE - 1];
        const bool masked = partial_keys || pos_last < 0 || pos_first < it.kv_start + TILE - 1 ||
                            (a.window > 0 && pos_last > it.kv_start + a.window);
        uint32_t p0[32], p1[32];
        mbar_wait(&st_full, idx & 1u, ab);
        tc_fence_after();
        tmem_ld32(TM_X + lane_off + (uint32_t)col0, p0);
        tmem_ld32(TM_X + lane_off + (uint32_t)col0 + 32, p1);
        tmem_ld_wait();
        // X holds S^T - lse / c: the probabilities are one multiply and one exponential per element
        prob_chunk_biased(p0, c, &s_pos[col0], masked, key_valid, key_pos, a.window);
        prob_chunk_biased(p1, c, &s_pos[col0 + 32], masked, key_valid, key_pos, a.window);
        {
          uint32_t pk[32];
          pack_chunk(p0, pk);
          pack_chunk(p1, pk + 16);
          // P^T (bf16) overwrites the first 32 of the 64 S^T columns this warp has just read
          tmem_st32(TM_X + lane_off + (uint32_t)col0, pk);
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive_warp(&p_ready);
        }
        mbar_wait(&dpt_full, idx & 1u, ab);
        tc_fence_after();
        uint32_t ds[32];   // dS^T of this thread's key row, 64 query columns, packed bf16
        {
          uint32_t d0[32];
          tmem_ld32(TM_Y + lane_off + (uint32_t)col0, d0);
          tmem_ld_wait();
          ds_pack_chunk_biased(p0, d0, ds);   // Y holds dP^T - delta
        }
        {
          uint32_t d1[32];
          tmem_ld32(TM_Y + lane_off + (uint32_t)col0 + 32, d1);
          tmem_ld_wait();
          ds_pack_chunk_biased(p1, d1, ds + 16);
        }
        tc_fence_before();   // Y has been read: after ds_ready the MMA warp may overwrite it with dQ^T
        // dS^T goes into the dO stage of this step as a [key][query] tile (two [128][64] blocks,
        // 128-byte swizzled): dV(s) was the last reader of the dO tile
        mbar_wait(&dv_done, idx & 1u, ab);
        {
          uint8_t* dst = sDO + (idx & 1u) * TILE_BYTES + (uint32_t)half * BLK_BYTES + (uint32_t)row * 128u;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(dst + (((uint32_t)ch ^ ((uint32_t)row & 7u)) << 4)) =
                make_uint4(ds[4 * ch], ds[4 * ch + 1], ds[4 * ch + 2], ds[4 * ch + 3]);
        }
        fence_proxy_async_smem();
        mbar_arrive_warp(&ds_ready);
        // hand the vectors over: every warp has finished reading this step's, then the next step's land
        named_barrier_sync(2, 256);
        if ((has_next || vec_next) && tid < TILE) s_pos[tid] = p_nx;
        named_barrier_sync(3, 256);
      }

      // (dK and dV of the item are written out by the read-out warps)
      tc_fence_before();
      ring_release(ring, n_ring);
      it = it_next;
      w = w_next;
      vec_ready = vec_next;
      ++n_ring;
    }
  } else if (warp < FUSED_EW_WARPS + FUSED_DQ_WARPS) {
    // ================= dQ read-out warps =================
    // Lane l of the warp of quarter q holds row 32 q + l of dQ^T (one element of the head dimension)
    // and the 128 query rows of the step as columns. The whole row comes into registers in one round
    // (Y is released right after it). Every warp then works alone: it owns 6 KB of X as three 2 KB
    // buffers, writes 16 query rows x its 32 head-dimension columns into one as fp32 [query row][32],
    // and its lane 0 sends the buffer to dq_acc with a bulk reduction of its own. A buffer is reused
    // only when the reduction issued three rounds earlier has read it, so the reductions (which drain at
    // about 20 bytes per clock per SM) run under the staging of the following rounds and under the
    // next step instead of being waited for one by one.
    reg_dec_dq();
    const int quad = warp & 3;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    float* const my_x = reinterpret_cast<float*>(sX + quad * 6144);   // this warp's three [16][32] fp32 buffers
    uint32_t idx = 0, n_items = 0, buf_no = 0;
    for (uint32_t n_ring = 0;; ++n_ring) {
      DkvItem it;
      const long long w = ring_pop(ring, n_ring, it, ab);
      if (w < 0) break;
      const int nq = it.i_end - it.i0;
      if (nq <= 0) {
        ring_release(ring, n_ring);
        continue;
      }
      for (int g = 0; g < G; ++g) {
        for (int i = it.i0; i < it.i_end; ++i, ++idx) {
          const int x = (it.kvh * G + g) * HEAD_DIM + quad * 32, y = it.bos_q + i * TILE;
          const int nvalid = min(it.nsel - i * TILE, TILE);
          const bool ok = mbar_wait(&dq_full, idx & 1u, ab);
          tc_fence_after();
          uint32_t r0[32], r1[32], r2[32], r3[32];
          tmem_ld32(TM_Y + lane_off, r0);
          tmem_ld32(TM_Y + lane_off + 32u, r1);
          tmem_ld32(TM_Y + lane_off + 64u, r2);
          tmem_ld32(TM_Y + lane_off + 96u, r3);
          tmem_ld_wait();
          tc_fence_before();
          mbar_arrive_warp(&dq_read);   // Y is free for the next dP^T
          // rows past the last valid query row of the tile hold exact zeros (their dS^T columns are
          // zero); rows past the end of the accumulator are clipped by the tensor map
          auto send = [&](const uint32_t (&r)[32], int k) {   // query rows 32 k .. 32 k + 31, two pieces of 16
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              if (nvalid <= 32 * k + 16 * hf) break;
              float* buf = my_x + buf_no * 512;
              if (lane == 0) bulk_wait_read_but_two();   // the reduction of three rounds ago has read this buffer
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 16; ++j) buf[j * 32 + lane] = __uint_as_float(r[16 * hf + j]);
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0 && ok) {
                tma_reduce_add_2d(&tm_dq, buf, x, y + 32 * k + 16 * hf);
                bulk_commit_group();
              }
              buf_no = buf_no == 2u ? 0u : buf_no + 1u;
            }
          };
          send(r0, 0);
          if (nvalid > 32) send(r1, 1);
          if (nvalid > 64) send(r2, 2);
          if (nvalid > 96) send(r3, 3);
        }
      }
      // ---- the item's dK * scale and dV -> bf16 rows, staged through this warp's part of X. The
      //      element-wise warps are already at the next item; the MMA warp starts its accumulators over
      //      once all four warps have read these. ----
      mbar_wait(&acc_done, n_items & 1u, ab);
      tc_fence_after();
      ++n_items;
      if (lane == 0) bulk_wait_read_all();   // no reduction still reads this warp's buffers
      __syncwarp();
      {
        const int key_pos = it.kv_start + quad * 32 + lane;
        const long long row_off =
            key_pos < it.len_k ? (long long)(((size_t)(it.bos_k + key_pos) * a.h + it.kvh) * HEAD_DIM) : -1;
        uint8_t* out_stage = reinterpret_cast<uint8_t*>(my_x);
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          const uint32_t base = (which == 0 ? TM_DK : TM_DV) + lane_off;
          const float mul = (which == 0) ? a.scale : 1.f;
#pragma unroll 1
          for (int chk = 0; chk < 4; ++chk) {
            uint32_t r[32], pk[16];
            tmem_ld32(base + chk * 32, r);
            tmem_ld_wait();
            if (which == 1 && chk == 3) {   // the accumulators are in registers / on their way out
              tc_fence_before();
              mbar_arrive_warp(&acc_read);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i)
              pk[i] = pack_bf16x2(__uint_as_float(r[2 * i]) * mul, __uint_as_float(r[2 * i + 1]) * mul);
            store_patch_32x32(out_stage, pk, which == 0 ? a.dk : a.dv, row_off >= 0 ? row_off + chk * 32 : -1, lane);
          }
        }
      }
      ring_release(ring, n_ring);
    }
    if (lane == 0) bulk_wait_all();   // the reductions of this warp are performed before the CTA leaves
  } else {
   reg_dec_misc();
   if (warp == FUSED_EW_WARPS + FUSED_DQ_WARPS) {
    // ================= producer: claims and decodes items, issues the TMA loads =================
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_do);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_vec);
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
        int g = 0, i = it.i0;   // query head of the group, query tile
        auto load_step = [&]() {   // the Q (+ row-vector) and dO tiles of the next step of this item
          if (i == it.i_end) {
            i = it.i0;
            ++g;
          }
          const uint32_t st = q_iter & 1u, ph = (q_iter >> 1) & 1u;
          const int x = (it.kvh * G + g) * HEAD_DIM, y = it.bos_q + i * TILE;
          mbar_wait(&q_empty[st], ph ^ 1u, ab);
          mbar_arrive_expect_tx(&q_full[st], TILE_BYTES + FusedSmem::VEC_BYTES);
          tma_load_2d(sQ + st * TILE_BYTES, &tm_q, &q_full[st], x, y);
          tma_load_2d(sQ + st * TILE_BYTES + BLK_BYTES, &tm_q, &q_full[st], x + 64, y);
          tma_load_2d(sVec + st * FusedSmem::VEC_BYTES, &tm_vec, &q_full[st], (it.kvh * G + g) * 16, y);
          mbar_wait(&do_empty[st], ph ^ 1u, ab);
          mbar_arrive_expect_tx(&do_full[st], TILE_BYTES);
          tma_load_2d(sDO + st * TILE_BYTES, &tm_do, &do_full[st], x, y);
          tma_load_2d(sDO + st * TILE_BYTES + BLK_BYTES, &tm_do, &do_full[st], x + 64, y);
          ++q_iter;
          ++i;
        };
        if (nq > 0) {
          // K and V are single-buffered. V is last read by the item's last dP^T, issued a whole step before
          // the item ends, so the next V tile comes in under that step; then the first Q / dO tiles (their
          // stages are free); only the K tile has to wait for the item's last product.
          const int xk = it.kvh * HEAD_DIM, yk = it.bos_k + it.kv_start;
          mbar_wait(&v_free, (n_items & 1u) ^ 1u, ab);
          mbar_arrive_expect_tx(&v_full, TILE_BYTES);
          tma_load_2d(sV, &tm_v, &v_full, xk, yk);
          tma_load_2d(sV + BLK_BYTES, &tm_v, &v_full, xk + 64, yk);
          load_step();
          mbar_wait(&k_free, (n_items & 1u) ^ 1u, ab);
          mbar_arrive_expect_tx(&k_full, TILE_BYTES);
          tma_load_2d(sK, &tm_k, &k_full, xk, yk);
          tma_load_2d(sK + BLK_BYTES, &tm_k, &k_full, xk + 64, yk);
          ++n_items;
        }
        const bool ahead = (total_items - w_last) > 6ll * gridDim.x;
        bool have_ahead = ahead ? next_item(it_ahead) : false;
        for (int s = 1; s < nq * G; ++s) load_step();
        if (!ahead) have_ahead = next_item(it_ahead);
        it = it_ahead;
        have = have_ahead;
      }
      if (abort_flag) {   // let copies in flight land before the CTA exits
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
   } else if (warp > FUSED_EW_WARPS + FUSED_DQ_WARPS + 1) {
    // ================= the two spare warps: dQ of the rows the selection leaves out is zero =================
    if (a.q_idx) {
      const int sq = min(max(__ldg(a.sq_ptr), 0), a.n_tokens);
      zero_unselected_rows_part(reinterpret_cast<uint4*>(a.dq), a.q_idx, sq, a.n_tokens, a.hq * HEAD_DIM / 8,
                                blockIdx.x * 2 + (warp - (FUSED_EW_WARPS + FUSED_DQ_WARPS + 2)), gridDim.x * 2, lane);
    }
   } else if (warp == FUSED_EW_WARPS + FUSED_DQ_WARPS + 1) {
    // ================= MMA issuer: the whole warp walks this code, an elected lane issues =================
    const uint32_t idesc_kk = umma_idesc_bf16(TILE, TILE, 0, 0);       // S^T, dP^T: both operands K-major
    const uint32_t idesc_mn = umma_idesc_bf16(TILE, HEAD_DIM, 0, 1);   // dV, dK: B operand MN-major
    const uint32_t idesc_mm = umma_idesc_bf16(HEAD_DIM, TILE, 1, 1);   // dQ^T: both operands MN-major
    const uint32_t k_base = smem_u32(sK), v_base = smem_u32(sV), q_base = smem_u32(sQ), do_base = smem_u32(sDO);
    uint32_t q_iter = 0, n_items = 0;

    // S^T = K Q^T - lse / c (ones_tile 0) or dP^T = V dO^T - delta (ones_tile 1): eight k-steps over the
    // head dimension and a ninth over the [128][16] vector tile of stage `vec_stage`
    const uint32_t ones_base = smem_u32(sOnes), vec_base = smem_u32(sVec);
    auto issue_kk = [&](uint32_t d_tmem, uint32_t a_base, uint32_t b_base, uint32_t ones_tile, uint32_t vec_stage) {
      umma_tile_k128<false, false>(d_tmem, umma_desc_sw128(a_base, 0, 1024), umma_desc_sw128(b_base, 0, 1024),
                                   idesc_kk, 0u);
      umma_ss(d_tmem, umma_desc_noswizzle(ones_base + ones_tile * FusedSmem::ONES_BYTES, 128, 0),
              umma_desc_sw32(vec_base + vec_stage * FusedSmem::VEC_BYTES), idesc_kk, 1u);
    };
    auto issue_dv = [&](uint32_t b_base, bool acc) {
      umma_tile_k128<true, true, 2>(TM_DV, TM_X, umma_desc_sw128(b_base, BLK_BYTES, 1024), idesc_mn, acc ? 1u : 0u);
    };
    auto issue_dk = [&](uint32_t ds_base, uint32_t b_base, bool acc) {
      umma_tile_k128<false, true>(TM_DK, umma_desc_sw128(ds_base, 0, 1024), umma_desc_sw128(b_base, BLK_BYTES, 1024),
                                  idesc_mn, acc ? 1u : 0u);
    };
    auto issue_dq = [&](uint32_t ds_base) {
      umma_tile_k128<false, true, 0, 0, 8, true>(TM_Y, umma_desc_sw128(k_base, BLK_BYTES, 1024),
                                                 umma_desc_sw128(ds_base, BLK_BYTES, 1024), idesc_mm, 0u);
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
      {
        const uint32_t st = q_iter & 1u, ph = (q_iter >> 1) & 1u;
        mbar_wait(&k_full, n_items & 1u, ab);
        mbar_wait(&q_full[st], ph, ab);
        tc_fence_after();
        issue_kk(TM_X, k_base, q_base + st * TILE_BYTES, 0u, st);
        umma_commit(&st_full);
        mbar_wait(&v_full, n_items & 1u, ab);
        mbar_wait(&do_full[st], ph, ab);
        // Y still holds dQ^T of the previous step (of the previous item) until the read-out warps have it
        if (q_iter > 0) mbar_wait(&dq_read, (q_iter - 1u) & 1u, ab);
        tc_fence_after();
        issue_kk(TM_Y, v_base, do_base + st * TILE_BYTES, 1u, st);
        umma_commit(&dpt_full);
        if (n_steps == 1) umma_commit(&v_free);   // no other product of this item reads V
        ++n_items;
      }
      for (int s = 0; s < n_steps; ++s, ++q_iter) {
        const uint32_t st = q_iter & 1u;
        const uint32_t nx = q_iter + 1u, st_n = nx & 1u, ph_n = (nx >> 1) & 1u;
        const bool has_next = (s + 1 < n_steps);
        mbar_wait(&p_ready, q_iter & 1u, ab);
        // dV / dK start over (accumulate = 0): the previous item's must have been read out
        if (s == 0 && n_items > 1) mbar_wait(&acc_read, n_items & 1u, ab);
        tc_fence_after();
        issue_dv(do_base + st * TILE_BYTES, s > 0);
        umma_commit(&dv_done);       // the dO tile of this stage may now be overwritten with dS^T
        if (has_next) {
          mbar_wait(&q_full[st_n], ph_n, ab);
          tc_fence_after();
          issue_kk(TM_X, k_base, q_base + st_n * TILE_BYTES, 0u, st_n);
          umma_commit(&st_full);
        }
        mbar_wait(&ds_ready, q_iter & 1u, ab);
        tc_fence_after();
        // dK first: it is the last reader of the Q stage, whose refill (two steps ahead) is what the next
        // but one S^T waits for; the read-out warps have slack for the 512 clocks dQ^T comes later
        issue_dk(do_base + st * TILE_BYTES, q_base + st * TILE_BYTES, s > 0);
        umma_commit(&q_empty[st]);   // the Q tile of this stage may be refilled
        issue_dq(do_base + st * TILE_BYTES);
        umma_commit(&dq_full);
        umma_commit(&do_empty[st]);  // dS^T (in the dO stage) has been consumed too
        // every product that reads K has been issued: the next item's K tile may come in
        if (!has_next) umma_commit(&k_free);
        if (has_next) {
          mbar_wait(&do_full[st_n], ph_n, ab);
          mbar_wait(&dq_read, q_iter & 1u, ab);
          tc_fence_after();
          issue_kk(TM_Y, v_base, do_base + st_n * TILE_BYTES, 1u, st_n);
          umma_commit(&dpt_full);
          if (s + 2 == n_steps) umma_commit(&v_free);   // that was the item's last dP^T: V may be replaced
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

// dq[token of row r] = bf16(scale * dq_acc[r]) for the rows the selection lists (every row when
// q_idx is null). One warp per row, four floats per lane and head.
__global__ void __launch_bounds__(256)
    bwd_dq_finish_kernel(const float* __restrict__ dq_acc, const int64_t* __restrict__ q_idx,
                         const int32_t* __restrict__ sq_ptr, __nv_bfloat16* __restrict__ dq, int n_tokens, int hq,
                         float scale, int* status) {
  const int sq = q_idx ? min(max(__ldg(sq_ptr), 0), n_tokens) : n_tokens;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < sq; r += warps) {
    long long tok = q_idx ? __ldg(q_idx + r) : (long long)r;
    if (tok < 0 || tok >= n_tokens) {
      if (lane == 0 && status) atomicCAS(status, 0, (int)DEV_BAD_INDEX);
      continue;
    }
    const float4* src = reinterpret_cast<const float4*>(dq_acc + (size_t)r * hq * HEAD_DIM) + lane;
    uint2* dst = reinterpret_cast<uint2*>(dq + (size_t)tok * hq * HEAD_DIM) + lane;
    for (int h = 0; h < hq; ++h) {
      const float4 v = __ldcs(src + h * 32);
      dst[h * 32] = make_uint2(pack_bf16x2(v.x * scale, v.y * scale), pack_bf16x2(v.z * scale, v.w * scale));
    }
  }
}

int launch_attn_bwd_fused(const CUtensorMap& tm_q, const CUtensorMap& tm_do, const CUtensorMap& tm_k,
                          const CUtensorMap& tm_v, const BwdArgs& a, float* dq_acc, const __nv_bfloat16* vec_split,
                          const int32_t* sq_ptr, cudaStream_t stream) {
  static thread_local int attr_set_dev = -1;
  int dev = 0;
  LOGO_CHECK_CUDA(cudaGetDevice(&dev));
  if (attr_set_dev != dev) {
    LOGO_CHECK_CUDA(
        cudaFuncSetAttribute(attn_bwd_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FusedSmem::BYTES));
    attr_set_dev = dev;
  }
  const int sms = sm_count();
  LOGO_CHECK_CUDA(cudaMemsetAsync(a.counter_dkv, 0, sizeof(int), stream));
  prof_begin(PROF_BWD_FUSED, stream);
  CUtensorMap tm_dq;
  const uint64_t acc_rows = a.q_idx ? (uint64_t)a.cap : (uint64_t)a.n_tokens;
  // one reduction = 16 query rows x 32 head-dimension columns (a 128-byte piece of each row)
  int rc = make_tmap_2d_f32(&tm_dq, dq_acc, (uint64_t)a.hq * HEAD_DIM, acc_rows, (uint64_t)a.hq * HEAD_DIM * 4, 32, 16);
  if (rc) return rc;
  CUtensorMap tm_vec;   // [rows][hq][16] bf16: the split -lse / c and -delta of every (row, head)
  rc = make_tmap_2d_bf16(&tm_vec, vec_split, (uint64_t)a.hq * 16, acc_rows, (uint64_t)a.hq * 32, 16, TILE, 32);
  if (rc) return rc;
  attn_bwd_fused_kernel<<<sms, FUSED_THREADS, FusedSmem::BYTES, stream>>>(tm_q, tm_do, tm_k, tm_v, tm_dq, tm_vec, a);
  prof_end(PROF_BWD_FUSED, stream);
  LOGO_CHECK_CUDA(cudaGetLastError());
  prof_begin(PROF_BWD_FINISH, stream);
  bwd_dq_finish_kernel<<<sms * 8, 256, 0, stream>>>(dq_acc, a.q_idx, sq_ptr, a.dq, a.n_tokens, a.hq, a.scale, a.status);
  prof_end(PROF_BWD_FINISH, stream);
  LOGO_CHECK_CUDA(cudaGetLastError());
  return LOGO_OK;
}

}  // namespace logo
