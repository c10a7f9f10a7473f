// Definitions shared by the forward and backward attention kernels: work-item decoding
// (which sequence / which compacted query rows / which head a CTA works on) and the
// argument block.
#pragma once

#include <stdint.h>

#include "ptx.cuh"

namespace logo {

constexpr int HEAD_DIM = 128;   // the only head size the kernels implement
constexpr int TILE = 128;       // rows of one query tile / keys of one key tile
constexpr uint32_t BLK_BYTES = 16384;   // one [128][64] bf16 block, 128-byte swizzled
constexpr uint32_t TILE_BYTES = 32768;  // one [128][128] bf16 tile = two blocks

struct AttnArgs {
  // activations, bf16, packed tokens
  const __nv_bfloat16* q;    // [n_tokens, hq, 128]
  const __nv_bfloat16* k;    // [n_tokens, h, 128]   (device pointer; the kernels read K/V through TMA)
  const __nv_bfloat16* v;    // [n_tokens, h, 128]
  __nv_bfloat16* o;          // [n_tokens, hq, 128]
  float* lse;                // [n_tokens, hq] base-2 log-sum-exp of the scaled scores
  // backward only
  const __nv_bfloat16* d_o;  // [n_tokens, hq, 128]
  float* delta;              // [n_tokens, hq]  sum_d o * do
  __nv_bfloat16* dq;         // [n_tokens, hq, 128]
  __nv_bfloat16* dk;         // [n_tokens, h, 128]
  __nv_bfloat16* dv;         // [n_tokens, h, 128]
  // selection metadata (q_idx == nullptr: every row is selected, identity mapping)
  const int64_t* q_idx;      // [Sq] ascending token index of each compacted row
  const int32_t* pos_ids;    // [Sq] position inside its sequence
  const int32_t* cu_q;       // [n_seq + 1] compacted-row prefix per sequence
  const int32_t* cu_k;       // [n_seq + 1] token prefix per sequence
  const int32_t* tile_off;   // [n_seq + 1] prefix of work tiles per sequence (unit depends on the kernel)
  const int32_t* n_tiles;    // [1] total number of work tiles
  int* work_counter;         // [1] zeroed before the launch: the next unclaimed work item
  int n_seq;
  int n_tokens;
  int hq;
  int h;
  int window;                // 0: full causal; w > 0: keys [pos - w, pos]
  float scale_log2;          // softmax scale * log2(e)
  float scale;               // softmax scale
  const int32_t* zero_sq;    // forward: when set ([1] number of selected rows), two spare warps of every CTA zero
                             // the rows of `o` that the selection leaves out
  int* status;
};

// Largest s in [0, n_seq) with off[s] <= x. `off` is a non-decreasing prefix array with off[0] = 0;
// sequences without tiles (off[s] == off[s+1]) are skipped because the last candidate wins.
__device__ __forceinline__ int find_sequence(const int32_t* __restrict__ off, int n_seq, int x) {
  int lo = 0, hi = n_seq;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(off + mid) <= x) lo = mid; else hi = mid;
  }
  return lo;
}

// Work distribution. Items (tile, head) are listed heaviest-first per sequence and claimed
// dynamically from a global counter, so CTAs that drew light items simply take more of them (a
// static round-robin leaves 10-60 % of the SMs idle at the tail; sorting all items by cost instead
// balances as well but scatters concurrent CTAs over the K/V streams and costs more in L2 misses
// than it gains). One thread of the producer warp claims an item, DECODES it (sequence lookup,
// binary searches over positions: chains of dependent global loads, microseconds long) and
// publishes the decoded record through a small shared-memory ring; it does so one item ahead of
// the loads it issues, so the MMA warp and the eight element-wise warps never wait for a decode.
constexpr int ITEM_RING = 4;
constexpr int ITEM_WORDS = 20;          // ints per published record; word 0 is the item index or -1

struct ItemRing {
  volatile int* items;   // [ITEM_RING][ITEM_WORDS]
  uint64_t* full;        // [ITEM_RING] count 1
  uint64_t* empty;       // [ITEM_RING] count = number of consumer warps
};

__device__ __forceinline__ void ring_init(const ItemRing& r, int consumer_warps) {
  for (int i = 0; i < ITEM_RING; ++i) {
    mbar_init(&r.full[i], 1);
    mbar_init(&r.empty[i], consumer_warps);
  }
}

// Producer (one thread): next unclaimed item, or -1 when the list is exhausted / the CTA aborted.
__device__ __forceinline__ long long ring_claim(int* counter, long long total, const AbortState& ab) {
  const long long w = (long long)atomicAdd(counter, 1);
  return (w >= total || *ab.smem_abort) ? -1 : w;
}

// Producer (one thread): publish record number `n` of this CTA (w < 0: the end marker).
template <class Item>
__device__ __forceinline__ void ring_publish(const ItemRing& r, uint32_t n, long long w, const Item& item,
                                             const AbortState& ab) {
  static_assert(sizeof(Item) <= (ITEM_WORDS - 1) * sizeof(int), "item record too large for the ring");
  const uint32_t slot = n % ITEM_RING, ph = (n / ITEM_RING) & 1u;
  mbar_wait(&r.empty[slot], ph ^ 1u, ab);
  volatile int* dst = r.items + slot * ITEM_WORDS;
  dst[0] = (int)w;
  if (w >= 0) {
    const int* src = reinterpret_cast<const int*>(&item);
#pragma unroll
    for (int i = 0; i < (int)(sizeof(Item) / sizeof(int)); ++i) dst[1 + i] = src[i];
  }
  mbar_arrive(&r.full[slot]);
}

// Consumer (every thread of the role): record number `n` of this CTA; returns the item index or -1.
template <class Item>
__device__ __forceinline__ long long ring_pop(const ItemRing& r, uint32_t n, Item& item, const AbortState& ab) {
  const uint32_t slot = n % ITEM_RING, ph = (n / ITEM_RING) & 1u;
  if (!mbar_wait(&r.full[slot], ph, ab)) return -1;
  const volatile int* src = r.items + slot * ITEM_WORDS;
  const int w = src[0];
  if (w >= 0) {
    int* dst = reinterpret_cast<int*>(&item);
#pragma unroll
    for (int i = 0; i < (int)(sizeof(Item) / sizeof(int)); ++i) dst[i] = src[1 + i];
  }
  return (long long)w;
}

// Consumer: the calling WARP is done with record `n` (call from all lanes; one arrives).
__device__ __forceinline__ void ring_release(const ItemRing& r, uint32_t n) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(&r.empty[n % ITEM_RING]);
}

// Epilogue helper. After a 32x32b tensor-memory load every lane owns one ROW of the tile; storing
// it directly makes each store instruction touch 32 different lines (the epilogue of one tile then
// costs thousands of cycles of address processing). This routine sends a [32 rows][32 columns] bf16
// patch (16 packed words per lane) through a warp-private 2 KB shared-memory buffer and writes it
// back out with 4 lanes per row: one instruction covers 8 rows x 64 contiguous bytes. Both
// shared-memory passes are free of bank conflicts (16-byte chunks XOR-swizzled by row / 2).
//   stage      : 2 KB, 16-byte aligned, private to the calling warp
//   base       : tensor the rows live in
//   my_row_off : element offset of (this lane's row, first column of the patch), or -1 to skip the row
__device__ __forceinline__ void store_patch_32x32(uint8_t* stage, const uint32_t* pk, __nv_bfloat16* base,
                                                  long long my_row_off, int lane) {
  uint8_t* wr = stage + lane * 64;
#pragma unroll
  for (int c = 0; c < 4; ++c)
    *reinterpret_cast<uint4*>(wr + (((c ^ (lane >> 1)) & 3) << 4)) =
        make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
  __syncwarp();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int r = 8 * k + (lane >> 2), c = lane & 3;
    const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 64 + (((c ^ (r >> 1)) & 3) << 4));
    const long long off = __shfl_sync(0xffffffffu, my_row_off, r);
    if (off >= 0) *reinterpret_cast<uint4*>(base + off + c * 8) = v;
  }
  __syncwarp();
}

// Position of compacted row `r` (relative to the start of the sequence's compacted rows).
__device__ __forceinline__ int row_position(const AttnArgs& a, int bos_q, int r) {
  return a.q_idx ? __ldg(a.pos_ids + bos_q + r) : r;
}

// Token index of compacted row `r` of the sequence.
__device__ __forceinline__ long long row_token(const AttnArgs& a, int bos_q, int bos_k, int r) {
  return a.q_idx ? (long long)__ldg(a.q_idx + bos_q + r) : (long long)(bos_k + r);
}

}  // namespace logo
