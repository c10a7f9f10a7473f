// Thin inline-PTX wrappers for the sm_100a features the attention kernels use:
// mbarrier, TMA tiled loads, tcgen05 (TMEM allocation, MMA, commit, ld/st) and
// the UMMA shared-memory / instruction descriptors.
//
// Every wait in this file is bounded: a wait that does not complete within
// LOGO_WAIT_TIMEOUT_NS raises a CTA-wide abort flag (in shared memory) and a
// status word (in global memory); all later waits of the CTA then fall through
// so that the kernel drains, frees its TMEM and returns instead of hanging.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace logo {

#ifndef LOGO_WAIT_TIMEOUT_NS
#define LOGO_WAIT_TIMEOUT_NS 1000000000ull  // 1 s
#endif

// ---------------------------------------------------------------------------
// status word values written by kernels (0 = ok)
// ---------------------------------------------------------------------------
enum DeviceStatus : int {
  DEV_OK = 0,
  DEV_WAIT_TIMEOUT = 1,   // a bounded mbarrier wait expired
  DEV_BAD_INDEX = 2,      // an index read from q_idx / cu_seqlens was out of range
  DEV_SCAN_TIMEOUT = 3,   // decoupled look-back spin expired
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Generic-proxy writes to shared memory -> visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

// One try_wait with a suspend-time hint: the thread sleeps in hardware until the phase completes
// or roughly `LOGO_TRYWAIT_HINT_NS` have passed, instead of burning issue slots in a poll loop.
#ifndef LOGO_TRYWAIT_HINT_NS
#define LOGO_TRYWAIT_HINT_NS 1000000u  // 1 ms
#endif

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(LOGO_TRYWAIT_HINT_NS)
      : "memory");
  return ok != 0;
}

// One arrival for the whole warp: every lane's preceding work is ordered before it by the warp
// barrier. A barrier that 128-512 threads arrive on individually costs one shared-memory atomic per
// thread on the hand-off path; with this form its count is the number of WARPS.
__device__ __forceinline__ void mbar_arrive_warp(uint64_t* bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}

// Per-CTA abort state, shared by all waits of a kernel.
struct AbortState {
  volatile int* smem_abort;  // CTA-wide flag in shared memory
  int* gmem_status;          // status word in global memory (may be null)
  uint64_t timeout_ns;       // limit of one wait; 0 = LOGO_WAIT_TIMEOUT_NS
};

// Bounded wait. Returns false if the CTA is (or becomes) aborted. The clock is only consulted
// after a number of failed (each up to LOGO_TRYWAIT_HINT_NS long) attempts.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const AbortState& ab) {
  if (mbar_try_wait(bar, parity)) return true;
  // failed attempts between two looks at the clock: few when each attempt sleeps, many when it polls
  constexpr uint32_t kCheckMask = (LOGO_TRYWAIT_HINT_NS >= 100000u) ? 15u : 8191u;
  uint64_t t0 = 0;
#pragma unroll 1
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & kCheckMask) == 0u) {
      if (*ab.smem_abort) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > (ab.timeout_ns ? ab.timeout_ns : LOGO_WAIT_TIMEOUT_NS)) {
        *ab.smem_abort = 1;
        if (ab.gmem_status) atomicCAS(ab.gmem_status, 0, (int)DEV_WAIT_TIMEOUT);
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// TMA: tiled 2-D load global -> shared, completion on an mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Bulk reduction shared -> global through a tensor map: global[box at (x, y)] += shared tile (the element
// type and the box come from the map). Completion is tracked per bulk group of the issuing thread.
__device__ __forceinline__ void tma_reduce_add_2d(const void* tmap, const void* smem_src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(tmap), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// every bulk group of this thread has finished READING its shared-memory source
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all but the newest bulk group of this thread have finished reading their shared-memory source
__device__ __forceinline__ void bulk_wait_read_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// ... all but the two newest
__device__ __forceinline__ void bulk_wait_read_but_two() { asm volatile("cp.async.bulk.wait_group.read 2;" ::: "memory"); }
// every bulk group of this thread has completed (its global writes are performed)
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05: TMEM allocation
// ---------------------------------------------------------------------------
// Executed by one full warp. ncols: power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------
// tcgen05: descriptors
// ---------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (sm_100).
//   bits [0,14)  start address >> 4
//   bits [16,30) leading-dimension byte offset >> 4
//   bits [32,46) stride-dimension byte offset >> 4
//   bits [46,48) version = 1
//   bits [61,64) layout type, 2 = 128-byte swizzle
// K-major operand  (rows = M/N, 64 bf16 of K per 128-byte row): SBO = 1024 (8-row group), LBO unused.
// MN-major operand (rows = K, 64 bf16 of M/N per 128-byte row): SBO = 1024 (8 K-rows),
//                   LBO = byte distance between consecutive 64-element M/N blocks.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// The same for a K-major operand of ONE k-step (16 bf16 = 32 bytes per row) stored with the 32-byte
// swizzle (rows of 32 bytes, 8-row groups of 256 bytes: SBO = 256; layout type 6). Written by TMA
// with CU_TENSOR_MAP_SWIZZLE_32B, or by threads when both 16-byte halves of a row hold the same
// values (the swizzle only exchanges the halves).
__device__ __forceinline__ uint64_t umma_desc_sw32(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(256 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)6 << 61;
  return d;
}

// The same without swizzle (layout type 0): 8-row x 16-byte core matrices of 128 contiguous bytes; for a
// K-major operand `lbo_bytes` is the distance between the core matrices of consecutive 16-byte K chunks
// and `sbo_bytes` the distance between consecutive 8-row groups.
__device__ __forceinline__ uint64_t umma_desc_noswizzle(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

// Instruction descriptor for kind::f16 with bf16 inputs and fp32 accumulation.
//   a_major / b_major: 0 = K-major, 1 = MN-major.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N, int a_major, int b_major) {
  return (1u << 4)                       // D format fp32
         | (1u << 7)                     // A format bf16
         | (1u << 10)                    // B format bf16
         | ((uint32_t)a_major << 15)     //
         | ((uint32_t)b_major << 16)     //
         | ((uint32_t)(N >> 3) << 17)    //
         | ((uint32_t)(M >> 4) << 24);
}

// True in exactly one lane. Must be called by all 32 lanes of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// Warp index as a value the compiler knows to be the same in every lane.
__device__ __forceinline__ int uniform_warp_idx() { return __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0); }

// ---------------------------------------------------------------------------
// tcgen05: MMA, commit
// ---------------------------------------------------------------------------
// The three wrappers below are WARP-COLLECTIVE: call them from all 32 lanes of a converged warp
// with warp-uniform arguments; the lane picked by elect.sync issues the instruction. The compiler
// recognises the elected region as single-threaded and feeds the descriptors through uniform
// registers: measured 64 clocks per 128x128x16 product (the tensor pipe's own rate), against ~110
// when a lone lane of a diverged warp (`if (lane == 0)`) issues.

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  if (elect_one()) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
  __syncwarp();
}

// D[tmem] (+)= A[tmem] * B[smem]; A must be K-major.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  if (elect_one()) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
  __syncwarp();
}

// A whole 128 x N x 128 tile product (eight k-steps of 16) issued inside ONE elected region: the
// operand descriptors advance by constants (the start-address field counts 16-byte units and cannot
// carry out of its 14 bits for addresses inside the 228 KB of shared memory), so the issuing lane
// spends a handful of uniform-register adds per instruction instead of rebuilding descriptors.
//   A_TMEM: A comes from tensor memory (8 columns per k-step), else from K-major 128B-swizzled
//           shared memory (two [128][64] blocks: 32 bytes per k-step, 16 KB between the blocks);
//   B_MN  : B is MN-major ([k][n] rows as they lie in memory, 2 KB per k-step), else K-major.
//   A_SPLIT (with A_TMEM): 0: A is 64 contiguous columns; 2: two halves of 32 columns, the second
//           64 columns after the first; 4: four quarters of 16 columns, 32 columns apart. With 2 / 4
//           every part of A lies inside the fp32 columns it was computed from, so the warps that
//           produce the parts never touch each other's columns.
//   K_BEGIN, K_END: the k-steps to issue (default all eight); `accumulate_first` applies to K_BEGIN.
//   A_MN  : A comes from shared memory MN-major ([k][m] rows as they lie in memory, 2 KB per k-step).
template <bool A_TMEM, bool B_MN, int A_SPLIT = 0, int K_BEGIN = 0, int K_END = 8, bool A_MN = false>
__device__ __forceinline__ void umma_tile_k128(uint32_t d_tmem, uint64_t a0, uint64_t b0, uint32_t idesc,
                                               uint32_t accumulate_first) {
  if (elect_one()) {
#pragma unroll
    for (int kk = K_BEGIN; kk < K_END; ++kk) {
      const uint32_t kmaj = (uint32_t)(kk >> 2) * 1024u + (uint32_t)(kk & 3) * 2u;   // K-major advance, 16 B units
      const uint64_t b = b0 + (B_MN ? (uint64_t)kk * 128u : (uint64_t)kmaj);
      const uint32_t acc = kk > K_BEGIN ? 1u : accumulate_first;
      if (A_TMEM) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
            "}\n"
            :
            : "r"(d_tmem), "r"((uint32_t)a0 + (A_SPLIT == 4 ? (uint32_t)(kk >> 1) * 32u + (uint32_t)(kk & 1) * 8u
                                                : (uint32_t)kk * 8u + ((A_SPLIT == 2 && kk >= 4) ? 32u : 0u))), "l"(b), "r"(idesc),
              "r"(acc)
            : "memory");
      } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
            "}\n"
            :
            : "r"(d_tmem), "l"(a0 + (A_MN ? (uint64_t)kk * 128u : (uint64_t)kmaj)), "l"(b), "r"(idesc), "r"(acc)
            : "memory");
      }
    }
  }
  __syncwarp();
}

// Make `bar` track completion of all tcgen05 async ops issued so far by the elected lane.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  if (elect_one()) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
  }
  __syncwarp();
}

// ---------------------------------------------------------------------------
// tcgen05: TMEM <-> registers. Shape 32x32b: thread i of the warp owns TMEM lane
// (warp_id % 4) * 32 + i and receives `N` consecutive 32-bit columns.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
        "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// TMEM address helpers: lane in bits [16,32), column in bits [0,16).
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}

// ---------------------------------------------------------------------------
// small math helpers
// ---------------------------------------------------------------------------
// 4-byte asynchronous copy global -> shared (no destination register, hence no scoreboard wait
// anywhere near the issue point); completion with cp_async_wait_all().
__device__ __forceinline__ void cp_async_4(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// barrier among `nthreads` threads (a multiple of 32) that name the same id (1..15; 0 is __syncthreads)
__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// max of three floats in one instruction (3-input max.f32, sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  // cvt.rn.bf16x2.f32 d, a, b : a -> upper half, b -> lower half
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Byte offset of element (row, col) of a [rows][64] bf16 block stored with the
// 128-byte swizzle that TMA SWIZZLE_128B and the UMMA 128B layouts share:
// the 16-byte chunk index is XOR-ed with (row % 8). The block base must be
// 1024-byte aligned.
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t col_elem) {
  const uint32_t chunk = col_elem >> 3;  // 8 bf16 per 16-byte chunk
  return row * 128u + (((chunk ^ (row & 7u)) << 4) | ((col_elem & 7u) << 1));
}

}  // namespace logo
