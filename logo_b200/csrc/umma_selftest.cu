// Single-CTA tcgen05 matrix multiply that pins the operand encodings used by the
// attention kernels: K-major and MN-major shared-memory descriptors with 128-byte
// swizzle, an A operand staged in tensor memory, thread-written swizzled shared
// memory, and the 32x32b tensor-memory load shape.
#include "host_common.cuh"
#include "ptx.cuh"

namespace logo {

struct SelftestArgs {
  int mode;
  int flags;
  uint32_t lbo;
  uint32_t sbo;
  uint32_t kstep;
};

// 128 threads. Shared memory (dynamic, 1024-byte aligned):
//   [0, 32K)   A: two [128][64] bf16 blocks (columns 0-63, 64-127), 128B-swizzled
//   [32K, 64K) B: same shape
//   [64K, 68K) / [68K, 72K): mode 4 only, columns 0-15 of A / of B as [128][16] tiles with the 32-byte swizzle
__global__ void __launch_bounds__(128, 1)
    umma_selftest_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                         const __grid_constant__ CUtensorMap tm_a32, const __grid_constant__ CUtensorMap tm_b32,
                         const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                         float* __restrict__ c, int* status, SelftestArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + 32768;
  uint8_t* sA32 = smem + 65536;
  uint8_t* sB32 = smem + 65536 + 4096;
  __shared__ uint64_t bar_load;
  __shared__ uint64_t bar_mma;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  const int warp = uniform_warp_idx();
  // flags bits 8-23: limit of every wait of this launch in microseconds (0: the library default)
  const uint64_t limit_us = (uint64_t)((args.flags >> 8) & 0xffff);
  AbortState ab{&abort_flag, status, limit_us * 1000ull};

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&bar_load, 1);
    mbar_init(&bar_mma, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t tmem_d = tmem_base;        // accumulator: columns [0,128)
  const uint32_t tmem_p = tmem_base + 128;  // A operand staged in TMEM: columns [128,192)

  const bool manual_a = (args.flags & 1) != 0;
  const bool manual_b = (args.flags & 4) != 0;
  const bool never_armed = (args.flags & 8) != 0;   // nothing ever completes bar_load: its wait must run out
  const bool a_in_smem = (args.mode != 2);

  // ---- stage operands ----
  if (tid == 0 && !never_armed) {
    uint32_t bytes = 0;
    if (!manual_b) bytes += 32768;
    if (a_in_smem && !manual_a) bytes += 32768;
    if (args.mode == 4) bytes += 8192;
    if (args.mode == 5) bytes += 4096;
    if (bytes) {
      mbar_arrive_expect_tx(&bar_load, bytes);
    } else {
      mbar_arrive(&bar_load);
    }
    if (!manual_b) {
      tma_load_2d(sB, &tm_b, &bar_load, 0, 0);
      tma_load_2d(sB + 16384, &tm_b, &bar_load, 64, 0);
    }
    if (a_in_smem && !manual_a) {
      tma_load_2d(sA, &tm_a, &bar_load, 0, 0);
      tma_load_2d(sA + 16384, &tm_a, &bar_load, 64, 0);
    }
    if (args.mode == 4) {
      tma_load_2d(sA32, &tm_a32, &bar_load, 0, 0);
      tma_load_2d(sB32, &tm_b32, &bar_load, 0, 0);
    }
    if (args.mode == 5) tma_load_2d(sB32, &tm_b32, &bar_load, 0, 0);
  }
  if (args.mode == 5 && tid < 16) {
    // two core matrices (8 rows x 16 bytes each) whose rows all hold a[0][0:8] / a[0][8:16]: with a zero
    // distance between 8-row groups the 256 bytes stand for a [128][16] tile of identical rows
    const uint4* src = reinterpret_cast<const uint4*>(a);
    reinterpret_cast<uint4*>(sA32)[tid] = src[tid >> 3];
    fence_proxy_async_smem();
  }
  // thread-written operands: each thread copies its own row, 16 bytes at a time, into the swizzled layout
  auto copy_row = [&](const __nv_bfloat16* src_mat, uint8_t* dst) {
    const uint4* src = reinterpret_cast<const uint4*>(src_mat + (size_t)tid * 128);
#pragma unroll
    for (int ch = 0; ch < 16; ++ch) {
      const uint4 v = src[ch];
      const int blk = ch >> 3;
      const uint32_t off = sw128_offset((uint32_t)tid, (uint32_t)(ch & 7) * 8);
      *reinterpret_cast<uint4*>(dst + blk * 16384 + off) = v;
    }
  };
  if (a_in_smem && manual_a) copy_row(a, sA);
  if (manual_b) copy_row(b, sB);
  if ((a_in_smem && manual_a) || manual_b) fence_proxy_async_smem();
  if (!a_in_smem) {
    // row `tid` of A -> TMEM lane tid, two bf16 per 32-bit column
    const uint32_t* src = reinterpret_cast<const uint32_t*>(a + (size_t)tid * 128);
    const uint32_t lane_base = (uint32_t)(warp * 32);
#pragma unroll
    for (int ch = 0; ch < 2; ++ch) {
      uint32_t r[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = src[ch * 32 + i];
      tmem_st32(tmem_addr(tmem_p, lane_base, ch * 32), r);
    }
    tmem_st_wait();
  }
  tc_fence_before();
  __syncthreads();

  // ---- MMA: warp 0 walks the loop, an elected lane issues ----
  if (warp == 0) {
    tc_fence_after();
    const bool loaded = mbar_wait(&bar_load, 0, ab);
    const uint32_t a_base = smem_u32(sA);
    const uint32_t b_base = smem_u32(sB);
    if (loaded) {
      if (args.mode == 0 || args.mode == 4 || args.mode == 5) {
        const uint32_t idesc = umma_idesc_bf16(128, 128, 0, 0);
#pragma unroll 1
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * 16384u + (uint32_t)(kk & 3) * 32u;
          umma_ss(tmem_d, umma_desc_sw128(a_base + off, args.lbo, 1024), umma_desc_sw128(b_base + off, args.lbo, 1024),
                  idesc, kk > 0);
        }
        // mode 4: a ninth k-step from the 32-byte-swizzled tiles: D += A[:, 0:16] B[:, 0:16]^T
        if (args.mode == 4) umma_ss(tmem_d, umma_desc_sw32(smem_u32(sA32)), umma_desc_sw32(smem_u32(sB32)), idesc, true);
        // mode 5: the ninth k-step's A operand is the 256-byte tile of identical rows, without swizzle
        // (lbo / sbo of the call describe it): D += ones x (a[0][0:16] . B[:, 0:16]^T)
        if (args.mode == 5)
          umma_ss(tmem_d, umma_desc_noswizzle(smem_u32(sA32), args.kstep, args.sbo), umma_desc_sw32(smem_u32(sB32)), idesc, true);
      } else if (args.mode == 1) {
        const uint32_t idesc = umma_idesc_bf16(128, 128, 0, 1);
#pragma unroll 1
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t aoff = (uint32_t)(kk >> 2) * 16384u + (uint32_t)(kk & 3) * 32u;
          umma_ss(tmem_d, umma_desc_sw128(a_base + aoff, 0, 1024),
                  umma_desc_sw128(b_base + (uint32_t)kk * args.kstep, args.lbo, args.sbo), idesc, kk > 0);
        }
      } else if (args.mode == 2) {
        const uint32_t idesc = umma_idesc_bf16(128, 128, 0, 1);
#pragma unroll 1
        for (int kk = 0; kk < 8; ++kk) {
          umma_ts(tmem_d, tmem_p + (uint32_t)kk * 8u, umma_desc_sw128(b_base + (uint32_t)kk * args.kstep, args.lbo, args.sbo),
                  idesc, kk > 0);
        }
      } else {
        // both operands MN-major: rows of the stored tiles are the reduction index
        const uint32_t idesc = umma_idesc_bf16(128, 128, 1, 1);
#pragma unroll 1
        for (int kk = 0; kk < 8; ++kk) {
          umma_ss(tmem_d, umma_desc_sw128(a_base + (uint32_t)kk * args.kstep, args.lbo, args.sbo),
                  umma_desc_sw128(b_base + (uint32_t)kk * args.kstep, args.lbo, args.sbo), idesc, kk > 0);
        }
      }
      umma_commit(&bar_mma);
    }
  }
  __syncwarp();

  // ---- read the accumulator back ----
  const bool ok = mbar_wait(&bar_mma, 0, ab);
  tc_fence_after();
  if (ok) {
    const uint32_t lane_base = (uint32_t)(warp * 32);
#pragma unroll 1
    for (int ch = 0; ch < 4; ++ch) {
      uint32_t r[32];
      tmem_ld32(tmem_addr(tmem_d, lane_base, ch * 32), r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) c[(size_t)tid * 128 + ch * 32 + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 256);
}

}  // namespace logo

extern "C" int logo_umma_selftest(int mode, int flags, const void* a, const void* b, float* c, uint32_t lbo_bytes,
                                  uint32_t sbo_bytes, uint32_t kstep_bytes, int32_t* status, logo_stream_t stream) {
  using namespace logo;
  LOGO_REQUIRE(mode >= 0 && mode <= 5, LOGO_ERR_INVALID, "selftest mode must be 0 .. 5");
  LOGO_REQUIRE(a && b && c, LOGO_ERR_INVALID, "selftest operands must not be NULL");
  CUtensorMap tm_a, tm_b;
  int rc = make_tmap_2d_bf16(&tm_a, a, 128, 128, 256, 64, 128);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tm_b, b, 128, 128, 256, 64, 128);
  if (rc) return rc;
  CUtensorMap tm_a32, tm_b32;
  rc = make_tmap_2d_bf16(&tm_a32, a, 128, 128, 256, 16, 128, 32);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tm_b32, b, 128, 128, 256, 16, 128, 32);
  if (rc) return rc;
  const int smem_bytes = 65536 + 8192 + 1024;
  LOGO_CHECK_CUDA(cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
  SelftestArgs args{mode, flags, lbo_bytes, sbo_bytes, kstep_bytes};
  umma_selftest_kernel<<<1, 128, smem_bytes, (cudaStream_t)stream>>>(tm_a, tm_b, tm_a32, tm_b32, (const __nv_bfloat16*)a,
                                                                    (const __nv_bfloat16*)b, c, status, args);
  LOGO_CHECK_CUDA(cudaGetLastError());
  return LOGO_OK;
}
