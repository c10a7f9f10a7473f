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
__global__ void __launch_bounds__(128, 1)
    umma_selftest_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                         const __nv_bfloat16* __restrict__ a, float* __restrict__ c, int* status,
                         SelftestArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + 32768;
  __shared__ uint64_t bar_load;
  __shared__ uint64_t bar_mma;
  __shared__ uint64_t bar_scratch;   // timing mode, bit 3: receives a commit after every tile product
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  const int warp = uniform_warp_idx();
  AbortState ab{&abort_flag, status};

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&bar_load, 1);
    mbar_init(&bar_mma, 1);
    mbar_init(&bar_scratch, 1u << 20);
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
  const bool a_in_smem = (args.mode != 2);

  // ---- stage operands ----
  if (tid == 0) {
    uint32_t bytes = 32768;  // B
    if (a_in_smem && !manual_a) bytes += 32768;
    mbar_arrive_expect_tx(&bar_load, bytes);
    tma_load_2d(sB, &tm_b, &bar_load, 0, 0);
    tma_load_2d(sB + 16384, &tm_b, &bar_load, 64, 0);
    if (a_in_smem && !manual_a) {
      tma_load_2d(sA, &tm_a, &bar_load, 0, 0);
      tma_load_2d(sA + 16384, &tm_a, &bar_load, 64, 0);
    }
  }
  if (a_in_smem && manual_a) {
    // each thread copies its own row, 16 bytes at a time, into the swizzled layout
    const uint4* src = reinterpret_cast<const uint4*>(a + (size_t)tid * 128);
#pragma unroll
    for (int ch = 0; ch < 16; ++ch) {
      const uint4 v = src[ch];
      const int blk = ch >> 3;
      const uint32_t off = sw128_offset((uint32_t)tid, (uint32_t)(ch & 7) * 8);
      *reinterpret_cast<uint4*>(sA + blk * 16384 + off) = v;
    }
    fence_proxy_async_smem();
  }
  if (!a_in_smem) {
    // row `tid` of A -> TMEM lane tid, two bf16 per 32-bit column
    const uint32_t* src = reinterpret_cast<const uint32_t*>(a + (size_t)tid * 128);
    const uint32_t lane_base = (uint32_t)(warp * 32);
#pragma unroll
    for (int ch = 0; ch < 2; ++ch) {
      uint32_t r[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        uint32_t w = src[ch * 32 + i];
        if (args.flags & 2) w = (w >> 16) | (w << 16);
        r[i] = w;
      }
      tmem_st32(tmem_addr(tmem_p, lane_base, ch * 32), r);
    }
    tmem_st_wait();
  }
  tc_fence_before();
  __syncthreads();

  // ---- MMA: warp 0 walks the loop, an elected lane issues ----
  if (warp == 0) {
    tc_fence_after();
    mbar_wait(&bar_load, 0, ab);
    const uint32_t a_base = smem_u32(sA);
    const uint32_t b_base = smem_u32(sB);
    const int repeat = (args.flags >> 8) & 0xffff;   // bits 8-23   // timing mode: issue the tile product `repeat` extra times
    const int n_cols = ((args.flags >> 4) & 1) ? 64 : 128;
    if (repeat > 0) {
      // timing-mode options: bit 5 alternates between two accumulators from one tile product to the
      // next (mode 0 only: the second one overlaps the staged A operand of mode 2), bit 6 makes the
      // first k-step of every tile product overwrite instead of accumulate
      const bool alt_acc = (args.flags >> 5) & 1, overwrite = (args.flags >> 6) & 1;
      const bool batched = (args.flags >> 7) & 1;   // bit 7: one elected region per tile product
      const bool commit_each = (args.flags >> 3) & 1;
      const uint64_t g0 = globaltimer_ns();
      const long long t0 = clock64();
      for (int rep = 0; rep < repeat; ++rep) {
        if (batched) {
          if (args.mode == 0)
            umma_tile_k128<false, false>(tmem_d, umma_desc_sw128(a_base, 0, 1024), umma_desc_sw128(b_base, 0, 1024),
                                         umma_idesc_bf16(128, n_cols, 0, 0), overwrite ? 0 : 1);
          else if (args.mode == 1)
            umma_tile_k128<false, true>(tmem_d, umma_desc_sw128(a_base, 0, 1024),
                                        umma_desc_sw128(b_base, args.lbo, args.sbo), umma_idesc_bf16(128, n_cols, 0, 1),
                                        overwrite ? 0 : 1);
          else
            umma_tile_k128<true, true>(tmem_d, tmem_p, umma_desc_sw128(b_base, args.lbo, args.sbo),
                                       umma_idesc_bf16(128, n_cols, 0, 1), overwrite ? 0 : 1);
          if (commit_each) umma_commit(&bar_scratch);
        } else if (args.mode == 0) {
          const uint32_t idesc = umma_idesc_bf16(128, n_cols, 0, 0);
          const uint32_t d = tmem_d + ((alt_acc && (rep & 1)) ? 128u : 0u);
#pragma unroll 1
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t off = (uint32_t)(kk >> 2) * 16384u + (uint32_t)(kk & 3) * 32u;
            umma_ss(d, umma_desc_sw128(a_base + off, 0, 1024), umma_desc_sw128(b_base + off, 0, 1024), idesc,
                    (overwrite && kk == 0) ? 0 : 1);
          }
        } else if (args.mode == 1) {
          const uint32_t idesc = umma_idesc_bf16(128, n_cols, 0, 1);
#pragma unroll 1
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t aoff = (uint32_t)(kk >> 2) * 16384u + (uint32_t)(kk & 3) * 32u;
            umma_ss(tmem_d, umma_desc_sw128(a_base + aoff, 0, 1024),
                    umma_desc_sw128(b_base + (uint32_t)kk * args.kstep, args.lbo, args.sbo), idesc, 1);
          }
        } else {
          const uint32_t idesc = umma_idesc_bf16(128, n_cols, 0, 1);
#pragma unroll 1
          for (int kk = 0; kk < 8; ++kk) {
            umma_ts(tmem_d, tmem_p + (uint32_t)kk * 8u,
                    umma_desc_sw128(b_base + (uint32_t)kk * args.kstep, args.lbo, args.sbo), idesc, 1);
          }
        }
      }
      const long long t1 = clock64();
      umma_commit(&bar_mma);
      mbar_wait(&bar_mma, 0, ab);
      const long long t2 = clock64();
      const uint64_t g1 = globaltimer_ns();
      if (tid == 0 && status && blockIdx.x == 0) {
        status[1] = (int)(t1 - t0);   // clocks spent issuing
        status[2] = (int)(t2 - t0);   // clocks until the last product completed
        status[3] = (int)(g1 - g0);   // the same span in nanoseconds (gives the SM clock under this load)
      }
      __syncwarp();
      if (tid == 0) {
        mbar_init(&bar_mma, 1);       // fresh phase for the checked product below
        fence_barrier_init();
      }
      __syncwarp();
    }
    if (args.mode == 0) {
      const uint32_t idesc = umma_idesc_bf16(128, 128, 0, 0);
#pragma unroll 1
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = (uint32_t)(kk >> 2) * 16384u + (uint32_t)(kk & 3) * 32u;
        umma_ss(tmem_d, umma_desc_sw128(a_base + off, args.lbo, 1024), umma_desc_sw128(b_base + off, args.lbo, 1024),
                idesc, kk > 0);
      }
    } else if (args.mode == 1) {
      const uint32_t idesc = umma_idesc_bf16(128, 128, 0, 1);
#pragma unroll 1
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t aoff = (uint32_t)(kk >> 2) * 16384u + (uint32_t)(kk & 3) * 32u;
        umma_ss(tmem_d, umma_desc_sw128(a_base + aoff, 0, 1024),
                umma_desc_sw128(b_base + (uint32_t)kk * args.kstep, args.lbo, args.sbo), idesc, kk > 0);
      }
    } else {
      const uint32_t idesc = umma_idesc_bf16(128, 128, 0, 1);
#pragma unroll 1
      for (int kk = 0; kk < 8; ++kk) {
        umma_ts(tmem_d, tmem_p + (uint32_t)kk * 8u, umma_desc_sw128(b_base + (uint32_t)kk * args.kstep, args.lbo, args.sbo),
                idesc, kk > 0);
      }
    }
    umma_commit(&bar_mma);
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
      if (blockIdx.x == 0) {
#pragma unroll
        for (int i = 0; i < 32; ++i) c[(size_t)tid * 128 + ch * 32 + i] = __uint_as_float(r[i]);
      }
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
  LOGO_REQUIRE(mode >= 0 && mode <= 2, LOGO_ERR_INVALID, "selftest mode must be 0, 1 or 2");
  LOGO_REQUIRE(a && b && c, LOGO_ERR_INVALID, "selftest operands must not be NULL");
  CUtensorMap tm_a, tm_b;
  int rc = make_tmap_2d_bf16(&tm_a, a, 128, 128, 256, 64, 128);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tm_b, b, 128, 128, 256, 64, 128);
  if (rc) return rc;
  const int smem_bytes = 65536 + 1024;
  LOGO_CHECK_CUDA(cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
  SelftestArgs args{mode, flags, lbo_bytes, sbo_bytes, kstep_bytes};
  const int grid = ((flags >> 24) & 0xff) ? ((flags >> 24) & 0xff) : 1;   // timing mode: identical CTAs load the chip
  umma_selftest_kernel<<<grid, 128, smem_bytes, (cudaStream_t)stream>>>(tm_a, tm_b, (const __nv_bfloat16*)a, c, status,
                                                                     args);
  LOGO_CHECK_CUDA(cudaGetLastError());
  return LOGO_OK;
}
