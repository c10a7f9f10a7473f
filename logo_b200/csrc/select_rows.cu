// Gate-threshold row selection and compaction.
//
// Kernel 1 (select_kernel): every warp tests 32 consecutive tokens at a time, turns the
// predicate into a bit mask with a warp ballot, ranks the selected lanes with popc, and
// the block obtains its global output offset with a single-pass decoupled look-back scan
// (blocks take their index from an atomic ticket, so every predecessor has started).
// Kernel 2 (finalize_kernel): per-sequence counts by binary search in the ascending index
// list, tile-offset prefix sums for the attention kernels, and the ordered gate sum.
//
// Bytes per launch (HBM-bound): n_tokens * sizeof(gate) read + Sq * 12 written.
#include "host_common.cuh"
#include "ptx.cuh"

#include <cuda_fp16.h>

#include <mutex>

namespace logo {

constexpr int SEL_THREADS = 256;
constexpr int SEL_WARPS = SEL_THREADS / 32;
constexpr int SEL_GROUPS = 8;                                  // 32-token groups per warp
constexpr int SEL_CHUNK = SEL_THREADS * SEL_GROUPS;            // 2048 tokens per block
constexpr size_t SEL_WS_HEADER = 16;                           // ticket (+ padding)

struct SelWorkspace {
  unsigned int* ticket;
  unsigned long long* state;   // [nblocks] (flag << 32) | value; flag 1 = aggregate, 2 = inclusive
  float* partial;              // [nblocks] per-block gate sums
};

__host__ __device__ inline int sel_num_blocks(int n_tokens) { return (n_tokens + SEL_CHUNK - 1) / SEL_CHUNK; }

__host__ __device__ inline SelWorkspace sel_ws(void* ws, int nblocks) {
  SelWorkspace w;
  uint8_t* p = static_cast<uint8_t*>(ws);
  w.ticket = reinterpret_cast<unsigned int*>(p);
  w.state = reinterpret_cast<unsigned long long*>(p + SEL_WS_HEADER);
  w.partial = reinterpret_cast<float*>(p + SEL_WS_HEADER + sizeof(unsigned long long) * (size_t)nblocks);
  return w;
}

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p, int i);
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p, int i) {
  return __bfloat162float(p[i]);
}
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half* p, int i) {
  return __half2float(p[i]);
}
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p, int i) {
  return p[i];
}
template <>
__device__ __forceinline__ float load_as_float<uint8_t>(const uint8_t* p, int i) {
  return p[i] ? 1.0f : 0.0f;
}

__device__ __forceinline__ float load_scalar(const void* p, int dtype) {
  if (dtype == LOGO_DTYPE_F32) return *static_cast<const float*>(p);
  if (dtype == LOGO_DTYPE_BF16) return __bfloat162float(*static_cast<const __nv_bfloat16*>(p));
  return __half2float(*static_cast<const __half*>(p));
}

// Largest s with cu[s] <= i (cu non-decreasing, cu[0] = 0): the sequence that owns token i.
// With empty sequences the LAST sequence starting at or before i is returned, which is what
// searchsorted(cu, i, right=True) - 1 gives.
__device__ __forceinline__ int owner_sequence(const int32_t* __restrict__ cu, int n_seq, int i) {
  int lo = 0, hi = n_seq;  // answer in [lo, hi)
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(cu + mid) <= i) lo = mid; else hi = mid;
  }
  return lo;
}

template <typename GateT, bool IS_BOOL>
__global__ void __launch_bounds__(SEL_THREADS)
    select_kernel(const GateT* __restrict__ gate, const void* __restrict__ thres_ptr, int thres_dtype,
                  const int32_t* __restrict__ cu, int n_seq, int n_tokens, int64_t* __restrict__ q_idx,
                  int32_t* __restrict__ pos_ids, void* ws_raw, int nblocks, int* status) {
  __shared__ int s_block;
  __shared__ int s_warp_count[SEL_WARPS];
  __shared__ float s_warp_sum[SEL_WARPS];
  __shared__ int s_block_excl;

  const SelWorkspace ws = sel_ws(ws_raw, nblocks);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  if (tid == 0) s_block = (int)atomicAdd(ws.ticket, 1u);
  __syncthreads();
  const int b = s_block;
  const float thres = IS_BOOL ? 0.5f : load_scalar(thres_ptr, thres_dtype);

  // ---- predicate + ballot per 32-token group ----
  const int warp_base = b * SEL_CHUNK + warp * (32 * SEL_GROUPS);
  unsigned masks[SEL_GROUPS];
  int warp_count = 0;
  float gsum = 0.f;
#pragma unroll
  for (int g = 0; g < SEL_GROUPS; ++g) {
    const int i = warp_base + g * 32 + lane;
    bool pred = false;
    if (i < n_tokens) {
      const float x = load_as_float<GateT>(gate, i);
      pred = (x >= thres);  // NaN compares false, as in the reference's `>=`
      if (!IS_BOOL) gsum += x;
    }
    masks[g] = __ballot_sync(0xffffffffu, pred);
    warp_count += __popc(masks[g]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) gsum += __shfl_xor_sync(0xffffffffu, gsum, o);
  if (lane == 0) {
    s_warp_count[warp] = warp_count;
    s_warp_sum[warp] = gsum;
  }
  __syncthreads();

  int warp_excl = 0, block_count = 0;
#pragma unroll
  for (int w = 0; w < SEL_WARPS; ++w) {
    const int c = s_warp_count[w];
    if (w < warp) warp_excl += c;
    block_count += c;
  }

  // ---- decoupled look-back over the blocks that hold earlier tickets ----
  if (warp == 0) {
    if (lane == 0) {
      float bs = 0.f;
#pragma unroll
      for (int w = 0; w < SEL_WARPS; ++w) bs += s_warp_sum[w];
      ws.partial[b] = bs;
    }
    int excl = 0;
    if (b > 0) {
      if (lane == 0) {
        const unsigned long long agg = (1ull << 32) | (unsigned)block_count;
        atomicExch(ws.state + b, agg);
      }
      int p = b - 1;
      bool done = false;
      const uint64_t t0 = globaltimer_ns();
      while (!done) {
        const int idx = p - lane;
        unsigned long long st = (2ull << 32);  // lanes before block 0 read as "inclusive 0"
        if (idx >= 0) {
          st = *reinterpret_cast<volatile unsigned long long*>(ws.state + idx);
        }
        const bool ready = (st >> 32) != 0;
        if (!__all_sync(0xffffffffu, ready)) {
          // the lanes read the clock independently: the verdict must be the same in all of them, or some
          // would leave the loop while the rest wait in the full-mask vote above
          const bool expired = __any_sync(0xffffffffu, globaltimer_ns() - t0 > LOGO_WAIT_TIMEOUT_NS);
          if (expired) {
            if (lane == 0 && status) atomicCAS(status, 0, (int)DEV_SCAN_TIMEOUT);
            break;
          }
          continue;
        }
        const unsigned incl_mask = __ballot_sync(0xffffffffu, (st >> 32) == 2);
        const int first_incl = incl_mask ? (__ffs(incl_mask) - 1) : 32;
        int v = (lane <= first_incl) ? (int)(unsigned)(st & 0xffffffffull) : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        excl += v;
        if (incl_mask) done = true; else p -= 32;
      }
    }
    if (lane == 0) {
      __threadfence();
      const unsigned long long inc = (2ull << 32) | (unsigned)(excl + block_count);
      atomicExch(ws.state + b, inc);
      s_block_excl = excl;
    }
  }
  __syncthreads();

  // ---- write the compacted lists ----
  int out = s_block_excl + warp_excl;
  const unsigned lt = (1u << lane) - 1u;
#pragma unroll
  for (int g = 0; g < SEL_GROUPS; ++g) {
    const unsigned m = masks[g];
    if ((m >> lane) & 1u) {
      const int i = warp_base + g * 32 + lane;
      const int dst = out + __popc(m & lt);
      const int s = owner_sequence(cu, n_seq, i);
      q_idx[dst] = (int64_t)i;
      pos_ids[dst] = i - __ldg(cu + s);
    }
    out += __popc(m);
  }
}

// One block. Writes cu_seqlens_q, the four tile-offset rows, meta and the gate sum.
__global__ void __launch_bounds__(1024)
    finalize_kernel(const int32_t* __restrict__ cu, int n_seq, int n_tokens, const int64_t* __restrict__ q_idx,
                    int32_t* __restrict__ cu_q, int32_t* __restrict__ tile_off,
                    int32_t* __restrict__ meta, float* __restrict__ gate_sum, void* ws_raw, int nblocks,
                    int* status) {
  __shared__ int s_scan_q[1024];
  __shared__ int s_scan_k[1024];
  __shared__ int s_scan_l[1024];
  __shared__ int s_scan_t[1024];
  __shared__ int s_carry_q, s_carry_k, s_carry_l, s_carry_t;
  int32_t* tile_off_q = tile_off;                      // selected rows, 256-row pairs
  int32_t* tile_off_k = tile_off + (n_seq + 1);        // keys, 128-row tiles
  int32_t* tile_off_l = tile_off + 2 * (n_seq + 1);    // all rows, 256-row pairs (local branch)
  int32_t* tile_off_t = tile_off + 3 * (n_seq + 1);    // selected rows, 128-row tiles (backward)
  const SelWorkspace ws = sel_ws(ws_raw, nblocks);
  const int tid = threadIdx.x;
  const int sq = nblocks > 0 ? (int)(unsigned)(ws.state[nblocks - 1] & 0xffffffffull) : 0;

  // per-sequence prefix of selected rows: number of selected indices below cu[s]
  bool bad = false;
  for (int s = tid; s <= n_seq; s += blockDim.x) {
    const int c = cu[s];
    if (c < 0 || c > n_tokens || (s > 0 && c < cu[s - 1]) || (s == 0 && c != 0) || (s == n_seq && c != n_tokens))
      bad = true;
    int lo = 0, hi = sq;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (q_idx[mid] < (int64_t)c) lo = mid + 1; else hi = mid;
    }
    cu_q[s] = lo;
  }
  if (bad && status) atomicCAS(status, 0, (int)DEV_BAD_INDEX);
  if (tid == 0) {
    s_carry_q = 0;
    s_carry_k = 0;
    s_carry_l = 0;
    s_carry_t = 0;
    tile_off_t[0] = 0;
    tile_off_q[0] = 0;
    tile_off_k[0] = 0;
    tile_off_l[0] = 0;
  }
  __syncthreads();

  // prefix sums of tiles per sequence, 1024 sequences per round
  for (int base = 0; base < n_seq; base += 1024) {
    const int s = base + tid;
    int tq = 0, tk = 0, tl = 0, tt = 0;
    if (s < n_seq) {
      const int nq = max(cu_q[s + 1] - cu_q[s], 0);
      const int nk = max(cu[s + 1] - cu[s], 0);
      tq = (nq + 2 * LOGO_TILE - 1) / (2 * LOGO_TILE);
      tk = (nk + LOGO_TILE - 1) / LOGO_TILE;
      tl = (nk + 2 * LOGO_TILE - 1) / (2 * LOGO_TILE);
      tt = (nq + LOGO_TILE - 1) / LOGO_TILE;
    }
    s_scan_q[tid] = tq;
    s_scan_k[tid] = tk;
    s_scan_l[tid] = tl;
    s_scan_t[tid] = tt;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      int aq = 0, ak = 0, al = 0, at = 0;
      if (tid >= off) {
        aq = s_scan_q[tid - off];
        ak = s_scan_k[tid - off];
        al = s_scan_l[tid - off];
        at = s_scan_t[tid - off];
      }
      __syncthreads();
      s_scan_q[tid] += aq;
      s_scan_k[tid] += ak;
      s_scan_l[tid] += al;
      s_scan_t[tid] += at;
      __syncthreads();
    }
    if (s < n_seq) {
      tile_off_q[s + 1] = s_carry_q + s_scan_q[tid];
      tile_off_k[s + 1] = s_carry_k + s_scan_k[tid];
      tile_off_l[s + 1] = s_carry_l + s_scan_l[tid];
      tile_off_t[s + 1] = s_carry_t + s_scan_t[tid];
    }
    __syncthreads();
    if (tid == 0) {
      s_carry_q += s_scan_q[1023];
      s_carry_k += s_scan_k[1023];
      s_carry_l += s_scan_l[1023];
      s_carry_t += s_scan_t[1023];
    }
    __syncthreads();
  }

  if (tid == 0) {
    meta[0] = sq;
    meta[1] = s_carry_q;
    meta[2] = s_carry_k;
    meta[3] = s_carry_l;
    meta[4] = s_carry_t;
    meta[5] = meta[6] = meta[7] = 0;
    if (gate_sum) {
      float acc = 0.f;
      for (int b = 0; b < nblocks; ++b) acc += ws.partial[b];
      *gate_sum = acc;
    }
  }
}

}  // namespace logo

extern "C" size_t logo_select_workspace_bytes(int n_tokens) {
  const int nb = logo::sel_num_blocks(n_tokens < 0 ? 0 : n_tokens);
  return logo::SEL_WS_HEADER + (size_t)nb * (sizeof(unsigned long long) + sizeof(float)) + 16;
}

namespace logo {

// Argument checks and the two launches shared by logo_select_rows and logo_select_rows_static;
// `scratch` holds logo_select_workspace_bytes(n_tokens) bytes, whoever owns them. It is cleared on the
// stream first: the ticket and the look-back words must start at zero.
static int select_rows_impl(const void* gate, int gate_dtype, const void* thres, int thres_dtype,
                            const int32_t* cu_seqlens, int n_seq, int n_tokens, int64_t* q_idx, int32_t* pos_ids,
                            int32_t* cu_seqlens_q, int32_t* tile_off, int32_t* meta, float* gate_sum, void* scratch,
                            int32_t* status, cudaStream_t stream) {
  LOGO_REQUIRE(cu_seqlens && cu_seqlens_q && tile_off && meta, LOGO_ERR_INVALID,
               "cu_seqlens, cu_seqlens_q, tile_off and meta must not be NULL");
  LOGO_REQUIRE(n_tokens == 0 || (gate && q_idx && pos_ids), LOGO_ERR_INVALID,
               "gate, q_idx and pos_ids must not be NULL");
  LOGO_REQUIRE(gate_dtype >= LOGO_DTYPE_BF16 && gate_dtype <= LOGO_DTYPE_BOOL, LOGO_ERR_INVALID,
               "unknown gate dtype %d", gate_dtype);
  if (gate_dtype != LOGO_DTYPE_BOOL) {
    LOGO_REQUIRE(thres != nullptr, LOGO_ERR_INVALID, "thres must not be NULL for a floating-point gate");
    LOGO_REQUIRE(thres_dtype >= LOGO_DTYPE_BF16 && thres_dtype <= LOGO_DTYPE_F16, LOGO_ERR_INVALID,
                 "unknown threshold dtype %d", thres_dtype);
  }
  const int nblocks = sel_num_blocks(n_tokens);
  LOGO_CHECK_CUDA(cudaMemsetAsync(scratch, 0, logo_select_workspace_bytes(n_tokens), stream));
  prof_begin(PROF_SELECT, stream);
  if (nblocks > 0) {
#define LOGO_LAUNCH_SELECT(T, ISB)                                                                        \
  select_kernel<T, ISB><<<nblocks, SEL_THREADS, 0, stream>>>(static_cast<const T*>(gate), thres, thres_dtype, \
                                                             cu_seqlens, n_seq, n_tokens, q_idx, pos_ids,  \
                                                             scratch, nblocks, status)
    switch (gate_dtype) {
      case LOGO_DTYPE_BF16: LOGO_LAUNCH_SELECT(__nv_bfloat16, false); break;
      case LOGO_DTYPE_F16: LOGO_LAUNCH_SELECT(__half, false); break;
      case LOGO_DTYPE_F32: LOGO_LAUNCH_SELECT(float, false); break;
      default: LOGO_LAUNCH_SELECT(uint8_t, true); break;
    }
#undef LOGO_LAUNCH_SELECT
    LOGO_CHECK_CUDA(cudaGetLastError());
  }
  finalize_kernel<<<1, 1024, 0, stream>>>(cu_seqlens, n_seq, n_tokens, q_idx, cu_seqlens_q, tile_off, meta, gate_sum,
                                          scratch, nblocks, status);
  prof_end(PROF_SELECT, stream);
  LOGO_CHECK_CUDA(cudaGetLastError());
  return LOGO_OK;
}

}  // namespace logo

extern "C" int logo_select_rows(const void* gate, int gate_dtype, const void* thres, int thres_dtype,
                                const int32_t* cu_seqlens, int n_seq, int n_tokens, int64_t* q_idx, int32_t* pos_ids,
                                int32_t* cu_seqlens_q, int32_t* tile_off, int32_t* meta, float* gate_sum,
                                void* workspace, size_t workspace_bytes, int32_t* status, logo_stream_t stream_) {
  using namespace logo;
  LOGO_REQUIRE(n_tokens >= 0 && n_seq >= 0, LOGO_ERR_INVALID, "n_tokens and n_seq must be non-negative");
  LOGO_REQUIRE(workspace && workspace_bytes >= logo_select_workspace_bytes(n_tokens), LOGO_ERR_WORKSPACE,
               "select workspace too small: need %zu bytes", logo_select_workspace_bytes(n_tokens));
  LOGO_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15u) == 0, LOGO_ERR_INVALID,
               "select workspace must be 16-byte aligned");
  return select_rows_impl(gate, gate_dtype, thres, thres_dtype, cu_seqlens, n_seq, n_tokens, q_idx, pos_ids,
                          cu_seqlens_q, tile_off, meta, gate_sum, workspace, status, (cudaStream_t)stream_);
}

// ---------------------------------------------------------------------------------------
// Variant of logo_select_rows for callers that cannot hand over a workspace.
//
// Some hosts of this library are not allowed to allocate device memory at all: a plugin
// inside a serving process whose memory budget is fixed at start-up, or a step function on a
// latency-critical path where cudaMalloc / cudaFree are banned because they serialise the
// whole device. For them the scan scratch (ticket, per-block look-back words, per-block gate
// partials) lives in the file-scope array below instead of a caller buffer. Every GPU that
// loads the library holds these LOGO_SELECT_STATIC_BYTES until the process exits.
//
// `g_select_scratch` is a device symbol: inside host code the name is only a stand-in, not
// an address a kernel could use. The device address is looked up with cudaGetSymbolAddress,
// once per device with that device current, and cached; kernels receive that pointer. The cached
// address does not survive cudaDeviceReset: a process that resets a device must not call this
// entry point on it afterwards.
// ---------------------------------------------------------------------------------------
namespace logo {

constexpr int SELECT_STATIC_MAX_TOKENS = LOGO_SELECT_STATIC_MAX_TOKENS;
constexpr size_t SELECT_STATIC_BYTES =
    SEL_WS_HEADER + (size_t)((SELECT_STATIC_MAX_TOKENS + SEL_CHUNK - 1) / SEL_CHUNK) * (sizeof(unsigned long long) + sizeof(float)) + 16;

static __device__ __align__(256) unsigned char g_select_scratch[SELECT_STATIC_BYTES];

static std::mutex g_select_scratch_mu;
static void* g_select_scratch_ptr[64] = {nullptr};

// Device address of g_select_scratch on the current device (set-up on the first call per device).
static int select_static_scratch(void** out) {
  int dev = 0;
  LOGO_CHECK_CUDA(cudaGetDevice(&dev));
  LOGO_REQUIRE(dev >= 0 && dev < 64, LOGO_ERR_UNSUPPORTED, "device ordinal %d is outside the supported range", dev);
  std::lock_guard<std::mutex> lk(g_select_scratch_mu);
  if (g_select_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_select_scratch);
    if (e != cudaSuccess || p == nullptr)
      return set_error(LOGO_ERR_CUDA, "cudaGetSymbolAddress(g_select_scratch) failed on device %d: %s", dev,
                       cudaGetErrorString(e));
    g_select_scratch_ptr[dev] = p;
  }
  *out = g_select_scratch_ptr[dev];
  return LOGO_OK;
}

}  // namespace logo

extern "C" int logo_select_rows_static(const void* gate, int gate_dtype, const void* thres, int thres_dtype,
                                       const int32_t* cu_seqlens, int n_seq, int n_tokens, int64_t* q_idx,
                                       int32_t* pos_ids, int32_t* cu_seqlens_q, int32_t* tile_off, int32_t* meta,
                                       float* gate_sum, int32_t* status, logo_stream_t stream_) {
  using namespace logo;
  LOGO_REQUIRE(n_tokens >= 0 && n_seq >= 0, LOGO_ERR_INVALID, "n_tokens and n_seq must be non-negative");
  LOGO_REQUIRE(n_tokens <= SELECT_STATIC_MAX_TOKENS, LOGO_ERR_UNSUPPORTED,
               "logo_select_rows_static handles at most %d tokens per call (got %d); use logo_select_rows with a "
               "caller workspace for larger inputs",
               SELECT_STATIC_MAX_TOKENS, n_tokens);
  void* scratch = nullptr;
  const int rc = select_static_scratch(&scratch);
  if (rc) return rc;
  // The array keeps what the previous call left; select_rows_impl clears the part this call uses.
  return select_rows_impl(gate, gate_dtype, thres, thres_dtype, cu_seqlens, n_seq, n_tokens, q_idx, pos_ids,
                          cu_seqlens_q, tile_off, meta, gate_sum, scratch, status, (cudaStream_t)stream_);
}
