// Error text, driver entry points and per-device properties for the C ABI.
#include "host_common.cuh"

#include <cudaTypedefs.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <vector>

namespace logo {

static thread_local char g_last_error[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
static std::once_flag g_encode_once;

static void load_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault, &qres);
  if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) {
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  }
}

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle_bytes) {
  std::call_once(g_encode_once, load_encode);
  if (!g_encode) return set_error(LOGO_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  if (!aligned16(base) || (row_stride_bytes & 15u))
    return set_error(LOGO_ERR_INVALID, "tensor base and row stride must be 16-byte aligned for TMA");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(LOGO_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return LOGO_OK;
}

int make_tmap_2d_f32(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                     uint32_t box_inner, uint32_t box_outer) {
  std::call_once(g_encode_once, load_encode);
  if (!g_encode) return set_error(LOGO_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  if (!aligned16(base) || (row_stride_bytes & 15u))
    return set_error(LOGO_ERR_INVALID, "tensor base and row stride must be 16-byte aligned for TMA");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(LOGO_ERR_CUDA, "cuTensorMapEncodeTiled (fp32) failed with CUresult %d", (int)r);
  return LOGO_OK;
}

int sm_count() {
  static int cached[64];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  std::lock_guard<std::mutex> lk(mu);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// ---------------------------------------------------------------------------------------
// optional per-kernel timing with CUDA events (off by default, per host thread)
// ---------------------------------------------------------------------------------------
struct ProfSlot {
  cudaEvent_t start, stop;
};
static thread_local bool g_prof_on = false;
static thread_local std::vector<ProfSlot>* g_prof = nullptr;   // [PROF_KINDS] vectors
// Events are recycled: creating events in the middle of a timed loop can stall the stream for
// milliseconds when the driver has to grow its event pool.
static thread_local std::vector<ProfSlot>* g_prof_free = nullptr;

bool prof_enabled() { return g_prof_on; }

void prof_begin(int kind, cudaStream_t stream) {
  if (!g_prof_on || kind < 0 || kind >= PROF_KINDS) return;
  ProfSlot s{};
  if (g_prof_free && !g_prof_free->empty()) {
    s = g_prof_free->back();
    g_prof_free->pop_back();
  } else if (cudaEventCreate(&s.start) != cudaSuccess || cudaEventCreate(&s.stop) != cudaSuccess) {
    return;
  }
  cudaEventRecord(s.start, stream);
  g_prof[kind].push_back(s);
}

void prof_end(int kind, cudaStream_t stream) {
  if (!g_prof_on || kind < 0 || kind >= PROF_KINDS || g_prof[kind].empty()) return;
  cudaEventRecord(g_prof[kind].back().stop, stream);
}

}  // namespace logo

extern "C" int logo_profile_enable(int on) {
  using namespace logo;
  if (!g_prof) g_prof = new std::vector<ProfSlot>[PROF_KINDS];
  if (!g_prof_free) g_prof_free = new std::vector<ProfSlot>();
  g_prof_on = (on != 0);
  return LOGO_OK;
}

extern "C" int logo_profile_reserve(int n_launches) {
  using namespace logo;
  if (!g_prof_free) g_prof_free = new std::vector<ProfSlot>();
  while ((int)g_prof_free->size() < n_launches && g_prof_free->size() < 4096) {
    ProfSlot s{};
    LOGO_CHECK_CUDA(cudaEventCreate(&s.start));
    LOGO_CHECK_CUDA(cudaEventCreate(&s.stop));
    g_prof_free->push_back(s);
  }
  return LOGO_OK;
}

extern "C" int logo_profile_read(double* total_ms, int* launches, int n) {
  using namespace logo;
  for (int k = 0; k < n; ++k) {
    double total = 0.0;
    int count = 0;
    if (g_prof && k < PROF_KINDS) {
      for (ProfSlot& s : g_prof[k]) {
        float ms = 0.f;
        if (cudaEventSynchronize(s.stop) == cudaSuccess && cudaEventElapsedTime(&ms, s.start, s.stop) == cudaSuccess) {
          total += ms;
          ++count;
        }
        if (g_prof_free && g_prof_free->size() < 4096) {
          g_prof_free->push_back(s);
        } else {
          cudaEventDestroy(s.start);
          cudaEventDestroy(s.stop);
        }
      }
      g_prof[k].clear();
    }
    if (total_ms) total_ms[k] = total;
    if (launches) launches[k] = count;
  }
  return LOGO_OK;
}

extern "C" int logo_version(void) { return 100; }

extern "C" int logo_last_error(char* buf, int n) {
  if (!buf || n <= 0) return (int)strlen(logo::g_last_error);
  strncpy(buf, logo::g_last_error, (size_t)n - 1);
  buf[n - 1] = '\0';
  return (int)strlen(buf);
}


// ---------------------------------------------------------------------------------------
// zero the unselected rows of an output tensor
// ---------------------------------------------------------------------------------------
namespace logo {

__global__ void __launch_bounds__(256)
    zero_unselected_rows_kernel(uint4* __restrict__ base, const int64_t* __restrict__ q_idx,
                                const int32_t* __restrict__ sq_ptr, int n_tokens, int row_chunks) {
  const int sq = min(max(__ldg(sq_ptr), 0), n_tokens);
  zero_unselected_rows_part(base, q_idx, sq, n_tokens, row_chunks, (blockIdx.x * blockDim.x + threadIdx.x) >> 5,
                            (gridDim.x * blockDim.x) >> 5, threadIdx.x & 31);
}

int launch_zero_unselected_rows(void* base, const int64_t* q_idx, const int32_t* sq_ptr, int n_tokens,
                                size_t row_bytes, cudaStream_t stream) {
  if (n_tokens <= 0) return LOGO_OK;
  LOGO_REQUIRE(base && q_idx && sq_ptr && row_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(base) & 15) == 0,
               LOGO_ERR_INVALID, "zero_unselected_rows: bad arguments");
  const int grid = sm_count() * 8;
  zero_unselected_rows_kernel<<<grid, 256, 0, stream>>>(static_cast<uint4*>(base), q_idx, sq_ptr, n_tokens,
                                                        (int)(row_bytes / 16));
  LOGO_CHECK_CUDA(cudaGetLastError());
  return LOGO_OK;
}

}  // namespace logo
