// Library-wide plumbing of librapidh3_b200: last-error string, CUDA error mapping, TMA tensor-map
// encoding through the driver entry point (no link-time dependency on libcuda), per-device SM
// count and the device status word that bounded waits report into.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "rapidh3_b200.h"

namespace rh3 {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return 0;
  snprintf(g_err, sizeof(g_err), "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
  return static_cast<int>(e);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tmap_nd(CUtensorMap* out, CUtensorMapDataType dt, uint32_t elem_bytes, const void* base, int rank,
                 const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return set_error(RH3_ARG_ERROR, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bx[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];  // stride of dim i (dim 0 is contiguous)
  }
  (void)elem_bytes;
  CUresult r = enc(out, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr, bx, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(RH3_ARG_ERROR, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

int make_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, uint32_t elem_bytes, const void* base, uint64_t inner,
                 uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                 CUtensorMapSwizzle swz) {
  const uint64_t dims[2] = {inner, outer};
  const uint64_t strides[1] = {row_stride_bytes};
  const uint32_t box[2] = {box_inner, box_outer};
  return make_tmap_nd(out, dt, elem_bytes, base, 2, dims, strides, box, swz);
}

int device_sm_count() {
  static int cache[64];
  static bool have[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!have[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev] = n;
    have[dev] = true;
  }
  return cache[dev];
}

// One status word per device, living in the module's device data segment (no allocation).
__device__ int g_status_word[4];

int* device_status_word() {
  static int* cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cache[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    cache[dev] = static_cast<int*>(p);
  }
  return cache[dev];
}

// Self-test of the bounded-wait machinery: 64 threads wait, with a limit of `max_polls` polls, on an mbarrier that
// nobody ever arrives at. The wait runs out, the first thread to give up raises the CTA's abort flag and records
// ST_TIMEOUT_SELFTEST in the status word, the others see the flag and leave, and the kernel returns by itself.
__global__ void wait_expiry_kernel(uint32_t max_polls, int* status, int* left_normally) {
  __shared__ uint64_t never;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&never, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  const bool done = mbar_wait_polls(&never, 0, &abort_flag, status, ST_TIMEOUT_SELFTEST, max_polls);
  __syncthreads();
  if (threadIdx.x == 0) {
    *left_normally = done ? 0 : 1;
    mbar_inval(&never);
  }
}

}  // namespace rh3

extern "C" int rh3_selftest_wait_expiry(int64_t max_polls, int* left_normally, cudaStream_t stream) {
  RH3_CHECK_ARG(max_polls >= 1 && max_polls <= (1 << 20), "selftest_wait_expiry: max_polls=%lld must be in [1, 2^20]",
                (long long)max_polls);
  RH3_CHECK_ARG(left_normally != nullptr, "selftest_wait_expiry: null result pointer");
  int* w = rh3::device_status_word();
  if (!w) return rh3::set_error(RH3_ARG_ERROR, "no device status word (is a CUDA device current?)");
  rh3::wait_expiry_kernel<<<1, 64, 0, stream>>>(static_cast<uint32_t>(max_polls), w, left_normally);
  return rh3::check_cuda(cudaGetLastError(), "selftest_wait_expiry launch");
}

extern "C" const char* rh3_last_error_string(void) { return rh3::g_err; }

extern "C" int rh3_version(void) { return 100; }

extern "C" int rh3_sm_count(void) { return rh3::device_sm_count(); }

// Synchronizes `stream`, returns the device status word (0 = every bounded wait completed) and
// clears it. A non-zero value names the wait that gave up (see common.cuh ST_*).
extern "C" int rh3_check_status(cudaStream_t stream, int* status_out) {
  int* w = rh3::device_status_word();
  if (!w) return rh3::set_error(RH3_ARG_ERROR, "no device status word (is a CUDA device current?)");
  int v = 0;
  if (int e = rh3::check_cuda(cudaMemcpyAsync(&v, w, sizeof(int), cudaMemcpyDeviceToHost, stream), "status read"))
    return e;
  if (int e = rh3::check_cuda(cudaStreamSynchronize(stream), "status sync")) return e;
  if (v != 0) {
    if (int e = rh3::check_cuda(cudaMemsetAsync(w, 0, sizeof(int), stream), "status clear")) return e;
    rh3::set_error(v, "a bounded device wait gave up (status %d)", v);
  }
  if (status_out) *status_out = v;
  return 0;
}
