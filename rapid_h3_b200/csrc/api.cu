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

// Issue-rate probe of the tensor pipe: one CTA per SM, one thread issues `groups` groups of 64 MMAs of 128 x 256 x 32
// (8-bit kinds) or 128 x 256 x 16 (bf16) on zeroed shared-memory operands, alternating between two TMEM accumulators,
// with a commit per group and a bounded wait for the group before the previous one (so two groups are always in
// flight). The accumulators just keep accumulating (int32 wraps, floats may saturate: the values are not read). No
// memory traffic beyond shared memory: what it measures is the rate the MMAs retire at under the clocks
// the GPU actually holds, the denominator for the 8-bit kernels' tensor rooflines.
template <int KIND>   // 0 = kind::i8, 1 = kind::f8f6f4 (e4m3), 2 = kind::f16 (bf16)
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int groups, int random_operands, int pattern, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar[4];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  // operands: zeros, or a fixed pseudo-random byte pattern (switching activity like real data, which is what the
  // power cap responds to; for e4m3 / bf16 the exponent bits are masked so that every value is finite)
  for (int i = threadIdx.x; i < (128 + 256) * 128 / 4; i += blockDim.x) {
    uint32_t w = 0;
    if (random_operands) {
      w = (static_cast<uint32_t>(i) + 1u) * 2654435761u;
      w ^= w >> 15;
      w *= 2246822519u;
      w ^= w >> 13;
      if (KIND == 1) w &= 0xBFBFBFBFu;      // e4m3: clear the top exponent bit of every byte (|x| < 2)
      if (KIND == 2) w &= 0xBFFFBFFFu;      // bf16: clear the top exponent bit of both halves (|x| < 2)
    }
    reinterpret_cast<uint32_t*>(smem)[i] = w;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; ++i) mbar_init(&bar[i], 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  fence_proxy_async_smem();
  if (threadIdx.x < 32) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  if (threadIdx.x == 0 && pattern != 3) {
    const uint64_t a_desc = make_desc_k128(smem_u32(smem)), b_desc = make_desc_k128(smem_u32(smem + 128 * 128));
    // pattern 4: the same back-to-back issue with 128-column MMAs (half the work per instruction)
    const int ncols = pattern == 4 ? 128 : 256;
    const uint32_t idesc = KIND == 0 ? make_idesc(2, 1, 1, 128, ncols) : (KIND == 1 ? make_idesc(1, 0, 0, 128, ncols)
                                                                                     : make_idesc(1, 1, 1, 128, ncols));
    bool ok = true;
    auto mma4 = [&](uint32_t d, uint64_t a, uint64_t b) {
      if (KIND == 0) mma4_i8_ss(d, a, b, idesc, 1);
      else if (KIND == 1) mma4_f8_ss(d, a, b, idesc, 1);
      else mma4_f16_ss(d, a, b, idesc, 1);
    };
    if (pattern == 0 || pattern == 4) {
      for (int g = 0; g < groups && ok; ++g) {
#pragma unroll 1
        for (int i = 0; i < 16; ++i) mma4(tmem_base + (i & 1) * 256, a_desc, b_desc);   // 16 x 4 MMAs
        mma_commit(&bar[g & 1]);
        if (g > 0) ok = mbar_wait(&bar[(g - 1) & 1], ((g - 1) >> 1) & 1, &abort_flag, status, ST_TIMEOUT_SELFTEST);
      }
      if (ok && groups > 0) mbar_wait(&bar[(groups - 1) & 1], ((groups - 1) >> 1) & 1, &abort_flag, status, ST_TIMEOUT_SELFTEST);
    } else {
      // The issue pattern of a pipelined GEMM main loop: a four-stage ring, and per stage (four MMAs) one wait on the
      // stage's barrier, the descriptors, the MMAs and one commit on the same barrier, which therefore completes four
      // stages later, when those MMAs have retired. pattern 1 builds the descriptors from the stage index every time;
      // pattern 2 keeps one descriptor pair per stage in registers and selects by a switch.
      const int n = groups * 16;
      const int stage_stride = (groups >> 20) * 1024;
      uint64_t a_s[4], b_s[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) a_s[q] = a_desc, b_s[q] = b_desc;
      int stage = 0;
      uint32_t phase = 0;
      for (int i = 0; i < n && ok; ++i) {
        if (i >= 4) ok = mbar_wait(&bar[stage], phase ^ 1, &abort_flag, status, ST_TIMEOUT_SELFTEST);
        tc_fence_after();
        const uint32_t d = tmem_base + (i & 1) * 256;
        if (pattern == 1) {
          // the same tile for every stage, but computed from the stage index as a main loop would (stage_stride is
          // zero at run time, which the compiler cannot know)
          const uint32_t a_addr = smem_u32(smem + stage * stage_stride);
          mma4(d, make_desc_k128(a_addr), make_desc_k128(a_addr + 128 * 128));
        } else {
          switch (stage) {
            case 0: mma4(d, a_s[0], b_s[0]); break;
            case 1: mma4(d, a_s[1], b_s[1]); break;
            case 2: mma4(d, a_s[2], b_s[2]); break;
            default: mma4(d, a_s[3], b_s[3]); break;
          }
        }
        mma_commit(&bar[stage]);
        if (++stage == 4) { stage = 0; phase ^= 1; }
      }
      // drain: the last commit of every stage
      for (int q = 0; q < 4 && ok; ++q) {
        const int last = n - 1 - ((n - 1 - q) % 4 + 4) % 4;   // last iteration that used stage q
        if (last >= 0 && (last % 4) == q) ok = mbar_wait(&bar[q], (last / 4) & 1, &abort_flag, status, ST_TIMEOUT_SELFTEST);
      }
    }
  }
  if (pattern == 3 && threadIdx.x < 32) {
    // The same ring with the WHOLE warp in the loop (waits, counters and descriptors are warp-uniform, so they can live
    // in the uniform datapath) and one elected lane issuing the MMAs and the commit.
    const uint64_t a_desc = make_desc_k128(smem_u32(smem)), b_desc = make_desc_k128(smem_u32(smem + 128 * 128));
    // pattern 4: the same back-to-back issue with 128-column MMAs (half the work per instruction)
    const int ncols = pattern == 4 ? 128 : 256;
    const uint32_t idesc = KIND == 0 ? make_idesc(2, 1, 1, 128, ncols) : (KIND == 1 ? make_idesc(1, 0, 0, 128, ncols)
                                                                                     : make_idesc(1, 1, 1, 128, ncols));
    const int n = groups * 16;
    const int stage_stride = (groups >> 20) * 1024;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int i = 0; i < n && ok; ++i) {
      if (i >= 4) ok = mbar_wait(&bar[stage], phase ^ 1, &abort_flag, status, ST_TIMEOUT_SELFTEST);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
      const uint32_t d = tmem_base + (i & 1) * 256;
      const uint32_t a_addr = smem_u32(smem + stage * stage_stride);
      if (elect_one()) {
        if (KIND == 0) mma4_i8_ss(d, make_desc_k128(a_addr), make_desc_k128(a_addr + 128 * 128), idesc, 1);
        else if (KIND == 1) mma4_f8_ss(d, make_desc_k128(a_addr), make_desc_k128(a_addr + 128 * 128), idesc, 1);
        else mma4_f16_ss(d, make_desc_k128(a_addr), make_desc_k128(a_addr + 128 * 128), idesc, 1);
        mma_commit(&bar[stage]);
      }
      __syncwarp();
      if (++stage == 4) { stage = 0; phase ^= 1; }
    }
    for (int q = 0; q < 4 && ok; ++q) {
      const int last = n - 1 - ((n - 1 - q) % 4 + 4) % 4;
      if (last >= 0 && (last % 4) == q) ok = mbar_wait(&bar[q], (last / 4) & 1, &abort_flag, status, ST_TIMEOUT_SELFTEST);
    }
    (void)a_desc; (void)b_desc;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// The main loop of a 128 x 256 int8 GEMM tile without an epilogue: a four-stage ring of 48 KB stages; warp 1 streams
// `fill_bytes` (0 .. 48 KB, multiples of 16 KB) per stage from global memory into the stage by bulk copies that
// complete on the stage's barrier, warp 0 (converged, one elected lane) waits for the stage, issues four MMAs of
// 128 x 256 x 32 on it and commits the stage free. Whatever bytes arrive are the int8 operands. What it measures:
// the MMA rate an SM sustains while it takes in fill_bytes per 512 tensor cycles from L2 / HBM.
__global__ void __launch_bounds__(128, 1) mma_feed_kernel(const uint8_t* __restrict__ src, long long src_bytes, int stages_total,
                                                           int fill_bytes, int* status) {
  constexpr int ST = 4, SB = 48 * 1024;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full[ST], empty[ST];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < ST * SB / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    for (int i = 0; i < ST; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    abort_flag = 0;
    fence_barrier_init();
  }
  fence_proxy_async_smem();
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  if (warp == 1) {
    // producer: every CTA walks its own window of the source so that the SMs do not all read the same lines
    const long long window = (src_bytes / SB) > 0 ? (src_bytes / SB) : 1;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int i = 0; i < stages_total && ok; ++i) {
      ok = __all_sync(0xffffffffu, mbar_wait(&empty[stage], phase ^ 1, &abort_flag, status, ST_TIMEOUT_SELFTEST));
      if (!ok) break;
      if (elect_one()) {
        if (fill_bytes > 0) {
          const uint8_t* g = src + ((static_cast<long long>(blockIdx.x) * 131 + i) % window) * SB;
          mbar_arrive_expect_tx(&full[stage], fill_bytes);
          for (int o = 0; o < fill_bytes; o += 16384)
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             smem_u32(smem + stage * SB + o)),
                         "l"(g + o), "r"(16384), "r"(smem_u32(&full[stage]))
                         : "memory");
        } else {
          mbar_arrive(&full[stage]);
        }
      }
      __syncwarp();
      if (++stage == ST) { stage = 0; phase ^= 1; }
    }
  } else if (warp == 0) {
    constexpr uint32_t idesc = make_idesc(2, 1, 1, 128, 256);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int i = 0; i < stages_total && ok; ++i) {
      ok = __all_sync(0xffffffffu, mbar_wait(&full[stage], phase, &abort_flag, status, ST_TIMEOUT_SELFTEST));
      if (!ok) break;
      tc_fence_after();
      const uint32_t a_addr = smem_u32(smem + stage * SB);
      if (elect_one()) {
        mma4_i8_ss(tmem_base + (i & 1) * 256, make_desc_k128(a_addr), make_desc_k128(a_addr + 128 * 128), idesc, 1);
        mma_commit(&empty[stage]);
      }
      __syncwarp();
      if (++stage == ST) { stage = 0; phase ^= 1; }
    }
    // drain: the last commit of every stage that was used
    for (int q = 0; q < ST && ok; ++q) {
      const int last = stages_total - 1 - ((stages_total - 1 - q) % ST + ST) % ST;
      if (last >= 0 && (last % ST) == q)
        ok = __all_sync(0xffffffffu, mbar_wait(&empty[q], (last / ST) & 1, &abort_flag, status, ST_TIMEOUT_SELFTEST));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace rh3

// The GEMM main loop without an epilogue on every SM (see mma_feed_kernel): `stages` stages of four int8 MMAs of
// 128 x 256 x 32, each stage preceded by a bulk copy of fill_bytes (0, 16384, 32768 or 49152) from `src` (device
// memory, src_bytes >= 49152, 16-byte aligned) into the stage. *ops_out = operations of the launch.
extern "C" int rh3_selftest_mma_feed(const void* src, int64_t src_bytes, int64_t stages, int fill_bytes, double* ops_out,
                                     cudaStream_t stream) {
  RH3_CHECK_ARG(stages >= 1 && stages <= (1 << 22), "selftest_mma_feed: stages=%lld must be in [1, 2^22]", (long long)stages);
  RH3_CHECK_ARG(fill_bytes >= 0 && fill_bytes <= 49152 && fill_bytes % 16384 == 0, "selftest_mma_feed: fill_bytes must be 0, 16384, 32768 or 49152");
  RH3_CHECK_ARG(fill_bytes == 0 || (src && src_bytes >= 49152 && (reinterpret_cast<uintptr_t>(src) & 15) == 0),
                "selftest_mma_feed: src must be a 16-byte aligned device buffer of at least 49152 bytes");
  int* w = rh3::device_status_word();
  if (!w) return rh3::set_error(RH3_ARG_ERROR, "no device status word (is a CUDA device current?)");
  const int sms = rh3::device_sm_count();
  const int smem = 4 * 48 * 1024 + 1024;
  if (int e = rh3::check_cuda(cudaFuncSetAttribute(rh3::mma_feed_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "mma_feed smem"))
    return e;
  rh3::mma_feed_kernel<<<sms, 128, smem, stream>>>(static_cast<const uint8_t*>(src), static_cast<long long>(src_bytes),
                                                   static_cast<int>(stages), fill_bytes, w);
  if (ops_out) *ops_out = static_cast<double>(sms) * static_cast<double>(stages) * 4.0 * 2.0 * 128.0 * 256.0 * 32.0;
  return rh3::check_cuda(cudaGetLastError(), "selftest_mma_feed launch");
}

// Launches the issue-rate probe on every SM; the caller times it with CUDA events. Operations per launch:
// sm_count * groups * 64 * 2 * 128 * 256 * (32 for kind 0 / 1, 16 for kind 2); *ops_out receives that number.
extern "C" int rh3_selftest_mma_rate(int kind, int64_t groups, int random_operands, int pattern, double* ops_out,
                                     cudaStream_t stream) {
  RH3_CHECK_ARG(kind >= 0 && kind <= 2, "selftest_mma_rate: kind must be 0 (i8), 1 (e4m3) or 2 (bf16)");
  RH3_CHECK_ARG(groups >= 1 && groups <= (1 << 16), "selftest_mma_rate: groups=%lld must be in [1, 65536]", (long long)groups);
  RH3_CHECK_ARG(pattern >= 0 && pattern <= 4, "selftest_mma_rate: pattern must be 0..4");
  int* w = rh3::device_status_word();
  if (!w) return rh3::set_error(RH3_ARG_ERROR, "no device status word (is a CUDA device current?)");
  const int sms = rh3::device_sm_count();
  const int smem = (128 + 256) * 128 + 1024;
  auto launch = [&](auto kern) {
    if (int e = rh3::check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "mma_rate smem"))
      return e;
    kern<<<sms, 128, smem, stream>>>(static_cast<int>(groups), random_operands, pattern, w);
    return rh3::check_cuda(cudaGetLastError(), "selftest_mma_rate launch");
  };
  int e = kind == 0 ? launch(rh3::mma_rate_kernel<0>) : (kind == 1 ? launch(rh3::mma_rate_kernel<1>) : launch(rh3::mma_rate_kernel<2>));
  if (ops_out)
    *ops_out = static_cast<double>(sms) * static_cast<double>(groups) * 64.0 * 2.0 * 128.0 * (pattern == 4 ? 128.0 : 256.0) * (kind == 2 ? 16.0 : 32.0);
  return e;
}

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
