// Per-token (row) activation quantizers: abs-max symmetric int8 / fp8-e4m3 with optional fused
// prologues. One CTA owns one row; the row is read ONCE from HBM with 128-bit loads, held in
// registers through the prologue, the abs-max reduction and the quantization, and the codes are
// written once. HBM-bound: algorithmic traffic is 2 bytes in + 1 byte out per element.
//
// Semantics follow the reference's PyTorch emulation exactly (bit-exact codes and scales):
//   int8: s = max(amax/127, 1e-12), q = clamp(round_half_even(x / s), -127, 127)
//   fp8 : s = max(amax/448, 1e-12), q = e4m3_rn(clamp(x / s, -448, 448))
// (reference: custom_nodes/rapid_h3/kernels.py:75-82; fast kernels triton_fp8.py:17-64).
// Prologues (reference: triton_fp8.py:128-148 `_load_act`):
//   KIND_PLAIN   x
//   KIND_SWIGLU  silu(x[:, k]) * x[:, F + k]
//   KIND_NORMMOD rms_norm(x) * w * (1 + scale[idx[row]]) + shift[idx[row]]
//   KIND_HEADS   x given group-major [G, M, gw] (gw = 128: head-major attention output);
//                output column k = group k/gw, channel k%gw
// The division x / s is done as fma(x, 1/s, 1.5 * 2^23) with an exact IEEE re-division only for the rare values
// whose product lands within 2^-14 of a rounding tie (product and rounded quotient are each at most 7.6e-6 away
// from the true quotient), which keeps the codes identical to a true division.
#include "common.cuh"
#include "rapidh3_b200.h"

namespace rh3 {
namespace {

enum { KIND_PLAIN = 0, KIND_SWIGLU = 1, KIND_NORMMOD = 2, KIND_HEADS = 3 };

struct QuantParams {
  const __nv_bfloat16* x;
  int64_t ldx;        // row stride of x in elements (KIND_HEADS: stride between heads)
  int64_t M, K;       // rows, quantized width
  void* q;
  int64_t ldq;
  float* s;
  // KIND_NORMMOD
  const __nv_bfloat16* w;  // may be null
  float eps;
  const int32_t* idx;
  const float* shift;
  const float* scale;
  int64_t ld_tab;
  // KIND_SWIGLU: F == K, the up half starts at column K
  int gw;  // KIND_HEADS: columns per group (128 for one head); x is [K/gw, M, gw] with group stride ldx
  const float* tensor_amax;  // when set: one abs-max for the whole tensor replaces every row's own (per-tensor scale)
};

__device__ __forceinline__ void unpack8(const uint4& u, float* v) {
  v[0] = bf16_lo(u.x); v[1] = bf16_hi(u.x); v[2] = bf16_lo(u.y); v[3] = bf16_hi(u.y);
  v[4] = bf16_lo(u.z); v[5] = bf16_hi(u.z); v[6] = bf16_lo(u.w); v[7] = bf16_hi(u.w);
}

// block-wide max over T threads; result returned to all threads
template <int T>
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int w = 1; w < T / 32; ++w) r = fmaxf(r, red[w]);
  __syncthreads();
  return r;
}
// block-wide sum in a fixed order: xor-butterfly inside each warp, then warps in index order
template <int T>
__device__ __forceinline__ float block_sum_fixed(float v, float* red) {
  v = warp_sum_xor(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int w = 1; w < T / 32; ++w) r = __fadd_rn(r, red[w]);
  __syncthreads();
  return r;
}

// H256 ConvRot rotation of one 256-channel group held by a warp (lane l owns channels 8l..8l+7):
// y = H256 x with H256 = (H4 (x) H4 (x) H4 (x) H4) / 16 and H4 the regular 4x4 Hadamard matrix (all ones except
// a -1 on the anti-diagonal). One radix-4 stage over the four values e0..e3 that differ in one base-4 digit of
// the channel index is, unscaled,
//     y_k = (e_k + e_(k^1)) + (e_(k^2) - e_(k^3))
// i.e. with a = e0+e1, b = e2+e3, c = e0-e1, d = e2-e3:  y0 = a+d, y1 = a-d, y2 = b+c, y3 = b-c.
// Four stages (digit 0 = fastest first), then one multiplication by 1/16. Digit 0 and the low bit of digit 1
// live in the thread, the rest in the lane number; written this way a cross-lane stage costs two shuffles per
// value (the partner of the pair, then the other pair's difference) and the half-in-thread stage one shuffle per
// pair. Every operation is a single rounded fp32 add, so the CPU oracle repeats it bit for bit.
// (reference: triton_fp8.py:70-112 regular_hadamard / _rot256)
__device__ __forceinline__ void rotate256(float* x, int lane) {
  // digit 0: channels j & 3 inside the thread
#pragma unroll
  for (int b = 0; b < 8; b += 4) {
    const float sa = __fadd_rn(x[b], x[b + 1]), sb = __fadd_rn(x[b + 2], x[b + 3]);
    const float dc = __fsub_rn(x[b], x[b + 1]), dd = __fsub_rn(x[b + 2], x[b + 3]);
    x[b] = __fadd_rn(sa, dd), x[b + 1] = __fsub_rn(sa, dd), x[b + 2] = __fadd_rn(sb, dc), x[b + 3] = __fsub_rn(sb, dc);
  }
  // digit 1 = (j >> 2) + 2 * (lane & 1): the pair (e_k, e_(k^1)) is (x[j], x[j+4]); the other pair sits in lane ^ 1
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float t = __fadd_rn(x[j], x[j + 4]);
    const float v = __shfl_xor_sync(0xffffffffu, __fsub_rn(x[j], x[j + 4]), 1);
    x[j] = __fadd_rn(t, v);
    x[j + 4] = __fsub_rn(t, v);
  }
  // digit 2 = (lane >> 1) & 3, digit 3 = lane >> 3: one value per lane
#pragma unroll
  for (int stage = 0; stage < 2; ++stage) {
    const int shift = stage == 0 ? 1 : 3;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float own = x[j];
      const float p1 = __shfl_xor_sync(0xffffffffu, own, 1 << shift);                      // e_(k^1)
      const float v = __shfl_xor_sync(0xffffffffu, __fsub_rn(own, p1), 2 << shift);        // e_(k^2) - e_(k^3)
      x[j] = __fadd_rn(__fadd_rn(own, p1), v);
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) x[j] = __fmul_rn(x[j], 0.0625f);
}

// Issue the 128-bit loads of one row (CPT chunks per thread); nothing waits on them here.
template <int KIND, int T, int CPT>
__device__ __forceinline__ void load_row(const QuantParams& p, int64_t row, int tid, int nchunk, uint4* raw,
                                         uint4* raw2) {
#pragma unroll
  for (int i = 0; i < CPT; ++i) {
    const int c = tid + i * T;
    raw[i] = make_uint4(0, 0, 0, 0);
    if (KIND == KIND_SWIGLU) raw2[i] = make_uint4(0, 0, 0, 0);
    if (c < nchunk) {
      const __nv_bfloat16* src;
      if (KIND == KIND_HEADS) {
        const int col = c << 3;
        const int grp = col / p.gw;
        src = p.x + static_cast<int64_t>(grp) * p.ldx + row * p.gw + (col - grp * p.gw);
      } else {
        src = p.x + row * p.ldx + (static_cast<int64_t>(c) << 3);
      }
      raw[i] = __ldg(reinterpret_cast<const uint4*>(src));
      if (KIND == KIND_SWIGLU) raw2[i] = __ldg(reinterpret_cast<const uint4*>(src + p.K));
    }
  }
}

// One CTA of T threads works on rows blockIdx.x, blockIdx.x + gridDim.x, ...; the loads of the next row
// are issued before the current row is reduced and stored, so every CTA always has a row in flight.
template <int KIND, int OUT_FP8, int T, int CPT, int ROT>
__global__ void __launch_bounds__(T) quant_rows_kernel(const QuantParams p) {
  __shared__ float red[T / 32];
  const int tid = threadIdx.x;
  const int nchunk = static_cast<int>(p.K >> 3);
  uint4 raw[CPT];
  uint4 raw2[KIND == KIND_SWIGLU ? CPT : 1];
  int64_t row = blockIdx.x;
  if (row < p.M) load_row<KIND, T, CPT>(p, row, tid, nchunk, raw, raw2);
  for (; row < p.M; row += gridDim.x) {
  float v[CPT][8];
#pragma unroll
  for (int i = 0; i < CPT; ++i) unpack8(raw[i], v[i]);

  if (KIND == KIND_SWIGLU) {
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
      float u[8];
      unpack8(raw2[i], u);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float g = v[i][j];
        const float sg = __fdiv_rn(1.f, __fadd_rn(1.f, expf(-g)));
        v[i][j] = __fmul_rn(__fmul_rn(g, sg), u[j]);
      }
    }
  }
  // the registers of `raw` are free again: start fetching the next row of this CTA
  if (row + gridDim.x < p.M) load_row<KIND, T, CPT>(p, row + gridDim.x, tid, nchunk, raw, raw2);

  if (KIND == KIND_NORMMOD) {
    // sum of squares in a fixed order (thread-sequential over its chunks, then the block tree)
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = __fadd_rn(ss, __fmul_rn(v[i][j], v[i][j]));
    }
    ss = block_sum_fixed<T>(ss, red);
    const float rstd = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(p.K)), p.eps)));
    const int64_t trow = static_cast<int64_t>(p.idx[row]) * p.ld_tab;
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
      const int c = tid + i * T;
      if (c < nchunk) {
        const int col = c << 3;
        float wv[8];
        if (p.w) {
          unpack8(__ldg(reinterpret_cast<const uint4*>(p.w + col)), wv);
        }
        const float4 sc0 = __ldg(reinterpret_cast<const float4*>(p.scale + trow + col));
        const float4 sc1 = __ldg(reinterpret_cast<const float4*>(p.scale + trow + col + 4));
        const float4 sh0 = __ldg(reinterpret_cast<const float4*>(p.shift + trow + col));
        const float4 sh1 = __ldg(reinterpret_cast<const float4*>(p.shift + trow + col + 4));
        const float sc[8] = {sc0.x, sc0.y, sc0.z, sc0.w, sc1.x, sc1.y, sc1.z, sc1.w};
        const float sh[8] = {sh0.x, sh0.y, sh0.z, sh0.w, sh1.x, sh1.y, sh1.z, sh1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float y = __fmul_rn(v[i][j], rstd);
          if (p.w) y = __fmul_rn(y, wv[j]);
          y = __fadd_rn(__fmul_rn(y, __fadd_rn(1.f, sc[j])), sh[j]);
          v[i][j] = y;
        }
      }
    }
  }

  if (ROT) {
    // chunk c = tid + i * T: the 32 lanes of a warp hold one whole 256-channel group per i
#pragma unroll
    for (int i = 0; i < CPT; ++i)
      if (tid - (tid & 31) + i * T < nchunk) rotate256(v[i], tid & 31);
  }

  // ---- abs-max and scale ----
  float am = 0.f;
#pragma unroll
  for (int i = 0; i < CPT; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(v[i][j]));
  }
  am = p.tensor_amax ? __ldg(p.tensor_amax) : block_max<T>(am, red);
  const float qmax = OUT_FP8 ? 448.f : 127.f;
  const float s = fmaxf(__fdiv_rn(am, qmax), 1e-12f);
  const float inv = __fdiv_rn(1.f, s);
  if (tid == 0) p.s[row] = s;

  // ---- quantize + store ----
  uint8_t* qrow = reinterpret_cast<uint8_t*>(p.q) + row * p.ldq;
#pragma unroll
  for (int i = 0; i < CPT; ++i) {
    const int c = tid + i * T;
    if (c < nchunk) {
      const uint2 o = OUT_FP8 ? quant8_e4m3(v[i], s, inv) : quant8_i8(v[i], s, inv);
      *reinterpret_cast<uint2*>(qrow + (static_cast<int64_t>(c) << 3)) = o;
    }
  }
  }  // rows of this CTA
}

// Second int8 pass on the quantization residual of selected rows (the text encoder's outlier rows):
//   r = rotate(x[rows[i]]) - q1[rows[i]] * s1[rows[i]]   (x fp32, so the residual also carries the bf16 rounding
//   of the first pass's input), then the plain int8 row quantizer on r. One CTA of K/8 threads per selected row.
// (reference: custom_nodes/rapid_h3/te_quant.py:96-105)
template <int T>
__global__ void __launch_bounds__(T) rot_residual_quant_kernel(const float* __restrict__ x, int64_t ldx,
                                                               const int8_t* __restrict__ q1, int64_t ldq1,
                                                               const float* __restrict__ s1,
                                                               const int32_t* __restrict__ rows, int64_t n, int K,
                                                               int8_t* __restrict__ q2, float* __restrict__ s2) {
  __shared__ float red[T / 32];
  const int tid = threadIdx.x;
  const int col = tid << 3;
  const bool active = col < K;
  for (int64_t i = blockIdx.x; i < n; i += gridDim.x) {
    const int64_t r = rows[i];
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    if (active) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(x + r * ldx + col));
      const float4 b = __ldg(reinterpret_cast<const float4*>(x + r * ldx + col + 4));
      v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
    }
    if (tid - (tid & 31) < (K >> 3)) rotate256(v, tid & 31);
    if (active) {
      const uint2 c = __ldg(reinterpret_cast<const uint2*>(q1 + r * ldq1 + col));
      const float sc = s1[r];
      const int8_t* cb = reinterpret_cast<const int8_t*>(&c);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __fsub_rn(v[j], __fmul_rn(static_cast<float>(cb[j]), sc));
    }
    float am = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(v[j]));
    am = block_max<T>(am, red);
    const float s = fmaxf(__fdiv_rn(am, 127.f), 1e-12f);
    const float inv = __fdiv_rn(1.f, s);
    if (tid == 0) s2[i] = s;
    if (active) *reinterpret_cast<uint2*>(q2 + i * K + col) = quant8_i8(v, s, inv);
  }
}

// max |x| over a whole [M, K] bf16 tensor into *out (which the caller zeroed): |x| >= 0, so the float order is the
// order of the bit patterns and one atomicMax on the bits per CTA finishes the reduction, in any order.
__global__ void __launch_bounds__(256) tensor_absmax_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, int64_t M,
                                                            int64_t K, float* __restrict__ out) {
  __shared__ float red[8];
  const int64_t nchunk = K >> 3, total = M * nchunk;
  float am = 0.f;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t row = i / nchunk, c = i - row * nchunk;
    float v[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(x + row * ldx + (c << 3))), v);
#pragma unroll
    for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(v[j]));
  }
  am = block_max<256>(am, red);
  if (threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned int*>(out), __float_as_uint(am));
}

template <int KIND, int OUT_FP8, int ROT = 0>
int launch_quant(const QuantParams& p, cudaStream_t stream) {
  const int64_t nchunk = p.K >> 3;
  if (p.M == 0) return 0;
  // as many CTAs as are resident at once (a multiple of the SM count), each looping over its rows
#define RH3_Q(T_, CPT_)                                                                                \
  do {                                                                                                 \
    auto kern = quant_rows_kernel<KIND, OUT_FP8, T_, CPT_, ROT>;                                       \
    int occ = 1;                                                                                       \
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, T_, 0) != cudaSuccess || occ < 1) occ = 1; \
    const int64_t resident = static_cast<int64_t>(device_sm_count()) * occ;                           \
    kern<<<static_cast<unsigned>(p.M < resident ? p.M : resident), T_, 0, stream>>>(p);               \
  } while (0)
  if (nchunk <= 128) RH3_Q(128, 1);
  else if (nchunk <= 256) RH3_Q(128, 2);
  else if (nchunk <= 512) RH3_Q(128, 4);
  else if (nchunk <= 1024) RH3_Q(128, 8);
  else if (nchunk <= 2048) RH3_Q(256, 8);
  else if (nchunk <= 4096) RH3_Q(512, 8);
  else if (nchunk <= 8192) RH3_Q(1024, 8);
  else return set_error(RH3_ARG_ERROR, "quant_rows: K=%lld is larger than 65536", (long long)p.K);
#undef RH3_Q
  return check_cuda(cudaGetLastError(), "quant_rows launch");
}

int check_common(const void* x, int64_t ldx, int64_t M, int64_t K, const void* q, int64_t ldq, const float* s) {
  RH3_CHECK_ARG(M >= 0 && K > 0, "quant_rows: bad shape M=%lld K=%lld", (long long)M, (long long)K);
  RH3_CHECK_ARG(M < (1ll << 31), "quant_rows: M too large");
  RH3_CHECK_ARG(K % 8 == 0, "quant_rows: K=%lld must be a multiple of 8", (long long)K);
  RH3_CHECK_ARG(M == 0 || (x && q && s), "quant_rows: null pointer");
  RH3_CHECK_ARG(ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0,
                "quant_rows: x must be 16-byte aligned with a row stride that is a multiple of 8 elements");
  RH3_CHECK_ARG(ldq % 8 == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0,
                "quant_rows: q must be 8-byte aligned with a row stride that is a multiple of 8");
  return 0;
}

}  // namespace
}  // namespace rh3

using namespace rh3;

extern "C" int rh3_quant_rows_i8(const void* x, int64_t ldx, int64_t M, int64_t K, void* q, int64_t ldq, float* s,
                                 cudaStream_t stream) {
  if (int e = check_common(x, ldx, M, K, q, ldq, s)) return e;
  RH3_CHECK_ARG(ldx >= K && ldq >= K, "quant_rows_i8: row strides smaller than K");
  QuantParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x); p.ldx = ldx; p.M = M; p.K = K; p.q = q; p.ldq = ldq; p.s = s;
  return launch_quant<KIND_PLAIN, 0>(p, stream);
}

extern "C" int rh3_quant_rows_fp8(const void* x, int64_t ldx, int64_t M, int64_t K, void* q, int64_t ldq, float* s,
                                  cudaStream_t stream) {
  if (int e = check_common(x, ldx, M, K, q, ldq, s)) return e;
  RH3_CHECK_ARG(ldx >= K && ldq >= K, "quant_rows_fp8: row strides smaller than K");
  QuantParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x); p.ldx = ldx; p.M = M; p.K = K; p.q = q; p.ldq = ldq; p.s = s;
  return launch_quant<KIND_PLAIN, 1>(p, stream);
}

extern "C" int rh3_quant_tensor_fp8(const void* x, int64_t ldx, int64_t M, int64_t K, void* q, int64_t ldq, float* s,
                                    float* amax, cudaStream_t stream) {
  if (int e = check_common(x, ldx, M, K, q, ldq, s)) return e;
  RH3_CHECK_ARG(ldx >= K && ldq >= K, "quant_tensor_fp8: row strides smaller than K");
  RH3_CHECK_ARG(amax != nullptr, "quant_tensor_fp8: null abs-max word");
  if (int e = check_cuda(cudaMemsetAsync(amax, 0, sizeof(float), stream), "quant_tensor_fp8 memset")) return e;
  if (M == 0) return 0;
  const int64_t chunks = M * (K >> 3);
  const int64_t want = (chunks + 255) / 256, cap = static_cast<int64_t>(device_sm_count()) * 8;
  tensor_absmax_kernel<<<static_cast<unsigned>(want < cap ? want : cap), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, M, K, amax);
  if (int e = check_cuda(cudaGetLastError(), "tensor_absmax launch")) return e;
  QuantParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x); p.ldx = ldx; p.M = M; p.K = K; p.q = q; p.ldq = ldq; p.s = s;
  p.tensor_amax = amax;
  return launch_quant<KIND_PLAIN, 1>(p, stream);
}

extern "C" int rh3_swiglu_quant_rows_i8(const void* x, int64_t ldx, int64_t M, int64_t F, void* q, int64_t ldq,
                                        float* s, cudaStream_t stream) {
  if (int e = check_common(x, ldx, M, F, q, ldq, s)) return e;
  RH3_CHECK_ARG(ldx >= 2 * F && ldq >= F, "swiglu_quant_rows_i8: row strides too small");
  QuantParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x); p.ldx = ldx; p.M = M; p.K = F; p.q = q; p.ldq = ldq; p.s = s;
  return launch_quant<KIND_SWIGLU, 0>(p, stream);
}

extern "C" int rh3_quant_groups_i8(const void* o, int64_t stride_g, int64_t G, int64_t gw, int64_t M, void* q,
                                   int64_t ldq, float* s, cudaStream_t stream) {
  RH3_CHECK_ARG(G > 0 && gw > 0 && gw % 8 == 0 && gw < (1ll << 30), "quant_groups_i8: G must be positive, gw a multiple of 8");
  if (int e = check_common(o, stride_g, M, G * gw, q, ldq, s)) return e;
  RH3_CHECK_ARG(stride_g >= M * gw && ldq >= G * gw, "quant_groups_i8: strides too small");
  QuantParams p{};
  p.x = static_cast<const __nv_bfloat16*>(o); p.ldx = stride_g; p.M = M; p.K = G * gw; p.q = q; p.ldq = ldq; p.s = s;
  p.gw = static_cast<int>(gw);
  return launch_quant<KIND_HEADS, 0>(p, stream);
}

extern "C" int rh3_quant_heads_i8(const void* o, int64_t stride_h, int64_t H, int64_t M, void* q, int64_t ldq,
                                  float* s, cudaStream_t stream) {
  return rh3_quant_groups_i8(o, stride_h, H, 128, M, q, ldq, s, stream);
}

extern "C" int rh3_norm_mod_quant_rows_i8(const void* x, int64_t ldx, const void* w, float eps, const int32_t* idx,
                                          const float* shift, const float* scale, int64_t ld_tab, int64_t M,
                                          int64_t K, void* q, int64_t ldq, float* s, cudaStream_t stream) {
  if (int e = check_common(x, ldx, M, K, q, ldq, s)) return e;
  RH3_CHECK_ARG(ldx >= K && ldq >= K, "norm_mod_quant_rows_i8: row strides smaller than K");
  RH3_CHECK_ARG(M == 0 || (idx && shift && scale), "norm_mod_quant_rows_i8: null modulation pointer");
  RH3_CHECK_ARG(ld_tab % 4 == 0 && (reinterpret_cast<uintptr_t>(shift) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(scale) & 15) == 0,
                "norm_mod_quant_rows_i8: shift/scale must be 16-byte aligned, row stride a multiple of 4");
  RH3_CHECK_ARG(!w || (reinterpret_cast<uintptr_t>(w) & 15) == 0, "norm_mod_quant_rows_i8: w must be 16-byte aligned");
  QuantParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x); p.ldx = ldx; p.M = M; p.K = K; p.q = q; p.ldq = ldq; p.s = s;
  p.w = static_cast<const __nv_bfloat16*>(w); p.eps = eps; p.idx = idx; p.shift = shift; p.scale = scale;
  p.ld_tab = ld_tab;
  return launch_quant<KIND_NORMMOD, 0>(p, stream);
}

// ---- the same quantizers with the H256 ConvRot rotation applied before the abs-max (K % 256 == 0) ----
#define RH3_ROT_CHECK(K, name) RH3_CHECK_ARG((K) % 256 == 0, name ": the rotated width must be a multiple of 256")

extern "C" int rh3_rot_quant_rows_i8(const void* x, int64_t ldx, int64_t M, int64_t K, void* q, int64_t ldq, float* s,
                                     cudaStream_t stream) {
  if (int e = check_common(x, ldx, M, K, q, ldq, s)) return e;
  RH3_ROT_CHECK(K, "rot_quant_rows_i8");
  RH3_CHECK_ARG(ldx >= K && ldq >= K, "rot_quant_rows_i8: row strides smaller than K");
  QuantParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x); p.ldx = ldx; p.M = M; p.K = K; p.q = q; p.ldq = ldq; p.s = s;
  return launch_quant<KIND_PLAIN, 0, 1>(p, stream);
}

extern "C" int rh3_swiglu_rot_quant_rows_i8(const void* x, int64_t ldx, int64_t M, int64_t F, void* q, int64_t ldq,
                                            float* s, cudaStream_t stream) {
  if (int e = check_common(x, ldx, M, F, q, ldq, s)) return e;
  RH3_ROT_CHECK(F, "swiglu_rot_quant_rows_i8");
  RH3_CHECK_ARG(ldx >= 2 * F && ldq >= F, "swiglu_rot_quant_rows_i8: row strides too small");
  QuantParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x); p.ldx = ldx; p.M = M; p.K = F; p.q = q; p.ldq = ldq; p.s = s;
  return launch_quant<KIND_SWIGLU, 0, 1>(p, stream);
}

extern "C" int rh3_rot_quant_groups_i8(const void* o, int64_t stride_g, int64_t G, int64_t gw, int64_t M, void* q,
                                       int64_t ldq, float* s, cudaStream_t stream) {
  RH3_CHECK_ARG(G > 0 && gw > 0 && gw % 8 == 0 && gw < (1ll << 30), "rot_quant_groups_i8: bad group shape");
  if (int e = check_common(o, stride_g, M, G * gw, q, ldq, s)) return e;
  RH3_ROT_CHECK(G * gw, "rot_quant_groups_i8");
  RH3_CHECK_ARG(stride_g >= M * gw && ldq >= G * gw, "rot_quant_groups_i8: strides too small");
  QuantParams p{};
  p.x = static_cast<const __nv_bfloat16*>(o); p.ldx = stride_g; p.M = M; p.K = G * gw; p.q = q; p.ldq = ldq; p.s = s;
  p.gw = static_cast<int>(gw);
  return launch_quant<KIND_HEADS, 0, 1>(p, stream);
}

extern "C" int rh3_norm_mod_rot_quant_rows_i8(const void* x, int64_t ldx, const void* w, float eps, const int32_t* idx,
                                              const float* shift, const float* scale, int64_t ld_tab, int64_t M,
                                              int64_t K, void* q, int64_t ldq, float* s, cudaStream_t stream) {
  if (int e = check_common(x, ldx, M, K, q, ldq, s)) return e;
  RH3_ROT_CHECK(K, "norm_mod_rot_quant_rows_i8");
  RH3_CHECK_ARG(ldx >= K && ldq >= K, "norm_mod_rot_quant_rows_i8: row strides smaller than K");
  RH3_CHECK_ARG(M == 0 || (idx && shift && scale), "norm_mod_rot_quant_rows_i8: null modulation pointer");
  RH3_CHECK_ARG(ld_tab % 4 == 0 && (reinterpret_cast<uintptr_t>(shift) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(scale) & 15) == 0,
                "norm_mod_rot_quant_rows_i8: shift/scale must be 16-byte aligned, row stride a multiple of 4");
  RH3_CHECK_ARG(!w || (reinterpret_cast<uintptr_t>(w) & 15) == 0, "norm_mod_rot_quant_rows_i8: w must be 16-byte aligned");
  QuantParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x); p.ldx = ldx; p.M = M; p.K = K; p.q = q; p.ldq = ldq; p.s = s;
  p.w = static_cast<const __nv_bfloat16*>(w); p.eps = eps; p.idx = idx; p.shift = shift; p.scale = scale;
  p.ld_tab = ld_tab;
  return launch_quant<KIND_NORMMOD, 0, 1>(p, stream);
}

// ---- residual pass of the text encoder's int8_rot linears (no rotation-free form exists) ----
extern "C" int rh3_rot_residual_quant_rows_i8(const float* x, int64_t ldx, const void* q1, int64_t ldq1, const float* s1,
                                              const int32_t* rows, int64_t n, int64_t K, void* q2, float* s2,
                                              cudaStream_t stream) {
  RH3_CHECK_ARG(n >= 0 && K > 0 && K % 256 == 0 && K <= 8192, "rot_residual_quant: K=%lld must be a multiple of 256, <= 8192",
                (long long)K);
  RH3_CHECK_ARG(ldx >= K && ldx % 4 == 0 && ldq1 >= K && ldq1 % 8 == 0, "rot_residual_quant: bad row strides");
  if (n == 0) return 0;
  RH3_CHECK_ARG(x && q1 && s1 && rows && q2 && s2, "rot_residual_quant: null pointer");
  RH3_CHECK_ARG((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(q1) & 7) == 0 &&
                    (reinterpret_cast<uintptr_t>(q2) & 7) == 0,
                "rot_residual_quant: x must be 16-byte aligned, q1 and q2 8-byte aligned");
  const int64_t threads = K / 8;
  const unsigned grid = static_cast<unsigned>(n < 4 * device_sm_count() ? n : 4 * device_sm_count());
#define RH3_RR(T_)                                                                                       \
  rot_residual_quant_kernel<T_><<<grid, T_, 0, stream>>>(x, ldx, static_cast<const int8_t*>(q1), ldq1, s1, rows, n, \
                                                         (int)K, static_cast<int8_t*>(q2), s2)
  if (threads <= 128) RH3_RR(128);
  else if (threads <= 256) RH3_RR(256);
  else if (threads <= 512) RH3_RR(512);
  else RH3_RR(1024);
#undef RH3_RR
  return check_cuda(cudaGetLastError(), "rot_residual_quant launch");
}
