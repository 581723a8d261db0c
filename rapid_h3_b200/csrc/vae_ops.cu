// Quantizer of the VAE transformer decoder's attention output (fp16 activations).
//
//   o [B, H, S, D] fp16 head-major (D = 64)  ->  q int8 [B*S, H*D], scale fp32 [B*S]
//
// Row (b, s) of the output gathers column c = head * D + d from o[b, head, s, d] (no transposed copy),
// replaces NaN by 0 and +-inf by +-65504 (torch.nan_to_num for fp16), rotates every group of 256 columns
// by the regular-Hadamard matrix H256 and quantizes the row to int8 with one scale:
//   scale = max(min(amax, 65504) * (1/127), 1e-30)
//   q     = clamp(rint(fp16(fp16(y) / fp16(scale))), -128, 127)     (value, scale and quotient pass through fp16)
// The rotation is written as four radix-4 stages with strides 1, 4, 16, 64 and, per stage,
//   y0 = 0.5 * (((x0 + x1) + x2) - x3)      y1 = 0.5 * (((x0 + x1) - x2) + x3)
//   y2 = 0.5 * (((x0 - x1) + x2) + x3)      y3 = 0.5 * (((-x0 + x1) + x2) + x3)
// evaluated left to right in fp32: the order of the reference's vae_out_quant
// (custom_nodes/rapid_h3/csrc/vae_ops.cu:63-142, which restates comfy-kitchen's ConvRot quantizer; the
// reference builds with approximate division, this kernel divides exactly, so the last code bit can differ
// from that binary: parity is defined by the CPU oracle, oracle/vae_ops.py).
//
// One CTA per row at a time (persistent), K / 8 threads, a warp owns one 256-column group: lane l holds
// columns 8l .. 8l+7, i.e. base-4 digits (d0 = j & 3, d1 = (j >> 2) + 2 (l & 1), d2 = (l >> 1) & 3, d3 = l >> 3).
// HBM-bound: 3 bytes per element (2 in, 1 out).
#include "common.cuh"
#include "rapidh3_b200.h"

namespace rh3 {
namespace {

__device__ __forceinline__ float nan_to_num_h(__half h) {
  if (__hisnan(h)) return 0.f;
  if (__hisinf(h)) return __hgt(h, __float2half(0.f)) ? 65504.f : -65504.f;
  return __half2float(h);
}

// one stage: the value at position k (0..3) of the quadruple (e0, e1, e2, e3)
__device__ __forceinline__ float fht_stage(float e0, float e1, float e2, float e3, int k) {
  float r;
  if (k == 0) r = __fsub_rn(__fadd_rn(__fadd_rn(e0, e1), e2), e3);
  else if (k == 1) r = __fadd_rn(__fsub_rn(__fadd_rn(e0, e1), e2), e3);
  else if (k == 2) r = __fadd_rn(__fadd_rn(__fsub_rn(e0, e1), e2), e3);
  else r = __fadd_rn(__fadd_rn(__fsub_rn(e1, e0), e2), e3);  // -x0 + x1 == x1 - x0 exactly
  return 0.5f * r;
}

__device__ __forceinline__ void fht256(float* x, int lane) {
#pragma unroll
  for (int b = 0; b < 8; b += 4) {  // stride 1
    const float e0 = x[b], e1 = x[b + 1], e2 = x[b + 2], e3 = x[b + 3];
#pragma unroll
    for (int k = 0; k < 4; ++k) x[b + k] = fht_stage(e0, e1, e2, e3, k);
  }
  {  // stride 4: positions 0, 1 are x[j], x[j+4] of the even lane, 2, 3 those of the odd lane
    const bool odd = lane & 1;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float u = x[j], w = x[j + 4];
      const float pu = __shfl_xor_sync(0xffffffffu, u, 1), pw = __shfl_xor_sync(0xffffffffu, w, 1);
      const float e0 = odd ? pu : u, e1 = odd ? pw : w, e2 = odd ? u : pu, e3 = odd ? w : pw;
      x[j] = odd ? fht_stage(e0, e1, e2, e3, 2) : fht_stage(e0, e1, e2, e3, 0);
      x[j + 4] = odd ? fht_stage(e0, e1, e2, e3, 3) : fht_stage(e0, e1, e2, e3, 1);
    }
  }
#pragma unroll
  for (int stage = 0; stage < 2; ++stage) {  // strides 16 and 64: one position per lane
    const int shift = stage == 0 ? 1 : 3;
    const int k = (lane >> shift) & 3;
    const int base = lane & ~(3 << shift);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float e0 = __shfl_sync(0xffffffffu, x[j], base);
      const float e1 = __shfl_sync(0xffffffffu, x[j], base | (1 << shift));
      const float e2 = __shfl_sync(0xffffffffu, x[j], base | (2 << shift));
      const float e3 = __shfl_sync(0xffffffffu, x[j], base | (3 << shift));
      x[j] = k == 0 ? fht_stage(e0, e1, e2, e3, 0)
                    : (k == 1 ? fht_stage(e0, e1, e2, e3, 1)
                              : (k == 2 ? fht_stage(e0, e1, e2, e3, 2) : fht_stage(e0, e1, e2, e3, 3)));
    }
  }
}

enum { ACT_NONE = 0, ACT_RMS_NORM = 1, ACT_SWIGLU = 2 };

struct OutQuantParams {
  int act;                // prologue applied to the loaded row before the rotation
  const __half* act_w;    // ACT_RMS_NORM: norm weight [K] or null
  float eps;              // ACT_RMS_NORM
  int64_t up_offset;      // ACT_SWIGLU: the "up" half of a row starts this many elements after the gate half
  const __half* o;
  int8_t* q;
  float* scales;
  int K, D;               // row width and width of one contiguous piece (head)
  int64_t head_stride;    // elements between consecutive D-wide pieces of a row
  int64_t row_stride;     // elements between rows
  int64_t rows;
};

template <int T>
__global__ void __launch_bounds__(T) vae_out_quant_kernel(const OutQuantParams p) {
  __shared__ float red[T / 32];
  const int tid = threadIdx.x;
  const int K = p.K;
  const int col = tid << 3;
  const bool active = col < K;
  const int head = active ? col / p.D : 0;
  const int d = col - head * p.D;
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    float v[8];
    if (active) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p.o + head * p.head_stride + row * p.row_stride + d));
      const __half* h = reinterpret_cast<const __half*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = nan_to_num_h(h[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    }
    if (p.act == ACT_RMS_NORM) {
      // y = (x * r) * w, r = 1 / sqrt(mean(x^2) + eps); the sum of squares in a fixed order: the 8 values of a
      // thread in order, an xor butterfly over the warp, then the warps in order
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = __fadd_rn(ss, __fmul_rn(v[j], v[j]));
      ss = warp_sum_xor(ss);
      if ((tid & 31) == 0) red[tid >> 5] = ss;
      __syncthreads();
      ss = red[0];
#pragma unroll
      for (int w = 1; w < T / 32; ++w) ss = __fadd_rn(ss, red[w]);
      __syncthreads();
      const float r = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(K)), p.eps)));
      if (active) {
        float wv[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
        if (p.act_w) {
          const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p.act_w + col));
          const __half* h = reinterpret_cast<const __half*>(&raw);
#pragma unroll
          for (int j = 0; j < 8; ++j) wv[j] = __half2float(h[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(__fmul_rn(v[j], r), wv[j]);
      }
    } else if (p.act == ACT_SWIGLU) {
      // y = silu(gate) * up with gate = this row's first K values, up = the K values up_offset further on
      if (active) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p.o + head * p.head_stride + row * p.row_stride + d + p.up_offset));
        const __half* h = reinterpret_cast<const __half*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float g = v[j], u = nan_to_num_h(h[j]);
          v[j] = __fmul_rn(__fmul_rn(g, __fdiv_rn(1.f, __fadd_rn(1.f, expf(-g)))), u);
        }
      }
    }
    if (tid - (tid & 31) < (K >> 3)) fht256(v, tid & 31);  // warp-uniform: K is a multiple of 256
    float am = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(v[j]));
    am = warp_max(am);
    if ((tid & 31) == 0) red[tid >> 5] = am;
    __syncthreads();
    am = red[0];
#pragma unroll
    for (int w = 1; w < T / 32; ++w) am = fmaxf(am, red[w]);
    __syncthreads();
    const float scale = fmaxf(__fmul_rn(fminf(am, 65504.f), 1.0f / 127.0f), 1.0e-30f);
    const float scale_h = __half2float(__float2half_rn(scale));
    if (tid == 0) p.scales[row] = scale;
    if (active) {
      uint32_t code[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float vh = __half2float(__float2half_rn(v[j]));
        const float qf = __half2float(__float2half_rn(__fdiv_rn(vh, scale_h)));
        code[j] = static_cast<uint32_t>(static_cast<int>(fminf(127.f, fmaxf(-128.f, rintf(qf)))));
      }
      const uint2 o = make_uint2(pack_low_bytes(code[0], code[1], code[2], code[3]),
                                 pack_low_bytes(code[4], code[5], code[6], code[7]));
      *reinterpret_cast<uint2*>(p.q + row * K + col) = o;
    }
  }
}

template <int T>
int launch_out_quant(const OutQuantParams& p, cudaStream_t stream) {
  auto kern = vae_out_quant_kernel<T>;
  int occ = 1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, T, 0) != cudaSuccess || occ < 1) occ = 1;
  const int64_t resident = static_cast<int64_t>(device_sm_count()) * occ;
  kern<<<static_cast<unsigned>(p.rows < resident ? p.rows : resident), T, 0, stream>>>(p);
  return check_cuda(cudaGetLastError(), "vae_out_quant launch");
}

}  // namespace
}  // namespace rh3

using namespace rh3;

namespace {
int out_quant_launch(const OutQuantParams& p, cudaStream_t stream) {
  const int64_t threads = p.K / 8;
  if (threads <= 128) return launch_out_quant<128>(p, stream);
  if (threads <= 256) return launch_out_quant<256>(p, stream);
  if (threads <= 512) return launch_out_quant<512>(p, stream);
  return launch_out_quant<1024>(p, stream);
}
}  // namespace

extern "C" int rh3_vae_out_quant(const void* o_f16, int64_t B, int64_t H, int64_t S, int64_t D, void* q, float* scales,
                                 cudaStream_t stream) {
  RH3_CHECK_ARG(B >= 0 && H > 0 && S >= 0 && D > 0 && D % 8 == 0, "vae_out_quant: bad shape B=%lld H=%lld S=%lld D=%lld",
                (long long)B, (long long)H, (long long)S, (long long)D);
  const int64_t K = H * D;
  RH3_CHECK_ARG(K % 256 == 0 && 256 % D == 0, "vae_out_quant: H*D must be a multiple of 256 and D must divide 256");
  RH3_CHECK_ARG(K <= 8192, "vae_out_quant: row width %lld is larger than 8192", (long long)K);
  RH3_CHECK_ARG(B * S < (1ll << 31), "vae_out_quant: too many rows");
  if (B == 0 || S == 0) return 0;
  RH3_CHECK_ARG(o_f16 && q && scales, "vae_out_quant: null pointer");
  RH3_CHECK_ARG((reinterpret_cast<uintptr_t>(o_f16) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0,
                "vae_out_quant: o must be 16-byte aligned and q 8-byte aligned");
  for (int64_t b = 0; b < B; ++b) {
    OutQuantParams p{};
    p.o = static_cast<const __half*>(o_f16) + b * H * S * D;
    p.q = static_cast<int8_t*>(q) + b * S * K;
    p.scales = scales + b * S;
    p.K = (int)K; p.D = (int)D; p.head_stride = S * D; p.row_stride = D; p.rows = S;
    if (int e = out_quant_launch(p, stream)) return e;
  }
  return 0;
}

// The same row arithmetic on a row-major fp16 matrix x [M, K] (row stride ldx): the quantizer the decoder's linears
// call on their inputs (vae_fast._quantize, custom_nodes/rapid_h3/vae_fast.py:71-85).
extern "C" int rh3_vae_quant_rows(const void* x_f16, int64_t ldx, int64_t M, int64_t K, void* q, float* scales,
                                  cudaStream_t stream) {
  RH3_CHECK_ARG(M >= 0 && K > 0 && K % 256 == 0 && K <= 8192, "vae_quant_rows: K=%lld must be a multiple of 256, <= 8192",
                (long long)K);
  RH3_CHECK_ARG(M < (1ll << 31) && ldx >= K && ldx % 8 == 0, "vae_quant_rows: bad M or row stride");
  if (M == 0) return 0;
  RH3_CHECK_ARG(x_f16 && q && scales, "vae_quant_rows: null pointer");
  RH3_CHECK_ARG((reinterpret_cast<uintptr_t>(x_f16) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0,
                "vae_quant_rows: x must be 16-byte aligned and q 8-byte aligned");
  OutQuantParams p{};
  p.o = static_cast<const __half*>(x_f16);
  p.q = static_cast<int8_t*>(q);
  p.scales = scales;
  p.K = (int)K; p.D = 256; p.head_stride = 256; p.row_stride = ldx; p.rows = M;
  return out_quant_launch(p, stream);
}

// The quantizer with a fused activation prologue (the `act` argument of the quantizer the reference calls in
// vae_fast._quantize, vae_fast.py:71-85: "rms_norm" for the inputs of to_qkv and w1, "swiglu" for the input of w2
// when the SwiGLU is not in w1's epilogue). act 1: x [M, K], y = (x * r) * weight (fp16 [K] or NULL),
// r = 1 / sqrt(mean(x^2) + eps); act 2: x [M, 2K] = [gate | up], y = gate / (1 + e^-gate) * up. y stays fp32 into
// the rotation. The per-row arithmetic of that fused form lives in a third-party binary (comfy-kitchen) whose source
// is not part of the reference repository; this entry defines it with IEEE operations (CPU oracle: oracle/vae_ops.py).
extern "C" int rh3_vae_quant_rows_act(const void* x_f16, int64_t ldx, int64_t M, int64_t K, int act,
                                      const void* act_weight_f16, float eps, void* q, float* scales,
                                      cudaStream_t stream) {
  RH3_CHECK_ARG(act == ACT_RMS_NORM || act == ACT_SWIGLU, "vae_quant_rows_act: act must be 1 (rms_norm) or 2 (swiglu)");
  RH3_CHECK_ARG(M >= 0 && K > 0 && K % 256 == 0 && K <= 8192, "vae_quant_rows_act: K=%lld must be a multiple of 256, <= 8192",
                (long long)K);
  RH3_CHECK_ARG(M < (1ll << 31) && ldx >= (act == ACT_SWIGLU ? 2 * K : K) && ldx % 8 == 0,
                "vae_quant_rows_act: bad M or row stride");
  if (M == 0) return 0;
  RH3_CHECK_ARG(x_f16 && q && scales, "vae_quant_rows_act: null pointer");
  RH3_CHECK_ARG((reinterpret_cast<uintptr_t>(x_f16) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0 &&
                    (reinterpret_cast<uintptr_t>(act_weight_f16) & 15) == 0,
                "vae_quant_rows_act: x and the norm weight must be 16-byte aligned and q 8-byte aligned");
  OutQuantParams p{};
  p.act = act;
  p.act_w = act == ACT_RMS_NORM ? static_cast<const __half*>(act_weight_f16) : nullptr;
  p.eps = eps;
  p.up_offset = K;
  p.o = static_cast<const __half*>(x_f16);
  p.q = static_cast<int8_t*>(q);
  p.scales = scales;
  p.K = (int)K; p.D = 256; p.head_stride = 256; p.row_stride = ldx; p.rows = M;
  return out_quant_launch(p, stream);
}
