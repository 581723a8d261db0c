// Attention pre-pass kernels (all HBM-bound, one pass over their inputs each):
//
//   rh3_rmsnorm_rope3d      per-(token, head) RMSNorm over 128 channels + split-half partial 3-D RoPE
//                           (rot_dim 96 = 3 axes x 16 frequencies x 2; pairs (i, i+48); channels
//                           96..127 are normalised only); bf16 in, bf16 out, token-local.
//   rh3_attn_kv_stats       per-(head, channel) K mean (smoothing), V mean and V scale, with a
//                           deterministic two-level sum: 256-token chunks, then chunks in order.
//   rh3_attn_quant_qk       int8 codes with ONE abs-max scale per 64-token block per head
//                           (K after subtracting the per-head channel mean), laid out [H][Lpad][128].
//   rh3_attn_quant_v        V - mean -> fp8 e4m3 with one scale per (head, channel), transposed to
//                           [H][128][Lpad] so that keys are the contiguous (K-major) axis of P.V.
//
// Reference for the arithmetic: custom_nodes/rapid_h3/csrc/attn_int8.cu:82-109 (stats_partial /
// stats_final), :130-170 (quant_qk), :217-260 (rms_rope_row), :404-443 (per-block K scale),
// :452-496 (quant_v incl. its e4m3 branch) and the error-emulation script bench/attn_emulate.py:10-23
// (`q8(x, 1, 64)`, `f8(x, 0)`). Differences that are deliberate: IEEE division/sqrt instead of the
// .approx.ftz forms (the CPU oracle must be able to reproduce every bit), block-64 scales and an
// e4m3 V scaled to 448 by its own abs-max.
#include <atomic>

#include "common.cuh"
#include "rapidh3_b200.h"

namespace rh3 {
namespace {

constexpr int D = 128;
constexpr int STAT_CHUNK = 256;

__device__ __forceinline__ void load4(const __nv_bfloat16* p, float* x) {
  const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
  x[0] = bf16_lo(raw.x); x[1] = bf16_hi(raw.x); x[2] = bf16_lo(raw.y); x[3] = bf16_hi(raw.y);
}

// ---------------------------------------------------------------------------------------------
// RMSNorm + 3-D RoPE. One warp per (token, head) row; lane l owns channels 4l..4l+3.
// ---------------------------------------------------------------------------------------------
// The rope-table words of one token for this lane (lanes 0..23 hold pair indices 4*(lane % 12) .. +3).
__device__ __forceinline__ void load_rope_words(const __nv_bfloat16* __restrict__ tab_row, int lane, uint32_t* tw) {
  if (tab_row != nullptr && lane < 24) {
    const int i0 = (lane < 12 ? lane : lane - 12) * 4;  // index of the pair in the table row
    const __nv_bfloat16* t = tab_row + i0 * 4;
    const uint4 t0 = __ldg(reinterpret_cast<const uint4*>(t));
    const uint4 t1 = __ldg(reinterpret_cast<const uint4*>(t + 8));
    tw[0] = t0.x, tw[1] = t0.y, tw[2] = t0.z, tw[3] = t0.w, tw[4] = t1.x, tw[5] = t1.y, tw[6] = t1.z, tw[7] = t1.w;
  }
}

// RMSNorm + rope of the four channels lane*4..lane*4+3 of one (token, head) row given its values, the norm weights
// of those channels and the token's rope words; returns the packed bf16 result.
__device__ __forceinline__ uint2 rmsnorm_rope_vals(const float* v, const float* wv, float eps, const uint32_t* tw,
                                                   bool has_tab, int lane) {
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) ss = __fadd_rn(ss, __fmul_rn(v[j], v[j]));
  ss = warp_sum_xor(ss);
  const float r = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, 128.f), eps)));
  float n[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) n[j] = bf16_round(__fmul_rn(__fmul_rn(r, v[j]), wv[j]));
  float o[4] = {n[0], n[1], n[2], n[3]};
  if (has_tab) {
    // partner lane holds the other half of the rotary pair (channels +-48 = 12 lanes away)
    const int partner = lane < 12 ? lane + 12 : (lane < 24 ? lane - 12 : lane);
    float pn[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) pn[j] = __shfl_sync(0xffffffffu, n[j], partner);
    if (lane < 24) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float t00 = bf16_lo(tw[2 * j]), t01 = bf16_hi(tw[2 * j]);
        const float t10 = bf16_lo(tw[2 * j + 1]), t11 = bf16_hi(tw[2 * j + 1]);
        const float a = lane < 12 ? n[j] : pn[j];
        const float b = lane < 12 ? pn[j] : n[j];
        o[j] = lane < 12 ? bf16_round(__fadd_rn(__fmul_rn(a, t00), __fmul_rn(b, t01)))
                         : bf16_round(__fadd_rn(__fmul_rn(a, t10), __fmul_rn(b, t11)));
      }
    }
  }
  return make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
}

__device__ __forceinline__ uint2 rmsnorm_rope_row(const __nv_bfloat16* __restrict__ xrow,
                                                  const __nv_bfloat16* __restrict__ w, float eps,
                                                  const __nv_bfloat16* __restrict__ tab_row, int lane) {
  float v[4], wv[4];
  uint32_t tw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  load4(xrow + lane * 4, v);
  load4(w + lane * 4, wv);
  load_rope_words(tab_row, lane, tw);
  return rmsnorm_rope_vals(v, wv, eps, tw, tab_row != nullptr, lane);
}

// One warp per (token, group of HG consecutive heads): the token's rope words and the norm weights are loaded
// once and the HG rows' loads are issued together. HG = 4 when H is a multiple of 4, else 1.
template <int HG>
__global__ void __launch_bounds__(256) rmsnorm_rope_kernel(const __nv_bfloat16* __restrict__ x, int64_t x_ss,
                                                           int64_t x_sh, __nv_bfloat16* __restrict__ y, int64_t y_ss,
                                                           int64_t y_sh, int64_t S, int H,
                                                           const __nv_bfloat16* __restrict__ w, float eps,
                                                           const __nv_bfloat16* __restrict__ tab) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = H / HG;
  const int64_t g = static_cast<int64_t>(blockIdx.x) * 8 + warp;
  if (g >= S * groups) return;
  const int64_t s = g / groups;
  const int h0 = static_cast<int>(g - s * groups) * HG;
  float v[HG][4], wv[4];
  uint32_t tw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
  for (int i = 0; i < HG; ++i) load4(x + s * x_ss + (h0 + i) * x_sh + lane * 4, v[i]);
  load4(w + lane * 4, wv);
  load_rope_words(tab ? tab + s * 48 * 4 : nullptr, lane, tw);
#pragma unroll
  for (int i = 0; i < HG; ++i) {
    const uint2 o = rmsnorm_rope_vals(v[i], wv, eps, tw, tab != nullptr, lane);
    *reinterpret_cast<uint2*>(y + s * y_ss + (h0 + i) * y_sh + lane * 4) = o;
  }
}

// ---------------------------------------------------------------------------------------------
// Sequence-parallel form: RMSNorm + RoPE of q and k fused with the token -> head exchange. The qkv rows of
// this rank's tokens are normalised, rotated and stored straight into the buffer of the rank that owns the
// head (its own memory or a peer's over NVLink): dst[r] is [total tokens, 3, (H/P)*128] on rank r, row0 is
// the global index of this rank's first token. Plain stores only; ordering against the readers is the
// caller's stream-ordered barrier. One warp per (token, head): q row, k row, v row (copied unchanged).
// ---------------------------------------------------------------------------------------------
struct ScatterDst {
  __nv_bfloat16* ptr[8];
};

__global__ void __launch_bounds__(256) rope_scatter_kernel(const __nv_bfloat16* __restrict__ qkv, int64_t ld, int64_t S,
                                                           int H, int heads_per_rank, int64_t row0,
                                                           const __nv_bfloat16* __restrict__ qw,
                                                           const __nv_bfloat16* __restrict__ kw, float eps,
                                                           const __nv_bfloat16* __restrict__ tab, const ScatterDst dst) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t g = static_cast<int64_t>(blockIdx.x) * 8 + warp;
  if (g >= S * H) return;
  const int64_t s = g / H;
  const int h = static_cast<int>(g - s * H);
  const int r = h / heads_per_rank, hh = h - r * heads_per_rank;
  const int64_t w = static_cast<int64_t>(heads_per_rank) * D;
  const __nv_bfloat16* row = qkv + s * ld + h * D;
  const __nv_bfloat16* tab_row = tab ? tab + s * 48 * 4 : nullptr;
  __nv_bfloat16* out = dst.ptr[r] + (row0 + s) * 3 * w + hh * D + lane * 4;
  const int64_t hd = static_cast<int64_t>(H) * D;
  float qv[4], kv[4], qwv[4], kwv[4];
  uint32_t tw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  load4(row + lane * 4, qv);
  load4(row + hd + lane * 4, kv);
  const uint2 vo = __ldg(reinterpret_cast<const uint2*>(row + 2 * hd + lane * 4));
  load4(qw + lane * 4, qwv);
  load4(kw + lane * 4, kwv);
  load_rope_words(tab_row, lane, tw);  // q and k of a token share its rope words
  const uint2 qo = rmsnorm_rope_vals(qv, qwv, eps, tw, tab_row != nullptr, lane);
  const uint2 ko = rmsnorm_rope_vals(kv, kwv, eps, tw, tab_row != nullptr, lane);
  *reinterpret_cast<uint2*>(out) = qo;
  *reinterpret_cast<uint2*>(out + w) = ko;
  *reinterpret_cast<uint2*>(out + 2 * w) = vo;
}

// ---------------------------------------------------------------------------------------------
// K/V statistics. Pass 1: one warp per (head, 256-token chunk), tokens in order. The partials are
// scratch: part[(h * nchunk + c) * 4 * 128 + {ksum, vsum, vmax, vmin} * 128 + channel].
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) kv_stats_partial_kernel(const __nv_bfloat16* __restrict__ K, int64_t k_ss,
                                                               int64_t k_sh, const __nv_bfloat16* __restrict__ V,
                                                               int64_t v_ss, int64_t v_sh, int64_t L, int H,
                                                               int nchunk, float* __restrict__ part) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x * 8 + warp, c = blockIdx.y;
  if (h >= H) return;
  const int64_t s0 = static_cast<int64_t>(c) * STAT_CHUNK;
  const int64_t s1 = s0 + STAT_CHUNK < L ? s0 + STAT_CHUNK : L;
  float ks[4] = {0.f, 0.f, 0.f, 0.f}, vs[4] = {0.f, 0.f, 0.f, 0.f};
  float vmx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}, vmn[4] = {INFINITY, INFINITY, INFINITY, INFINITY};
  for (int64_t s = s0; s < s1; ++s) {
    float kv[4], vv[4];
    load4(K + s * k_ss + h * k_sh + lane * 4, kv);
    load4(V + s * v_ss + h * v_sh + lane * 4, vv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ks[i] = __fadd_rn(ks[i], kv[i]);
      vs[i] = __fadd_rn(vs[i], vv[i]);
      vmx[i] = fmaxf(vmx[i], vv[i]);
      vmn[i] = fminf(vmn[i], vv[i]);
    }
  }
  float* p = part + (static_cast<int64_t>(h) * nchunk + c) * 4 * D + lane * 4;
  *reinterpret_cast<float4*>(p) = make_float4(ks[0], ks[1], ks[2], ks[3]);
  *reinterpret_cast<float4*>(p + D) = make_float4(vs[0], vs[1], vs[2], vs[3]);
  *reinterpret_cast<float4*>(p + 2 * D) = make_float4(vmx[0], vmx[1], vmx[2], vmx[3]);
  *reinterpret_cast<float4*>(p + 3 * D) = make_float4(vmn[0], vmn[1], vmn[2], vmn[3]);
}

// Pass 2: one thread per (head, channel), chunks in order.
__global__ void __launch_bounds__(128) kv_stats_final_kernel(const float* __restrict__ part, int nchunk, int64_t L,
                                                             float* __restrict__ kmean, float* __restrict__ vmean,
                                                             float* __restrict__ vscale) {
  const int h = blockIdx.x, d = threadIdx.x;
  const float* p = part + static_cast<int64_t>(h) * nchunk * 4 * D + d;
  float ks = 0.f, vs = 0.f, vmx = -INFINITY, vmn = INFINITY;
  for (int c = 0; c < nchunk; ++c) {
    ks = __fadd_rn(ks, p[0]);
    vs = __fadd_rn(vs, p[D]);
    vmx = fmaxf(vmx, p[2 * D]);
    vmn = fminf(vmn, p[3 * D]);
    p += 4 * D;
  }
  const float fl = static_cast<float>(L);
  const float km = __fdiv_rn(ks, fl), vm = __fdiv_rn(vs, fl);
  kmean[h * D + d] = km;
  vmean[h * D + d] = vm;
  const float am = fmaxf(__fsub_rn(vmx, vm), __fsub_rn(vm, vmn));
  vscale[h * D + d] = __fdiv_rn(fmaxf(am, 1e-8f), 448.f);
}

// ---------------------------------------------------------------------------------------------
// Q/K block-64 int8. One CTA per (64-token block, head); 8 warps x 8 tokens, lane = 4 channels.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quant_block64_kernel(const __nv_bfloat16* __restrict__ X, int64_t x_ss,
                                                            int64_t x_sh, int64_t L, int64_t Lpad,
                                                            const float* __restrict__ mean,  // [H][128] or null
                                                            int8_t* __restrict__ out, float* __restrict__ scales) {
  __shared__ float red[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y;
  const int64_t blk = blockIdx.x;
  float m[4] = {0.f, 0.f, 0.f, 0.f};
  if (mean) {
    const float4 mm = *reinterpret_cast<const float4*>(mean + h * D + lane * 4);
    m[0] = mm.x; m[1] = mm.y; m[2] = mm.z; m[3] = mm.w;
  }
  float v[8][4];
  float am = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t s = blk * 64 + warp * 8 + i;
    if (s < L) {
      load4(X + s * x_ss + h * x_sh + lane * 4, v[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[i][j] = __fsub_rn(v[i][j], m[j]);
        am = fmaxf(am, fabsf(v[i][j]));
      }
    } else {
      v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f;
    }
  }
  am = warp_max(am);
  if (lane == 0) red[warp] = am;
  __syncthreads();
  am = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) am = fmaxf(am, red[w]);
  const float sc = __fdiv_rn(fmaxf(am, 1e-8f), 127.f);
  const float inv = __fdiv_rn(1.f, sc);
  if (threadIdx.x == 0) scales[static_cast<int64_t>(h) * (Lpad / 64) + blk] = sc;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t s = blk * 64 + warp * 8 + i;
    const uint32_t packed = pack_low_bytes(quant_code_i8(v[i][0], sc, inv), quant_code_i8(v[i][1], sc, inv),
                                           quant_code_i8(v[i][2], sc, inv), quant_code_i8(v[i][3], sc, inv));
    *reinterpret_cast<uint32_t*>(out + (static_cast<int64_t>(h) * Lpad + s) * D + lane * 4) = packed;
  }
}

// ---------------------------------------------------------------------------------------------
// V -> e4m3, transposed. One CTA per (128-token tile, head).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quant_v_kernel(const __nv_bfloat16* __restrict__ V, int64_t v_ss, int64_t v_sh,
                                                      int64_t L, int64_t Lpad, const float* __restrict__ vmean,
                                                      const float* __restrict__ vscale, uint8_t* __restrict__ Vt) {
  constexpr int T = 128, P = D + 4;  // tile[token][channel], padded rows
  __shared__ uint8_t tile[T * P];
  const int h = blockIdx.y, tid = threadIdx.x;
  const int64_t s0 = static_cast<int64_t>(blockIdx.x) * T;
  for (int i = tid; i < T * (D / 4); i += 256) {
    const int r = i / (D / 4), c4 = (i % (D / 4)) * 4;
    const int64_t s = s0 + r;
    uint32_t packed = 0;
    if (s < L) {
      float x[4];
      load4(V + s * v_ss + h * v_sh + c4, x);
      const float4 m = *reinterpret_cast<const float4*>(vmean + h * D + c4);
      const float4 sc = *reinterpret_cast<const float4*>(vscale + h * D + c4);
      const float mm[4] = {m.x, m.y, m.z, m.w}, ss[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        packed |= quant_code_e4m3(__fsub_rn(x[j], mm[j]), ss[j], __fdiv_rn(1.f, ss[j])) << (8 * j);
    }
    *reinterpret_cast<uint32_t*>(&tile[r * P + c4]) = packed;
  }
  __syncthreads();
  // write: channel d, 16 consecutive tokens per 16-byte store
  for (int i = tid; i < D * (T / 16); i += 256) {
    const int d = i / (T / 16), cc = (i % (T / 16)) * 16;
    alignas(16) uint8_t o[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j] = tile[(cc + j) * P + d];
    *reinterpret_cast<uint4*>(Vt + (static_cast<int64_t>(h) * D + d) * Lpad + s0 + cc) = *reinterpret_cast<uint4*>(o);
  }
}

bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

}  // namespace
}  // namespace rh3

using namespace rh3;

extern "C" int rh3_rmsnorm_rope3d(const void* x, int64_t x_ss, int64_t x_sh, void* y, int64_t y_ss, int64_t y_sh,
                                  int64_t S, int64_t H, const void* weight, float eps, const void* rope_table,
                                  cudaStream_t stream) {
  RH3_CHECK_ARG(S >= 0 && H > 0 && H < 65536, "rmsnorm_rope3d: bad shape S=%lld H=%lld", (long long)S, (long long)H);
  if (S == 0) return 0;
  RH3_CHECK_ARG(x && y && weight, "rmsnorm_rope3d: null pointer");
  RH3_CHECK_ARG(aligned(x, 8) && aligned(y, 8) && aligned(weight, 8) && x_ss % 4 == 0 && x_sh % 4 == 0 &&
                    y_ss % 4 == 0 && y_sh % 4 == 0,
                "rmsnorm_rope3d: rows must be 8-byte aligned (strides multiples of 4 elements)");
  RH3_CHECK_ARG(!rope_table || aligned(rope_table, 16), "rmsnorm_rope3d: rope table must be 16-byte aligned");
  const int hg = H % 4 == 0 ? 4 : 1;
  const int64_t warps = S * (H / hg);
  RH3_CHECK_ARG((warps + 7) / 8 < (1ll << 31), "rmsnorm_rope3d: too many rows");
  const unsigned grid = static_cast<unsigned>((warps + 7) / 8);
  const auto* xp = static_cast<const __nv_bfloat16*>(x);
  auto* yp = static_cast<__nv_bfloat16*>(y);
  const auto* wp = static_cast<const __nv_bfloat16*>(weight);
  const auto* tp = static_cast<const __nv_bfloat16*>(rope_table);
  if (hg == 4) rmsnorm_rope_kernel<4><<<grid, 256, 0, stream>>>(xp, x_ss, x_sh, yp, y_ss, y_sh, S, (int)H, wp, eps, tp);
  else rmsnorm_rope_kernel<1><<<grid, 256, 0, stream>>>(xp, x_ss, x_sh, yp, y_ss, y_sh, S, (int)H, wp, eps, tp);
  return check_cuda(cudaGetLastError(), "rmsnorm_rope3d launch");
}

extern "C" int rh3_rope_scatter_heads(const void* qkv, int64_t ld, int64_t S, int64_t H, int64_t P, int64_t row0,
                                      const void* q_weight, const void* k_weight, float eps, const void* rope_table,
                                      void* const* dst, cudaStream_t stream) {
  RH3_CHECK_ARG(S >= 0 && H > 0 && H < 65536 && P > 0 && P <= 8 && H % P == 0 && row0 >= 0,
                "rope_scatter_heads: bad shape S=%lld H=%lld P=%lld", (long long)S, (long long)H, (long long)P);
  if (S == 0) return 0;
  RH3_CHECK_ARG(qkv && q_weight && k_weight && dst, "rope_scatter_heads: null pointer");
  RH3_CHECK_ARG(aligned(qkv, 8) && aligned(q_weight, 8) && aligned(k_weight, 8) && ld % 4 == 0 && ld >= 3 * H * D,
                "rope_scatter_heads: rows must be 8-byte aligned and hold q | k | v");
  RH3_CHECK_ARG(!rope_table || aligned(rope_table, 16), "rope_scatter_heads: rope table must be 16-byte aligned");
  ScatterDst d{};
  for (int r = 0; r < P; ++r) {
    RH3_CHECK_ARG(dst[r] && aligned(dst[r], 8), "rope_scatter_heads: destination %d is null or misaligned", r);
    d.ptr[r] = static_cast<__nv_bfloat16*>(dst[r]);
  }
  const int64_t rows = S * H;
  RH3_CHECK_ARG((rows + 7) / 8 < (1ll << 31), "rope_scatter_heads: too many rows");
  rope_scatter_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(qkv), ld, S, (int)H, (int)(H / P), row0,
      static_cast<const __nv_bfloat16*>(q_weight), static_cast<const __nv_bfloat16*>(k_weight), eps,
      static_cast<const __nv_bfloat16*>(rope_table), d);
  return check_cuda(cudaGetLastError(), "rope_scatter_heads launch");
}

extern "C" int64_t rh3_attn_kv_stats_scratch_bytes(int64_t L, int64_t H) {
  const int64_t nchunk = (L + STAT_CHUNK - 1) / STAT_CHUNK;
  return H * nchunk * 4 * D * static_cast<int64_t>(sizeof(float));
}

extern "C" int rh3_attn_kv_stats(const void* k, int64_t k_ss, int64_t k_sh, const void* v, int64_t v_ss, int64_t v_sh,
                                 int64_t L, int64_t H, void* scratch, int64_t scratch_bytes, float* kmean,
                                 float* vmean, float* vscale, cudaStream_t stream) {
  RH3_CHECK_ARG(L > 0 && H > 0 && H < 65536, "attn_kv_stats: bad shape L=%lld H=%lld", (long long)L, (long long)H);
  RH3_CHECK_ARG(k && v && scratch && kmean && vmean && vscale, "attn_kv_stats: null pointer");
  RH3_CHECK_ARG(scratch_bytes >= rh3_attn_kv_stats_scratch_bytes(L, H), "attn_kv_stats: scratch too small (%lld < %lld)",
                (long long)scratch_bytes, (long long)rh3_attn_kv_stats_scratch_bytes(L, H));
  RH3_CHECK_ARG(aligned(k, 8) && aligned(v, 8) && aligned(scratch, 16) && k_ss % 4 == 0 && k_sh % 4 == 0 &&
                    v_ss % 4 == 0 && v_sh % 4 == 0,
                "attn_kv_stats: misaligned input");
  const int nchunk = static_cast<int>((L + STAT_CHUNK - 1) / STAT_CHUNK);
  RH3_CHECK_ARG(nchunk < 65536, "attn_kv_stats: L too large");
  kv_stats_partial_kernel<<<dim3(static_cast<unsigned>((H + 7) / 8), nchunk), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(k), k_ss, k_sh, static_cast<const __nv_bfloat16*>(v), v_ss, v_sh, L, (int)H,
      nchunk, static_cast<float*>(scratch));
  if (int e = check_cuda(cudaGetLastError(), "attn_kv_stats partial launch")) return e;
  kv_stats_final_kernel<<<static_cast<unsigned>(H), 128, 0, stream>>>(static_cast<const float*>(scratch), nchunk, L,
                                                                      kmean, vmean, vscale);
  return check_cuda(cudaGetLastError(), "attn_kv_stats final launch");
}

// ---------------------------------------------------------------------------------------------
// Allocation-free K/V statistics.
//
// Some hosts of this library may not create device memory at the moment they need the statistics:
// a sampler loop running under a framework that has already handed every byte of VRAM to its own
// pool, a latency-critical serving thread where cudaMalloc (which synchronises the device) is
// banned, or a plugin that is only ever given input and output buffers. For them the chunk
// partials live in a fixed array inside the library's device image instead of caller scratch.
// The array costs 16 MiB on every GPU that loads the library, for the life of the process.
//
// Host code cannot use `g_kv_stats_scratch` as a pointer: on the host that name is only a handle
// for the symbol. The real device address is looked up once per device, with that device current,
// through cudaGetSymbolAddress, and that address is what the kernels receive.
// ---------------------------------------------------------------------------------------------
constexpr int64_t KV_STATS_NOALLOC_MAX_UNITS = 8192;  // limit on H * ceil(L / 256)
static __device__ __align__(256) float g_kv_stats_scratch[KV_STATS_NOALLOC_MAX_UNITS * 4 * 128];

static int kv_stats_scratch_address(float** out) {
  // Filled on the first call per device. Host threads that race here each look the address up and store the same
  // value; the entries are atomics so that such a race is well defined.
  static std::atomic<float*> per_device[64] = {};
  int dev = -1;
  if (int e = rh3::check_cuda(cudaGetDevice(&dev), "attn_kv_stats_noalloc: cudaGetDevice")) return e;
  if (dev < 0 || dev >= 64) return rh3::set_error(RH3_ARG_ERROR, "attn_kv_stats_noalloc: device index %d out of range", dev);
  float* addr = per_device[dev].load(std::memory_order_acquire);
  if (addr == nullptr) {
    void* p = nullptr;
    if (int e = rh3::check_cuda(cudaGetSymbolAddress(&p, g_kv_stats_scratch),
                                "attn_kv_stats_noalloc: cudaGetSymbolAddress"))
      return e;
    addr = static_cast<float*>(p);
    per_device[dev].store(addr, std::memory_order_release);
  }
  *out = addr;
  return 0;
}

extern "C" int rh3_attn_kv_stats_noalloc(const void* k, int64_t k_ss, int64_t k_sh, const void* v, int64_t v_ss,
                                         int64_t v_sh, int64_t L, int64_t H, float* kmean, float* vmean,
                                         float* vscale, cudaStream_t stream) {
  RH3_CHECK_ARG(L > 0 && H > 0 && H < 65536, "attn_kv_stats_noalloc: bad shape L=%lld H=%lld", (long long)L,
                (long long)H);
  const int64_t nchunk64 = (L + STAT_CHUNK - 1) / STAT_CHUNK;
  RH3_CHECK_ARG(H * nchunk64 <= KV_STATS_NOALLOC_MAX_UNITS,
                "attn_kv_stats_noalloc: H * ceil(L/256) = %lld exceeds the built-in scratch limit of %lld; "
                "use rh3_attn_kv_stats with caller-provided scratch",
                (long long)(H * nchunk64), (long long)KV_STATS_NOALLOC_MAX_UNITS);
  RH3_CHECK_ARG(k && v && kmean && vmean && vscale, "attn_kv_stats_noalloc: null pointer");
  RH3_CHECK_ARG(aligned(k, 8) && aligned(v, 8) && k_ss % 4 == 0 && k_sh % 4 == 0 && v_ss % 4 == 0 && v_sh % 4 == 0,
                "attn_kv_stats_noalloc: misaligned input");
  float* scratch = nullptr;
  if (int e = kv_stats_scratch_address(&scratch)) return e;
  const int nchunk = static_cast<int>(nchunk64);
  // every partial that the second kernel reads is written by the first one in this call, so nothing
  // left over from an earlier call needs clearing
  kv_stats_partial_kernel<<<dim3(static_cast<unsigned>((H + 7) / 8), nchunk), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(k), k_ss, k_sh, static_cast<const __nv_bfloat16*>(v), v_ss, v_sh, L, (int)H,
      nchunk, scratch);
  if (int e = check_cuda(cudaGetLastError(), "attn_kv_stats_noalloc partial launch")) return e;
  kv_stats_final_kernel<<<static_cast<unsigned>(H), 128, 0, stream>>>(scratch, nchunk, L, kmean, vmean, vscale);
  return check_cuda(cudaGetLastError(), "attn_kv_stats_noalloc final launch");
}

extern "C" int rh3_attn_quant_qk(const void* x, int64_t x_ss, int64_t x_sh, int64_t L, int64_t Lpad, int64_t H,
                                 const float* mean, void* codes, float* scales, cudaStream_t stream) {
  RH3_CHECK_ARG(L > 0 && H > 0 && H < 65536 && Lpad >= L && Lpad % 128 == 0,
                "attn_quant_qk: bad shape L=%lld Lpad=%lld H=%lld (Lpad must be a multiple of 128)", (long long)L,
                (long long)Lpad, (long long)H);
  RH3_CHECK_ARG(x && codes && scales, "attn_quant_qk: null pointer");
  RH3_CHECK_ARG(aligned(x, 8) && aligned(codes, 16) && x_ss % 4 == 0 && x_sh % 4 == 0 && (!mean || aligned(mean, 16)),
                "attn_quant_qk: misaligned input");
  quant_block64_kernel<<<dim3(static_cast<unsigned>(Lpad / 64), static_cast<unsigned>(H)), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), x_ss, x_sh, L, Lpad, mean, static_cast<int8_t*>(codes), scales);
  return check_cuda(cudaGetLastError(), "attn_quant_qk launch");
}

extern "C" int rh3_attn_quant_v(const void* v, int64_t v_ss, int64_t v_sh, int64_t L, int64_t Lpad, int64_t H,
                                const float* vmean, const float* vscale, void* vt, cudaStream_t stream) {
  RH3_CHECK_ARG(L > 0 && H > 0 && H < 65536 && Lpad >= L && Lpad % 128 == 0,
                "attn_quant_v: bad shape L=%lld Lpad=%lld H=%lld (Lpad must be a multiple of 128)", (long long)L,
                (long long)Lpad, (long long)H);
  RH3_CHECK_ARG(v && vmean && vscale && vt, "attn_quant_v: null pointer");
  RH3_CHECK_ARG(aligned(v, 8) && aligned(vt, 16) && aligned(vmean, 16) && aligned(vscale, 16) && v_ss % 4 == 0 &&
                    v_sh % 4 == 0,
                "attn_quant_v: misaligned input");
  quant_v_kernel<<<dim3(static_cast<unsigned>(Lpad / 128), static_cast<unsigned>(H)), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(v), v_ss, v_sh, L, Lpad, vmean, vscale, static_cast<uint8_t*>(vt));
  return check_cuda(cudaGetLastError(), "attn_quant_v launch");
}
