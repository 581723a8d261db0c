// Attention pre-pass: everything that turns bf16 q / k / v rows into the operands of the INT8 attention kernel.
// All of it is HBM-bound row work, laid out the same way everywhere: a HALF-WARP owns one (token, head) row of 128
// channels, lane i of the half-warp holds channels 8i .. 8i+7, so every global access is one 16-byte load or store
// per lane (256 B per row per instruction) and a warp has two rows in flight.
//
//   rh3_attn_prepass        the whole pre-pass of one attention call in three launches:
//                             1. rope_stats_kernel  Q rows: (RMSNorm + 3-D RoPE) -> block-64 int8 codes and scales,
//                                                   straight from registers;
//                                                   K rows: (RMSNorm + RoPE, stored once as bf16) and V rows:
//                                                   per-(head, channel) partial sums / extrema of 256-token chunks
//                             2. kv_stats_final     K mean (smoothing), V mean and V scale from the partials
//                             3. quant_kv_kernel    K - mean -> block-64 int8; (V - mean) / scale -> e4m3, transposed
//                           q is read once, k and v twice, and nothing but the roped k is written besides the operands.
//   rh3_rmsnorm_rope3d      the RMSNorm + RoPE alone (bf16 in, bf16 out)
//   rh3_attn_kv_stats, rh3_attn_quant_qk, rh3_attn_quant_v   the stages one by one, on the same kernels
//   rh3_rope_scatter_heads  RMSNorm + RoPE fused with the token -> head exchange of sequence parallelism
//
// Arithmetic contract (what the CPU oracle restates bit for bit; reference: custom_nodes/rapid_h3/csrc/
// attn_int8.cu:82-109 stats, :130-170 / :404-443 Q/K quantizers, :217-260 rms_rope_row, :452-496 quant_v, and the
// emulation script bench/attn_emulate.py:10-23 `q8(x, 1, 64)` / `f8(x, 0)`):
//   RMSNorm   sum of squares: the 8 channels of a lane in order, then an xor butterfly over the 16 lanes;
//             r = 1 / sqrt(ss / 128 + eps) with IEEE division and square root (the reference uses the .approx forms,
//             which no CPU reproduces); y = bf16((r * x) * w)
//   RoPE      pairs (i, i + 48), i < 48, table row [48][2][2] bf16 = (t00, t01, t10, t11):
//             out_i = bf16(a * t00 + b * t01), out_{i+48} = bf16(a * t10 + b * t11), a = y_i, b = y_{i+48};
//             channels 96..127 are normalised only
//   K / V statistics over the STORED bf16 values: inside a 256-token chunk the 16 tokens of a half-warp in order,
//             then the 16 half-warps in order; then the chunks in order; mean = sum / L;
//             vscale = max(max(vmax - vmean, vmean - vmin), 1e-8) / 448
//   Q / K     one scale per 64-token block per head, s = max(amax, 1e-8) / 127, code = rint((x - mean) / s)
//   V         e4m3((v - vmean) / vscale) clamped to +-448, stored [H][128][Lpad] so that keys are contiguous
#include <atomic>

#include "common.cuh"
#include "rapidh3_b200.h"

namespace rh3 {
namespace {

constexpr int D = 128;
constexpr int CHUNK = 256;         // tokens per statistics chunk = per CTA of rope_stats_kernel
constexpr int HW_PER_CTA = 16;     // half-warps in a 256-thread CTA
constexpr int TOK_PER_HW = CHUNK / HW_PER_CTA;   // K / V side: 16 tokens per half-warp, in batches of 4
constexpr int Q_TILE = 128;                      // Q side: a CTA covers two 64-token blocks, 8 tokens per half-warp
constexpr int Q_TOK_PER_HW = Q_TILE / HW_PER_CTA;

// ---------------------------------------------------------------------------------------------
// half-warp row helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void unpack8(const uint4 raw, float* x) {
  x[0] = bf16_lo(raw.x); x[1] = bf16_hi(raw.x); x[2] = bf16_lo(raw.y); x[3] = bf16_hi(raw.y);
  x[4] = bf16_lo(raw.z); x[5] = bf16_hi(raw.z); x[6] = bf16_lo(raw.w); x[7] = bf16_hi(raw.w);
}
__device__ __forceinline__ uint4 pack8(const float* x) {
  return make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
}
__device__ __forceinline__ uint4 load_row16(const __nv_bfloat16* row, int l16) {
  return __ldg(reinterpret_cast<const uint4*>(row + l16 * 8));
}
// sum over the 16 lanes of a half-warp, same value in every lane, fixed order (xor 8, 4, 2, 1)
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float half_warp_max(float v) {
#pragma unroll
  for (int o = 8; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// What a lane needs of the norm weight and of one token's rope table row.
struct NormRope {
  float w[8];        // norm weight of this lane's channels
  uint32_t t[16];    // rope words of this lane's 8 pairs: t[2j] = (t00, t01), t[2j+1] = (t10, t11) of pair j
};
__device__ __forceinline__ void load_norm_weight(const __nv_bfloat16* __restrict__ w, int l16, NormRope& nr) {
  unpack8(load_row16(w, l16), nr.w);
}
// Lanes 0..5 hold the first halves of the rotary pairs (channels 0..47), lanes 6..11 the second halves (48..95);
// both read the 64 bytes of the table row that describe their 8 pairs. Lanes 12..15 only normalise.
__device__ __forceinline__ void load_rope_row(const __nv_bfloat16* __restrict__ tab_row, int l16, NormRope& nr) {
  if (l16 < 12) {
    const uint4* p = reinterpret_cast<const uint4*>(tab_row + (l16 < 6 ? l16 : l16 - 6) * 32);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 q = __ldg(p + i);
      nr.t[4 * i] = q.x, nr.t[4 * i + 1] = q.y, nr.t[4 * i + 2] = q.z, nr.t[4 * i + 3] = q.w;
    }
  }
}
// RMSNorm (+ RoPE when `rope`) of one row held as 8 floats per lane; the result is the bf16-rounded row, as floats.
__device__ __forceinline__ void norm_rope_row(float* v, const NormRope& nr, float eps, bool rope, int lane) {
  const int l16 = lane & 15;
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss = __fadd_rn(ss, __fmul_rn(v[j], v[j]));
  ss = half_warp_sum(ss);
  const float r = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, 128.f), eps)));
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = bf16_round(__fmul_rn(__fmul_rn(r, v[j]), nr.w[j]));
  if (rope) {
    // the other half of every pair lives 6 lanes away (48 channels) in the same half-warp
    const int partner = (lane & 16) | (l16 < 6 ? l16 + 6 : (l16 < 12 ? l16 - 6 : l16));
    float other[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) other[j] = __shfl_sync(0xffffffffu, v[j], partner);
    if (l16 < 12) {
      const bool first = l16 < 6;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t tw = first ? nr.t[2 * j] : nr.t[2 * j + 1];
        const float a = first ? v[j] : other[j], b = first ? other[j] : v[j];
        v[j] = bf16_round(__fadd_rn(__fmul_rn(a, bf16_lo(tw)), __fmul_rn(b, bf16_hi(tw))));
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// RMSNorm + RoPE alone: a half-warp per (token, head) row
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rmsnorm_rope_kernel(const __nv_bfloat16* __restrict__ x, int64_t x_ss, int64_t x_sh,
                                                           __nv_bfloat16* __restrict__ y, int64_t y_ss, int64_t y_sh,
                                                           int64_t S, int H, const __nv_bfloat16* __restrict__ w,
                                                           float eps, const __nv_bfloat16* __restrict__ tab) {
  const int lane = threadIdx.x & 31, l16 = lane & 15;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * HW_PER_CTA + (threadIdx.x >> 4);
  const bool live = row < S * H;
  const int64_t s = live ? row / H : 0;
  const int h = live ? static_cast<int>(row - s * H) : 0;
  NormRope nr;
  load_norm_weight(w, l16, nr);
  if (tab) load_rope_row(tab + s * 48 * 4, l16, nr);
  float v[8];
  unpack8(load_row16(x + s * x_ss + h * x_sh, l16), v);
  norm_rope_row(v, nr, eps, tab != nullptr, lane);   // both half-warps take part in the shuffles
  if (live) *reinterpret_cast<uint4*>(y + s * y_ss + h * y_sh + l16 * 8) = pack8(v);
}

// ---------------------------------------------------------------------------------------------
// Sequence-parallel form: RMSNorm + RoPE of q and k fused with the token -> head exchange. The qkv rows of this
// rank's tokens are normalised, rotated and stored straight into the buffer of the rank that owns the head (its
// own memory or a peer's over NVLink): dst[r] is [total tokens, 3, (H/P)*128] on rank r, row0 is the global index
// of this rank's first token. Plain stores only; ordering against the readers is the caller's stream-ordered
// barrier. A half-warp per (token, head): q row, k row, v row (copied unchanged).
// ---------------------------------------------------------------------------------------------
struct ScatterDst {
  __nv_bfloat16* ptr[8];
};

__global__ void __launch_bounds__(256) rope_scatter_kernel(const __nv_bfloat16* __restrict__ qkv, int64_t ld, int64_t S,
                                                           int H, int heads_per_rank, int64_t row0,
                                                           const __nv_bfloat16* __restrict__ qw,
                                                           const __nv_bfloat16* __restrict__ kw, float eps,
                                                           const __nv_bfloat16* __restrict__ tab,
                                                           const __grid_constant__ ScatterDst dst) {
  const int lane = threadIdx.x & 31, l16 = lane & 15;
  const int64_t id = static_cast<int64_t>(blockIdx.x) * HW_PER_CTA + (threadIdx.x >> 4);
  const bool live = id < S * H;
  const int64_t s = live ? id / H : 0;
  const int h = live ? static_cast<int>(id - s * H) : 0;
  const int64_t hd = static_cast<int64_t>(H) * D;
  const __nv_bfloat16* row = qkv + s * ld + h * D;
  NormRope nq, nk;
  load_norm_weight(qw, l16, nq);
  load_norm_weight(kw, l16, nk);
  if (tab) {
    load_rope_row(tab + s * 48 * 4, l16, nq);   // q and k of a token share its rope words
#pragma unroll
    for (int i = 0; i < 16; ++i) nk.t[i] = nq.t[i];
  }
  float q[8], k[8];
  unpack8(load_row16(row, l16), q);
  unpack8(load_row16(row + hd, l16), k);
  const uint4 v = load_row16(row + 2 * hd, l16);
  norm_rope_row(q, nq, eps, tab != nullptr, lane);
  norm_rope_row(k, nk, eps, tab != nullptr, lane);
  if (live) {
    const int r = h / heads_per_rank, hh = h - r * heads_per_rank;
    const int64_t w = static_cast<int64_t>(heads_per_rank) * D;
    __nv_bfloat16* out = dst.ptr[r] + (row0 + s) * 3 * w + hh * D + l16 * 8;
    *reinterpret_cast<uint4*>(out) = pack8(q);
    *reinterpret_cast<uint4*>(out + w) = pack8(k);
    *reinterpret_cast<uint4*>(out + 2 * w) = v;
  }
}

// ---------------------------------------------------------------------------------------------
// Launch 1 of the pre-pass. CTAs [0, q_ctas) quantize Q: one CTA = 128 tokens (two 64-token blocks) of one head, a
// half-warp owns 8 of them, loads all 8 rows before it touches the first and keeps them as packed bf16 until the
// block maximum is known. The other CTAs prepare K and V: one CTA = one 256-token statistics chunk of one head, a
// half-warp owns 16 tokens and works through them four at a time (eight 16-byte loads in flight per lane). Heads
// vary fastest, so the CTAs that share a token's rope table row run together and find it in L2.
// ---------------------------------------------------------------------------------------------
struct RopeStatsParams {
  // Q side
  const __nv_bfloat16* q; int64_t q_ss, q_sh; int64_t Lq, Lq_pad;
  const __nv_bfloat16* q_w;           // norm weight or null (q is already normalised / rotated)
  __nv_bfloat16* q_out; int64_t qo_ss, qo_sh;  // optional: the normalised / rotated q as bf16 (null = not stored)
  int8_t* q8; float* qs;
  // K / V side
  const __nv_bfloat16* k; int64_t k_ss, k_sh;
  const __nv_bfloat16* k_w;           // norm weight or null
  __nv_bfloat16* k_out; int64_t ko_ss, ko_sh;  // where the normalised / rotated k goes (may be k itself); unused if !k_w
  const __nv_bfloat16* v; int64_t v_ss, v_sh;
  int64_t Lk;
  float* part;                        // [H][nchunk_k][4][128]: k sum, v sum, v max, v min
  int nchunk_k;
  // common
  const __nv_bfloat16* tab;           // rope table [L][48][2][2] or null
  float eps;
  int H;
  int q_ctas;
};

__global__ void __launch_bounds__(256, 2) rope_stats_kernel(const RopeStatsParams p) {
  __shared__ float sh[HW_PER_CTA * 4 * D];  // Q side: 16 block maxima; K/V side: per half-warp partials [hw][4][128]
  const int lane = threadIdx.x & 31, l16 = lane & 15, hw = threadIdx.x >> 4;
  const bool q_side = static_cast<int>(blockIdx.x) < p.q_ctas;
  const int idx = q_side ? blockIdx.x : blockIdx.x - p.q_ctas;
  const int chunk = idx / p.H, h = idx - chunk * p.H;
  NormRope nr;

  if (q_side) {
    // ---- Q: (norm + rope) -> rows kept as packed bf16 -> block-64 abs-max -> int8 codes ----
    const int64_t tok0 = static_cast<int64_t>(chunk) * Q_TILE + hw * Q_TOK_PER_HW;
    if (p.q_w) load_norm_weight(p.q_w, l16, nr);
    uint4 kept[Q_TOK_PER_HW];
#pragma unroll
    for (int i = 0; i < Q_TOK_PER_HW; ++i) {
      const int64_t s = tok0 + i < p.Lq ? tok0 + i : 0;
      kept[i] = load_row16(p.q + s * p.q_ss + h * p.q_sh, l16);
    }
    float am = 0.f;
#pragma unroll
    for (int i = 0; i < Q_TOK_PER_HW; ++i) {
      const int64_t s = tok0 + i;
      const bool live = s < p.Lq;   // uniform over the half-warp
      float v[8];
      unpack8(kept[i], v);
      if (p.q_w) {
        if (p.tab) load_rope_row(p.tab + (live ? s : 0) * 48 * 4, l16, nr);
        norm_rope_row(v, nr, p.eps, p.tab != nullptr, lane);
        if (p.q_out && live) *reinterpret_cast<uint4*>(p.q_out + s * p.qo_ss + h * p.qo_sh + l16 * 8) = pack8(v);
        kept[i] = pack8(v);
      }
      if (live) {
#pragma unroll
        for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(v[j]));
      } else {
        kept[i] = make_uint4(0, 0, 0, 0);
      }
    }
    am = half_warp_max(am);
    if (l16 == 0) sh[hw] = am;
    __syncthreads();
    const int b8 = hw & ~7;  // the eight half-warps of this 64-token block
    am = sh[b8];
#pragma unroll
    for (int i = 1; i < 8; ++i) am = fmaxf(am, sh[b8 + i]);
    const float scale = __fdiv_rn(fmaxf(am, 1e-8f), 127.f), inv = __fdiv_rn(1.f, scale);
    if ((hw & 7) == 0 && l16 == 0) p.qs[static_cast<int64_t>(h) * (p.Lq_pad / 64) + chunk * 2 + (hw >> 3)] = scale;
    int8_t* out = p.q8 + (static_cast<int64_t>(h) * p.Lq_pad + tok0) * D + l16 * 8;
#pragma unroll
    for (int i = 0; i < Q_TOK_PER_HW; ++i) {
      float v[8];
      unpack8(kept[i], v);   // rows beyond Lq hold zeros and get zero codes
      *reinterpret_cast<uint2*>(out + i * D) = quant8_i8(v, scale, inv);
    }
    return;
  }

  // ---- K (norm + rope, stored once) and V: chunk partials of the stored values ----
  const int64_t tok0 = static_cast<int64_t>(chunk) * CHUNK + hw * TOK_PER_HW;
  if (p.k_w) load_norm_weight(p.k_w, l16, nr);
  float ks[8], vs[8], vmx[8], vmn[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) ks[j] = 0.f, vs[j] = 0.f, vmx[j] = -INFINITY, vmn[j] = INFINITY;
#pragma unroll 1
  for (int i0 = 0; i0 < TOK_PER_HW; i0 += 4) {
    uint4 kraw[4], vraw[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t s = tok0 + i0 + u < p.Lk ? tok0 + i0 + u : 0;
      kraw[u] = load_row16(p.k + s * p.k_ss + h * p.k_sh, l16);
      vraw[u] = load_row16(p.v + s * p.v_ss + h * p.v_sh, l16);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t s = tok0 + i0 + u;
      const bool live = s < p.Lk;
      float kv[8], vv[8];
      unpack8(kraw[u], kv);
      unpack8(vraw[u], vv);
      if (p.k_w) {
        if (p.tab) load_rope_row(p.tab + (live ? s : 0) * 48 * 4, l16, nr);
        norm_rope_row(kv, nr, p.eps, p.tab != nullptr, lane);
        if (live) *reinterpret_cast<uint4*>(p.k_out + s * p.ko_ss + h * p.ko_sh + l16 * 8) = pack8(kv);
      }
      if (live) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ks[j] = __fadd_rn(ks[j], kv[j]);
          vs[j] = __fadd_rn(vs[j], vv[j]);
          vmx[j] = fmaxf(vmx[j], vv[j]);
          vmn[j] = fminf(vmn[j], vv[j]);
        }
      }
    }
  }
  float* mine = sh + hw * 4 * D + l16 * 8;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    mine[j] = ks[j];
    mine[D + j] = vs[j];
    mine[2 * D + j] = vmx[j];
    mine[3 * D + j] = vmn[j];
  }
  __syncthreads();
  // the 16 half-warps of the chunk in order; thread t: channel t % 128, the two sums (t < 128) or the two extrema
  const int c = threadIdx.x & 127, pair = threadIdx.x >> 7;
  float a = pair ? -INFINITY : 0.f, b = pair ? INFINITY : 0.f;
  for (int g = 0; g < HW_PER_CTA; ++g) {
    const float x0 = sh[g * 4 * D + (2 * pair) * D + c], x1 = sh[g * 4 * D + (2 * pair + 1) * D + c];
    a = pair ? fmaxf(a, x0) : __fadd_rn(a, x0);
    b = pair ? fminf(b, x1) : __fadd_rn(b, x1);
  }
  float* out = p.part + (static_cast<int64_t>(h) * p.nchunk_k + chunk) * 4 * D;
  out[(2 * pair) * D + c] = a;
  out[(2 * pair + 1) * D + c] = b;
}

// ---------------------------------------------------------------------------------------------
// Launch 2: chunk partials -> K mean, V mean, V scale. A thread per (head, channel) walks the chunks in order.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) kv_stats_final_kernel(const float* __restrict__ part, int nchunk, int64_t L,
                                                             float* __restrict__ kmean, float* __restrict__ vmean,
                                                             float* __restrict__ vscale, float v_qmax) {
  const int h = blockIdx.x, c = threadIdx.x;
  const float* p = part + static_cast<int64_t>(h) * nchunk * 4 * D + c;
  float ksum = 0.f, vsum = 0.f, vhi = -INFINITY, vlo = INFINITY;
  for (int i = 0; i < nchunk; ++i, p += 4 * D) {
    ksum = __fadd_rn(ksum, p[0]);
    vsum = __fadd_rn(vsum, p[D]);
    vhi = fmaxf(vhi, p[2 * D]);
    vlo = fminf(vlo, p[3 * D]);
  }
  const float n = static_cast<float>(L);
  const float mk = __fdiv_rn(ksum, n), mv = __fdiv_rn(vsum, n);
  kmean[h * D + c] = mk;
  vmean[h * D + c] = mv;
  // largest |v - mean| from the two extrema (the subtraction is monotonic, so this is the abs-max of v - mean)
  vscale[h * D + c] = __fdiv_rn(fmaxf(fmaxf(__fsub_rn(vhi, mv), __fsub_rn(mv, vlo)), 1e-8f), v_qmax);
}

// ---------------------------------------------------------------------------------------------
// Launch 3. One CTA = one 128-token tile of one head (the key tile of the attention kernel); half-warp hw owns
// tokens 8*hw .. 8*hw+7. K: minus the channel mean, block-64 abs-max, int8 codes. V: e4m3 codes of
// (v - mean) / scale written row-major into a 16 KB shared tile and read back by channel, 32 keys (two 16-byte
// stores, one full 32-byte sector) at a time.
// ---------------------------------------------------------------------------------------------
// Eight int8 codes of values that each have their own scale: rint(y / s) with the IEEE quotient.
__device__ __forceinline__ uint2 quant8_i8_per_channel(const float* y, const float* s) {
  uint32_t w[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) w[j] = __float_as_uint(__fadd_rn(__fdiv_rn(y[j], s[j]), 12582912.f));
  return make_uint2(pack_low_bytes(w[0], w[1], w[2], w[3]), pack_low_bytes(w[4], w[5], w[6], w[7]));
}

template <bool DO_K, bool DO_V, bool V_I8 = false>
__global__ void __launch_bounds__(256, 3) quant_kv_kernel(const __nv_bfloat16* __restrict__ K, int64_t k_ss, int64_t k_sh,
                                                       const __nv_bfloat16* __restrict__ V, int64_t v_ss, int64_t v_sh,
                                                       int64_t L, int64_t Lpad, const float* __restrict__ kmean,
                                                       const float* __restrict__ vmean, const float* __restrict__ vscale,
                                                       int8_t* __restrict__ k8, float* __restrict__ kscale,
                                                       uint8_t* __restrict__ Vt) {
  __shared__ __align__(16) uint8_t tile[DO_V ? 128 * D : 16];
  __shared__ float red[HW_PER_CTA];
  const int l16 = threadIdx.x & 15, hw = threadIdx.x >> 4;
  const int h = blockIdx.y;
  const int64_t tile0 = static_cast<int64_t>(blockIdx.x) * 128, tok0 = tile0 + hw * 8;

  if (DO_K) {
    float mean[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (kmean) {
      const float4 m0 = *reinterpret_cast<const float4*>(kmean + h * D + l16 * 8);
      const float4 m1 = *reinterpret_cast<const float4*>(kmean + h * D + l16 * 8 + 4);
      mean[0] = m0.x, mean[1] = m0.y, mean[2] = m0.z, mean[3] = m0.w;
      mean[4] = m1.x, mean[5] = m1.y, mean[6] = m1.z, mean[7] = m1.w;
    }
    uint4 kept[8];
    float am = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const bool live = tok0 + i < L;
      kept[i] = live ? load_row16(K + (tok0 + i) * k_ss + h * k_sh, l16) : make_uint4(0, 0, 0, 0);
      if (live) {
        float v[8];
        unpack8(kept[i], v);
#pragma unroll
        for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(__fsub_rn(v[j], mean[j])));
      }
    }
    am = half_warp_max(am);
    if (l16 == 0) red[hw] = am;
    __syncthreads();
    const int b8 = hw & ~7;  // the eight half-warps of this 64-token block
    am = red[b8];
#pragma unroll
    for (int i = 1; i < 8; ++i) am = fmaxf(am, red[b8 + i]);
    const float scale = __fdiv_rn(fmaxf(am, 1e-8f), 127.f), inv = __fdiv_rn(1.f, scale);
    if ((hw & 7) == 0 && l16 == 0) kscale[static_cast<int64_t>(h) * (Lpad / 64) + blockIdx.x * 2 + (hw >> 3)] = scale;
    int8_t* out = k8 + (static_cast<int64_t>(h) * Lpad + tok0) * D + l16 * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float v[8];
      unpack8(kept[i], v);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __fsub_rn(v[j], mean[j]);
      // rows beyond L get zero codes (their mean must not be subtracted)
      *reinterpret_cast<uint2*>(out + i * D) = tok0 + i < L ? quant8_i8(v, scale, inv) : make_uint2(0, 0);
    }
  }

  if (DO_V) {
    float mean[8], sc[8], inv[8];
    {
      const float4 m0 = *reinterpret_cast<const float4*>(vmean + h * D + l16 * 8);
      const float4 m1 = *reinterpret_cast<const float4*>(vmean + h * D + l16 * 8 + 4);
      const float4 s0 = *reinterpret_cast<const float4*>(vscale + h * D + l16 * 8);
      const float4 s1 = *reinterpret_cast<const float4*>(vscale + h * D + l16 * 8 + 4);
      mean[0] = m0.x, mean[1] = m0.y, mean[2] = m0.z, mean[3] = m0.w;
      mean[4] = m1.x, mean[5] = m1.y, mean[6] = m1.z, mean[7] = m1.w;
      sc[0] = s0.x, sc[1] = s0.y, sc[2] = s0.z, sc[3] = s0.w;
      sc[4] = s1.x, sc[5] = s1.y, sc[6] = s1.z, sc[7] = s1.w;
#pragma unroll
      for (int j = 0; j < 8; ++j) inv[j] = __fdiv_rn(1.f, sc[j]);
    }
    uint4 raw[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) raw[i] = load_row16(V + (tok0 + i < L ? tok0 + i : 0) * v_ss + h * v_sh, l16);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float v[8];
      unpack8(raw[i], v);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __fsub_rn(v[j], mean[j]);
      *reinterpret_cast<uint2*>(tile + (hw * 8 + i) * D + l16 * 8) =
          tok0 + i < L ? (V_I8 ? quant8_i8_per_channel(v, sc) : quant8_e4m3_per_channel(v, sc, inv)) : make_uint2(0, 0);
    }
    __syncthreads();
    // item = (channel d, group of 32 keys): consecutive threads take consecutive channels, so one load instruction
    // reads 32 consecutive bytes of one token row (no bank conflict) and every thread stores a full 32-byte sector
#pragma unroll
    for (int rep = 0; rep < 2; ++rep) {
      const int item = threadIdx.x + rep * 256, d = item & 127, grp = item >> 7;
      uint32_t w[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const uint8_t* src = tile + (grp * 32 + q * 4) * D + d;
        w[q] = static_cast<uint32_t>(src[0]) | (static_cast<uint32_t>(src[D]) << 8) |
               (static_cast<uint32_t>(src[2 * D]) << 16) | (static_cast<uint32_t>(src[3 * D]) << 24);
      }
      uint4* dst = reinterpret_cast<uint4*>(Vt + (static_cast<int64_t>(h) * D + d) * Lpad + tile0 + grp * 32);
      dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
      dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Per-token operands of the token-scaled attention kernel (attn_tok.cu). A half-warp per (token, head) row:
//   (RMSNorm + RoPE when asked) -> minus the channel mean (K) -> 128-point Hadamard rotation, unnormalised:
//   butterflies (a, b) -> (a + b, a - b) over channel distance 1, 2, 4 inside the lane's 8 channels, then over lane
//   distance 1, 2, 4, 8 (channel distance 8 .. 64), every add a correctly rounded fp32 add -> abs-max of the row ->
//   s = max(amax, 1e-8) / 127, code = rint(y / s).
// Q rows store s; K rows store the pair (s / 128, 0) the main kernel multiplies the integer scores with (the
// rotation multiplies Q.K^T by 128) and (0, -inf) for the padding keys, whose codes are zero.
// Reference: the per-token Q/K quantizer with `hadamard128` of custom_nodes/rapid_h3/csrc/README.md ("Q, K -> int8,
// per token"), kernels attn_int8.cu:130-170.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void hadamard128(float* v, int lane) {
#pragma unroll
  for (int d = 1; d < 8; d <<= 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if ((j & d) == 0) {
        const float a = v[j], b = v[j + d];
        v[j] = __fadd_rn(a, b);
        v[j + d] = __fsub_rn(a, b);
      }
    }
  }
#pragma unroll
  for (int o = 1; o < 16; o <<= 1) {
    const bool upper = (lane & o) != 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, v[j], o);
      v[j] = upper ? __fsub_rn(other, v[j]) : __fadd_rn(v[j], other);
    }
  }
}

template <bool IS_K>
__global__ void __launch_bounds__(256) quant_tok_kernel(const __nv_bfloat16* __restrict__ x, int64_t x_ss, int64_t x_sh,
                                                        int64_t L, int64_t Lpad, int H,
                                                        const __nv_bfloat16* __restrict__ w, float eps,
                                                        const __nv_bfloat16* __restrict__ tab,
                                                        __nv_bfloat16* __restrict__ x_out, int64_t xo_ss, int64_t xo_sh,
                                                        const float* __restrict__ mean, int8_t* __restrict__ q8,
                                                        float* __restrict__ scales) {
  const int lane = threadIdx.x & 31, l16 = lane & 15;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * HW_PER_CTA + (threadIdx.x >> 4);
  const bool in_grid = row < Lpad * H;
  const int64_t s = in_grid ? row / H : 0;
  const int h = in_grid ? static_cast<int>(row - s * H) : 0;
  const bool live = in_grid && s < L;
  float v[8];
  unpack8(load_row16(x + (live ? s : 0) * x_ss + h * x_sh, l16), v);
  if (!live) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;   // padding rows: zero codes and the smallest scale
  }
  if (w) {
    NormRope nr;
    load_norm_weight(w, l16, nr);
    if (tab) load_rope_row(tab + (live ? s : 0) * 48 * 4, l16, nr);
    norm_rope_row(v, nr, eps, tab != nullptr, lane);
    if (x_out && live) *reinterpret_cast<uint4*>(x_out + s * xo_ss + h * xo_sh + l16 * 8) = pack8(v);
  }
  if (IS_K && mean) {
    const float4 m0 = *reinterpret_cast<const float4*>(mean + h * D + l16 * 8);
    const float4 m1 = *reinterpret_cast<const float4*>(mean + h * D + l16 * 8 + 4);
    const float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __fsub_rn(v[j], mm[j]);
  }
  hadamard128(v, lane);   // both half-warps take part in the shuffles
  float am = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(v[j]));
  am = half_warp_max(am);
  const float scale = __fdiv_rn(fmaxf(am, 1e-8f), 127.f), inv = __fdiv_rn(1.f, scale);
  if (!in_grid) return;
  *reinterpret_cast<uint2*>(q8 + (static_cast<int64_t>(h) * Lpad + s) * D + l16 * 8) =
      live ? quant8_i8(v, scale, inv) : make_uint2(0, 0);
  if (l16 == 0) {
    if (IS_K) {
      float* t = scales + (static_cast<int64_t>(h) * (Lpad / 128) + s / 128) * 256 + (s & 127);
      t[0] = live ? __fmul_rn(scale, 0.0078125f) : 0.f;
      t[128] = live ? 0.f : -INFINITY;
    } else {
      scales[static_cast<int64_t>(h) * Lpad + s] = scale;
    }
  }
}

bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
bool strides16(int64_t a, int64_t b) { return a % 8 == 0 && b % 8 == 0; }  // rows start on 16-byte boundaries

int launch_rope_stats(const RopeStatsParams& p, int kv_ctas, cudaStream_t stream) {
  const int64_t ctas = static_cast<int64_t>(p.q_ctas) + kv_ctas;
  if (ctas == 0) return 0;
  RH3_CHECK_ARG(ctas < (1ll << 31), "attention pre-pass: too many tokens x heads");
  rope_stats_kernel<<<static_cast<unsigned>(ctas), 256, 0, stream>>>(p);
  return check_cuda(cudaGetLastError(), "attention pre-pass (rope / statistics) launch");
}

int kv_stats_run(const void* k, int64_t k_ss, int64_t k_sh, const void* v, int64_t v_ss, int64_t v_sh, int64_t L,
                 int64_t H, float* part, float* kmean, float* vmean, float* vscale, cudaStream_t stream,
                 const char* who) {
  const int64_t nchunk = (L + CHUNK - 1) / CHUNK;
  RH3_CHECK_ARG(nchunk * H < (1ll << 31), "%s: L x H too large", who);
  RopeStatsParams p{};
  p.k = static_cast<const __nv_bfloat16*>(k); p.k_ss = k_ss; p.k_sh = k_sh;
  p.v = static_cast<const __nv_bfloat16*>(v); p.v_ss = v_ss; p.v_sh = v_sh;
  p.Lk = L; p.part = part; p.nchunk_k = static_cast<int>(nchunk); p.H = static_cast<int>(H);
  if (int e = launch_rope_stats(p, static_cast<int>(nchunk * H), stream)) return e;
  kv_stats_final_kernel<<<static_cast<unsigned>(H), 128, 0, stream>>>(part, static_cast<int>(nchunk), L, kmean, vmean,
                                                                      vscale, 448.f);
  return check_cuda(cudaGetLastError(), "attention pre-pass (statistics) launch");
}

}  // namespace
}  // namespace rh3

using namespace rh3;

extern "C" int rh3_rmsnorm_rope3d(const void* x, int64_t x_ss, int64_t x_sh, void* y, int64_t y_ss, int64_t y_sh,
                                  int64_t S, int64_t H, const void* weight, float eps, const void* rope_table,
                                  cudaStream_t stream) {
  RH3_CHECK_ARG(S >= 0 && H > 0 && H < 65536, "rmsnorm_rope3d: bad shape S=%lld H=%lld", (long long)S, (long long)H);
  if (S == 0) return 0;
  RH3_CHECK_ARG(x && y && weight, "rmsnorm_rope3d: null pointer");
  RH3_CHECK_ARG(aligned(x, 16) && aligned(y, 16) && aligned(weight, 16) && strides16(x_ss, x_sh) && strides16(y_ss, y_sh),
                "rmsnorm_rope3d: rows must be 16-byte aligned (strides multiples of 8 elements)");
  RH3_CHECK_ARG(!rope_table || aligned(rope_table, 16), "rmsnorm_rope3d: rope table must be 16-byte aligned");
  const int64_t rows = S * H;
  RH3_CHECK_ARG((rows + HW_PER_CTA - 1) / HW_PER_CTA < (1ll << 31), "rmsnorm_rope3d: too many rows");
  rmsnorm_rope_kernel<<<static_cast<unsigned>((rows + HW_PER_CTA - 1) / HW_PER_CTA), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), x_ss, x_sh, static_cast<__nv_bfloat16*>(y), y_ss, y_sh, S, (int)H,
      static_cast<const __nv_bfloat16*>(weight), eps, static_cast<const __nv_bfloat16*>(rope_table));
  return check_cuda(cudaGetLastError(), "rmsnorm_rope3d launch");
}

extern "C" int rh3_rope_scatter_heads(const void* qkv, int64_t ld, int64_t S, int64_t H, int64_t P, int64_t row0,
                                      const void* q_weight, const void* k_weight, float eps, const void* rope_table,
                                      void* const* dst, cudaStream_t stream) {
  RH3_CHECK_ARG(S >= 0 && H > 0 && H < 65536 && P > 0 && P <= 8 && H % P == 0 && row0 >= 0,
                "rope_scatter_heads: bad shape S=%lld H=%lld P=%lld", (long long)S, (long long)H, (long long)P);
  if (S == 0) return 0;
  RH3_CHECK_ARG(qkv && q_weight && k_weight && dst, "rope_scatter_heads: null pointer");
  RH3_CHECK_ARG(aligned(qkv, 16) && aligned(q_weight, 16) && aligned(k_weight, 16) && ld % 8 == 0 && ld >= 3 * H * D,
                "rope_scatter_heads: rows must be 16-byte aligned and hold q | k | v");
  RH3_CHECK_ARG(!rope_table || aligned(rope_table, 16), "rope_scatter_heads: rope table must be 16-byte aligned");
  ScatterDst d{};
  for (int r = 0; r < P; ++r) {
    RH3_CHECK_ARG(dst[r] && aligned(dst[r], 16), "rope_scatter_heads: destination %d is null or misaligned", r);
    d.ptr[r] = static_cast<__nv_bfloat16*>(dst[r]);
  }
  const int64_t rows = S * H;
  RH3_CHECK_ARG((rows + HW_PER_CTA - 1) / HW_PER_CTA < (1ll << 31), "rope_scatter_heads: too many rows");
  rope_scatter_kernel<<<static_cast<unsigned>((rows + HW_PER_CTA - 1) / HW_PER_CTA), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(qkv), ld, S, (int)H, (int)(H / P), row0,
      static_cast<const __nv_bfloat16*>(q_weight), static_cast<const __nv_bfloat16*>(k_weight), eps,
      static_cast<const __nv_bfloat16*>(rope_table), d);
  return check_cuda(cudaGetLastError(), "rope_scatter_heads launch");
}

extern "C" int64_t rh3_attn_kv_stats_scratch_bytes(int64_t L, int64_t H) {
  const int64_t nchunk = (L + CHUNK - 1) / CHUNK;
  return H * nchunk * 4 * D * static_cast<int64_t>(sizeof(float));
}

extern "C" int rh3_attn_kv_stats(const void* k, int64_t k_ss, int64_t k_sh, const void* v, int64_t v_ss, int64_t v_sh,
                                 int64_t L, int64_t H, void* scratch, int64_t scratch_bytes, float* kmean,
                                 float* vmean, float* vscale, cudaStream_t stream) {
  RH3_CHECK_ARG(L > 0 && H > 0 && H < 65536, "attn_kv_stats: bad shape L=%lld H=%lld", (long long)L, (long long)H);
  RH3_CHECK_ARG(k && v && scratch && kmean && vmean && vscale, "attn_kv_stats: null pointer");
  RH3_CHECK_ARG(scratch_bytes >= rh3_attn_kv_stats_scratch_bytes(L, H), "attn_kv_stats: scratch too small (%lld < %lld)",
                (long long)scratch_bytes, (long long)rh3_attn_kv_stats_scratch_bytes(L, H));
  RH3_CHECK_ARG(aligned(k, 16) && aligned(v, 16) && aligned(scratch, 16) && strides16(k_ss, k_sh) && strides16(v_ss, v_sh),
                "attn_kv_stats: rows must be 16-byte aligned (strides multiples of 8 elements)");
  return kv_stats_run(k, k_ss, k_sh, v, v_ss, v_sh, L, H, static_cast<float*>(scratch), kmean, vmean, vscale, stream,
                      "attn_kv_stats");
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
  const int64_t nchunk = (L + CHUNK - 1) / CHUNK;
  RH3_CHECK_ARG(H * nchunk <= KV_STATS_NOALLOC_MAX_UNITS,
                "attn_kv_stats_noalloc: H * ceil(L/256) = %lld exceeds the built-in scratch limit of %lld; "
                "use rh3_attn_kv_stats with caller-provided scratch",
                (long long)(H * nchunk), (long long)KV_STATS_NOALLOC_MAX_UNITS);
  RH3_CHECK_ARG(k && v && kmean && vmean && vscale, "attn_kv_stats_noalloc: null pointer");
  RH3_CHECK_ARG(aligned(k, 16) && aligned(v, 16) && strides16(k_ss, k_sh) && strides16(v_ss, v_sh),
                "attn_kv_stats_noalloc: rows must be 16-byte aligned (strides multiples of 8 elements)");
  float* scratch = nullptr;
  if (int e = kv_stats_scratch_address(&scratch)) return e;
  // every partial that the second kernel reads is written by the first one in this call, so nothing
  // left over from an earlier call needs clearing
  return kv_stats_run(k, k_ss, k_sh, v, v_ss, v_sh, L, H, scratch, kmean, vmean, vscale, stream, "attn_kv_stats_noalloc");
}

extern "C" int rh3_attn_quant_qk(const void* x, int64_t x_ss, int64_t x_sh, int64_t L, int64_t Lpad, int64_t H,
                                 const float* mean, void* codes, float* scales, cudaStream_t stream) {
  RH3_CHECK_ARG(L > 0 && H > 0 && H < 65536 && Lpad >= L && Lpad % 128 == 0,
                "attn_quant_qk: bad shape L=%lld Lpad=%lld H=%lld (Lpad must be a multiple of 128)", (long long)L,
                (long long)Lpad, (long long)H);
  RH3_CHECK_ARG(x && codes && scales, "attn_quant_qk: null pointer");
  RH3_CHECK_ARG(aligned(x, 16) && aligned(codes, 16) && strides16(x_ss, x_sh) && (!mean || aligned(mean, 16)),
                "attn_quant_qk: rows must be 16-byte aligned (strides multiples of 8 elements)");
  RH3_CHECK_ARG(Lpad / 128 < (1ll << 31), "attn_quant_qk: L too large");
  quant_kv_kernel<true, false><<<dim3(static_cast<unsigned>(Lpad / 128), static_cast<unsigned>(H)), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), x_ss, x_sh, nullptr, 0, 0, L, Lpad, mean, nullptr, nullptr,
      static_cast<int8_t*>(codes), scales, nullptr);
  return check_cuda(cudaGetLastError(), "attn_quant_qk launch");
}

extern "C" int rh3_attn_quant_v(const void* v, int64_t v_ss, int64_t v_sh, int64_t L, int64_t Lpad, int64_t H,
                                const float* vmean, const float* vscale, void* vt, cudaStream_t stream) {
  RH3_CHECK_ARG(L > 0 && H > 0 && H < 65536 && Lpad >= L && Lpad % 128 == 0,
                "attn_quant_v: bad shape L=%lld Lpad=%lld H=%lld (Lpad must be a multiple of 128)", (long long)L,
                (long long)Lpad, (long long)H);
  RH3_CHECK_ARG(v && vmean && vscale && vt, "attn_quant_v: null pointer");
  RH3_CHECK_ARG(aligned(v, 16) && aligned(vt, 16) && aligned(vmean, 16) && aligned(vscale, 16) && strides16(v_ss, v_sh),
                "attn_quant_v: rows must be 16-byte aligned (strides multiples of 8 elements)");
  quant_kv_kernel<false, true><<<dim3(static_cast<unsigned>(Lpad / 128), static_cast<unsigned>(H)), 256, 0, stream>>>(
      nullptr, 0, 0, static_cast<const __nv_bfloat16*>(v), v_ss, v_sh, L, Lpad, nullptr, vmean, vscale, nullptr, nullptr,
      static_cast<uint8_t*>(vt));
  return check_cuda(cudaGetLastError(), "attn_quant_v launch");
}

// The whole pre-pass of one attention call (see the head of this file): three launches.
extern "C" int rh3_attn_prepass(const void* q, int64_t q_ss, int64_t q_sh, int64_t Lq, int64_t Lq_pad, const void* k,
                                int64_t k_ss, int64_t k_sh, const void* v, int64_t v_ss, int64_t v_sh, int64_t Lk,
                                int64_t Lk_pad, int64_t H, const void* q_weight, const void* k_weight, float eps,
                                const void* rope_table, void* q_roped, int64_t qr_ss, int64_t qr_sh, void* k_roped,
                                int64_t kr_ss, int64_t kr_sh, void* scratch, int64_t scratch_bytes, void* q8, float* qs,
                                void* k8, float* ks, void* vt, float* vscale, float* vmean, float* kmean,
                                cudaStream_t stream) {
  RH3_CHECK_ARG(Lq > 0 && Lk > 0 && H > 0 && H < 65536, "attn_prepass: bad shape Lq=%lld Lk=%lld H=%lld", (long long)Lq,
                (long long)Lk, (long long)H);
  RH3_CHECK_ARG(Lq_pad >= Lq && Lq_pad % 256 == 0 && Lk_pad >= Lk && Lk_pad % 128 == 0,
                "attn_prepass: Lq_pad must be a multiple of 256 and Lk_pad a multiple of 128, covering Lq / Lk");
  RH3_CHECK_ARG(q && k && v && scratch && q8 && qs && k8 && ks && vt && vscale && vmean && kmean,
                "attn_prepass: null pointer");
  RH3_CHECK_ARG((q_weight == nullptr) == (k_weight == nullptr), "attn_prepass: q and k norm weights come together");
  RH3_CHECK_ARG(!rope_table || (q_weight && Lq == Lk), "attn_prepass: a rope table needs the norm weights and Lq == Lk");
  RH3_CHECK_ARG(!k_weight || k_roped, "attn_prepass: the normalised k needs a place to go (k_roped; it may be k itself)");
  RH3_CHECK_ARG(aligned(q, 16) && aligned(k, 16) && aligned(v, 16) && strides16(q_ss, q_sh) && strides16(k_ss, k_sh) &&
                    strides16(v_ss, v_sh) && (!q_roped || (aligned(q_roped, 16) && strides16(qr_ss, qr_sh))) &&
                    (!k_roped || (aligned(k_roped, 16) && strides16(kr_ss, kr_sh))),
                "attn_prepass: rows must be 16-byte aligned (strides multiples of 8 elements)");
  RH3_CHECK_ARG(aligned(scratch, 16) && aligned(q8, 16) && aligned(k8, 16) && aligned(vt, 16) && aligned(vscale, 16) &&
                    aligned(vmean, 16) && aligned(kmean, 16) &&
                    (!q_weight || (aligned(q_weight, 16) && aligned(k_weight, 16))) &&
                    (!rope_table || aligned(rope_table, 16)),
                "attn_prepass: operand buffers, weights and the rope table must be 16-byte aligned");
  RH3_CHECK_ARG(scratch_bytes >= rh3_attn_kv_stats_scratch_bytes(Lk, H), "attn_prepass: scratch too small (%lld < %lld)",
                (long long)scratch_bytes, (long long)rh3_attn_kv_stats_scratch_bytes(Lk, H));
  const int64_t nchunk_k = (Lk + CHUNK - 1) / CHUNK, nchunk_q = Lq_pad / Q_TILE;
  RH3_CHECK_ARG((nchunk_k + nchunk_q) * H < (1ll << 31) && Lk_pad / 128 < (1ll << 31), "attn_prepass: L x H too large");
  RopeStatsParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q); p.q_ss = q_ss; p.q_sh = q_sh; p.Lq = Lq; p.Lq_pad = Lq_pad;
  p.q_w = static_cast<const __nv_bfloat16*>(q_weight);
  p.q_out = static_cast<__nv_bfloat16*>(q_roped); p.qo_ss = qr_ss; p.qo_sh = qr_sh;
  p.q8 = static_cast<int8_t*>(q8); p.qs = qs;
  p.k = static_cast<const __nv_bfloat16*>(k); p.k_ss = k_ss; p.k_sh = k_sh;
  p.k_w = static_cast<const __nv_bfloat16*>(k_weight);
  p.k_out = static_cast<__nv_bfloat16*>(k_roped); p.ko_ss = kr_ss; p.ko_sh = kr_sh;
  p.v = static_cast<const __nv_bfloat16*>(v); p.v_ss = v_ss; p.v_sh = v_sh;
  p.Lk = Lk; p.part = static_cast<float*>(scratch); p.nchunk_k = static_cast<int>(nchunk_k);
  p.tab = static_cast<const __nv_bfloat16*>(rope_table); p.eps = eps; p.H = static_cast<int>(H);
  p.q_ctas = static_cast<int>(nchunk_q * H);
  if (int e = launch_rope_stats(p, static_cast<int>(nchunk_k * H), stream)) return e;
  kv_stats_final_kernel<<<static_cast<unsigned>(H), 128, 0, stream>>>(p.part, p.nchunk_k, Lk, kmean, vmean, vscale, 448.f);
  if (int e = check_cuda(cudaGetLastError(), "attn_prepass statistics launch")) return e;
  // K is read where the first launch left it: the normalised copy when there is one
  const __nv_bfloat16* kq = k_weight ? static_cast<const __nv_bfloat16*>(k_roped) : static_cast<const __nv_bfloat16*>(k);
  const int64_t kq_ss = k_weight ? kr_ss : k_ss, kq_sh = k_weight ? kr_sh : k_sh;
  quant_kv_kernel<true, true><<<dim3(static_cast<unsigned>(Lk_pad / 128), static_cast<unsigned>(H)), 256, 0, stream>>>(
      kq, kq_ss, kq_sh, static_cast<const __nv_bfloat16*>(v), v_ss, v_sh, Lk, Lk_pad, kmean, vmean, vscale,
      static_cast<int8_t*>(k8), ks, static_cast<uint8_t*>(vt));
  return check_cuda(cudaGetLastError(), "attn_prepass quantizer launch");
}

// The pre-pass of the token-scaled attention kernel (rh3_attn_int8_tok): K/V statistics (the K side also applies and
// stores RMSNorm + RoPE when the weights are given), per-token rotated int8 Q and K, int8 V^T. Five launches.
extern "C" int rh3_attn_tok_prepass(const void* q, int64_t q_ss, int64_t q_sh, int64_t Lq, int64_t Lq_pad, const void* k,
                                    int64_t k_ss, int64_t k_sh, const void* v, int64_t v_ss, int64_t v_sh, int64_t Lk,
                                    int64_t Lk_pad, int64_t H, const void* q_weight, const void* k_weight, float eps,
                                    const void* rope_table, void* q_roped, int64_t qr_ss, int64_t qr_sh, void* k_roped,
                                    int64_t kr_ss, int64_t kr_sh, void* scratch, int64_t scratch_bytes, void* q8,
                                    float* qs, void* k8, float* ksb, void* vt, float* vscale, float* vmean,
                                    float* kmean, cudaStream_t stream) {
  RH3_CHECK_ARG(Lq > 0 && Lk > 0 && H > 0 && H < 65536, "attn_tok_prepass: bad shape Lq=%lld Lk=%lld H=%lld",
                (long long)Lq, (long long)Lk, (long long)H);
  RH3_CHECK_ARG(Lq_pad >= Lq && Lq_pad % 256 == 0 && Lk_pad >= Lk && Lk_pad % 128 == 0,
                "attn_tok_prepass: Lq_pad must be a multiple of 256 and Lk_pad a multiple of 128, covering Lq / Lk");
  RH3_CHECK_ARG(q && k && v && scratch && q8 && qs && k8 && ksb && vt && vscale && vmean && kmean,
                "attn_tok_prepass: null pointer");
  RH3_CHECK_ARG((q_weight == nullptr) == (k_weight == nullptr), "attn_tok_prepass: q and k norm weights come together");
  RH3_CHECK_ARG(!rope_table || (q_weight && Lq == Lk), "attn_tok_prepass: a rope table needs the norm weights and Lq == Lk");
  RH3_CHECK_ARG(!k_weight || k_roped, "attn_tok_prepass: the normalised k needs a place to go (k_roped; it may be k itself)");
  RH3_CHECK_ARG(aligned(q, 16) && aligned(k, 16) && aligned(v, 16) && strides16(q_ss, q_sh) && strides16(k_ss, k_sh) &&
                    strides16(v_ss, v_sh) && (!q_roped || (aligned(q_roped, 16) && strides16(qr_ss, qr_sh))) &&
                    (!k_roped || (aligned(k_roped, 16) && strides16(kr_ss, kr_sh))),
                "attn_tok_prepass: rows must be 16-byte aligned (strides multiples of 8 elements)");
  RH3_CHECK_ARG(aligned(scratch, 16) && aligned(q8, 16) && aligned(k8, 16) && aligned(vt, 16) && aligned(vscale, 16) &&
                    aligned(vmean, 16) && aligned(kmean, 16) && aligned(ksb, 16) &&
                    (!q_weight || (aligned(q_weight, 16) && aligned(k_weight, 16))) &&
                    (!rope_table || aligned(rope_table, 16)),
                "attn_tok_prepass: operand buffers, weights and the rope table must be 16-byte aligned");
  RH3_CHECK_ARG(scratch_bytes >= rh3_attn_kv_stats_scratch_bytes(Lk, H), "attn_tok_prepass: scratch too small (%lld < %lld)",
                (long long)scratch_bytes, (long long)rh3_attn_kv_stats_scratch_bytes(Lk, H));
  const int64_t nchunk_k = (Lk + CHUNK - 1) / CHUNK;
  const int64_t q_ctas = (Lq_pad * H + HW_PER_CTA - 1) / HW_PER_CTA, k_ctas = (Lk_pad * H + HW_PER_CTA - 1) / HW_PER_CTA;
  RH3_CHECK_ARG(nchunk_k * H < (1ll << 31) && q_ctas < (1ll << 31) && k_ctas < (1ll << 31), "attn_tok_prepass: L x H too large");
  // 1 + 2: K (norm + rope, stored) and V chunk partials -> means and the int8 V scale
  RopeStatsParams p{};
  p.k = static_cast<const __nv_bfloat16*>(k); p.k_ss = k_ss; p.k_sh = k_sh;
  p.k_w = static_cast<const __nv_bfloat16*>(k_weight);
  p.k_out = static_cast<__nv_bfloat16*>(k_roped); p.ko_ss = kr_ss; p.ko_sh = kr_sh;
  p.v = static_cast<const __nv_bfloat16*>(v); p.v_ss = v_ss; p.v_sh = v_sh;
  p.Lk = Lk; p.part = static_cast<float*>(scratch); p.nchunk_k = static_cast<int>(nchunk_k);
  p.tab = static_cast<const __nv_bfloat16*>(rope_table); p.eps = eps; p.H = static_cast<int>(H);
  if (int e = launch_rope_stats(p, static_cast<int>(nchunk_k * H), stream)) return e;
  kv_stats_final_kernel<<<static_cast<unsigned>(H), 128, 0, stream>>>(p.part, p.nchunk_k, Lk, kmean, vmean, vscale, 127.f);
  if (int e = check_cuda(cudaGetLastError(), "attn_tok_prepass statistics launch")) return e;
  // 3: Q rows (norm + rope fused), 4: K rows from the normalised copy, 5: V
  quant_tok_kernel<false><<<static_cast<unsigned>(q_ctas), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(q), q_ss, q_sh, Lq, Lq_pad, static_cast<int>(H),
      static_cast<const __nv_bfloat16*>(q_weight), eps, static_cast<const __nv_bfloat16*>(rope_table),
      static_cast<__nv_bfloat16*>(q_roped), qr_ss, qr_sh, nullptr, static_cast<int8_t*>(q8), qs);
  if (int e = check_cuda(cudaGetLastError(), "attn_tok_prepass Q launch")) return e;
  const __nv_bfloat16* kq = k_weight ? static_cast<const __nv_bfloat16*>(k_roped) : static_cast<const __nv_bfloat16*>(k);
  const int64_t kq_ss = k_weight ? kr_ss : k_ss, kq_sh = k_weight ? kr_sh : k_sh;
  quant_tok_kernel<true><<<static_cast<unsigned>(k_ctas), 256, 0, stream>>>(
      kq, kq_ss, kq_sh, Lk, Lk_pad, static_cast<int>(H), nullptr, eps, nullptr, nullptr, 0, 0, kmean,
      static_cast<int8_t*>(k8), ksb);
  if (int e = check_cuda(cudaGetLastError(), "attn_tok_prepass K launch")) return e;
  quant_kv_kernel<false, true, true><<<dim3(static_cast<unsigned>(Lk_pad / 128), static_cast<unsigned>(H)), 256, 0, stream>>>(
      nullptr, 0, 0, static_cast<const __nv_bfloat16*>(v), v_ss, v_sh, Lk, Lk_pad, nullptr, vmean, vscale, nullptr, nullptr,
      static_cast<uint8_t*>(vt));
  return check_cuda(cudaGetLastError(), "attn_tok_prepass V launch");
}
