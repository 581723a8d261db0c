// INT8 flash attention for head_dim 128, non-causal, on the Blackwell tensor cores.
//
//   S = Q8 . K8^T            int8 x int8 -> int32 in TMEM (tcgen05 kind::i8), one 128x128 tile at a time
//   t = fma(1.5*2^23 + S, c, off),  c = (qs[q block] * sl2) * ks[k block],  off = (8 - M) - 1.5*2^23 * c
//       (sl2 = softmax_scale * log2 e; one scale per 64-token block; the reference's magic-number
//       dequantisation, attn_int8.cu:22-27,2365-2370)
//   online softmax in base 2; the running maximum is kept rounded UP to an integer M, so every
//   rescale of O and l is an exact power of two and P's fp8 rounding does not depend on the order
//   in which key tiles arrive
//   P = e4m3(2^(t - M + 8))  in (128, 256] at the row maximum; l += 2^(t - M + 8) (fp32, unrounded)
//   O += P . V8              e4m3 x e4m3 -> fp32 in TMEM (tcgen05 kind::f8f6f4), V8 = e4m3((V - vmean)/vscale)
//   out = bf16((O / l) * vscale + vmean)
//
// Reference: the INT8-QK^T / FP8-P.V design of custom_nodes/rapid_h3/csrc/attn_int8.cu:1538-1759
// (attn_fwd5: P relative to the running maximum, V e4m3 per channel, l summed before rounding,
// epilogue O/l*vscale+vmean) with the per-key-block scale structure of :1781-1889 (attn_fwd6) and
// the operand definitions of bench/attn_emulate.py:10-23,88,101-103.
//
// One CTA = TWO 128-query tiles of one head (256 rows), 384 threads = three warp groups, one CTA per
// SM. The two tiles share every K / V^T tile that TMA brings in (3-stage ring) and run as two
// independent softmax pipelines:
//   warp group 0  service: warp 0 = TMA producer (Q once, then K tile 128 keys x 128 B + V^T tile 128
//                 channels x 128 keys per step), warp 1 = MMA issuer (for both query tiles, Q.K^T of
//                 key tile j+1 is issued before P.V of tile j); gives its registers away (setmaxnreg)
//   warp groups 1, 2  softmax of query tile 0 / 1, one query row per thread, 232 registers each so a
//                 whole row of S (128 values) lives in registers: the accumulator is pre-biased with
//                 1.5*2^23 so its int32 bits are a float (no conversion); the row is read from TMEM
//                 ONCE and S is handed straight back, so the next Q.K^T runs under the whole softmax;
//                 3-input max over the raw values, then t = fma(bits, c, off) in packed f32x2, exp2,
//                 e4m3 pack; P goes to shared memory in the 128-byte-swizzled K-major layout the MMA
//                 reads; O and l are rescaled by an exact power of two when the integer maximum grows
// TMEM (512 columns): S0 | S1 | O0 | O1, 128 columns each.
// Tensor-core bound: 4 * Lq * Lk * 128 operations per head.
#include <limits.h>

#include "common.cuh"
#include "rapidh3_b200.h"

namespace rh3 {
namespace {

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int QG = 2;                  // query tiles per CTA
constexpr int TILE_BYTES = 128 * 128;  // every operand tile is 128 rows x 128 bytes
constexpr int KV_STAGES = 3;
constexpr int ATTN_THREADS = 384;      // service warp group + two softmax warp groups

struct AttnParams {
  const float* qs;      // [H][Lq_pad/64]
  const float* ks;      // [H][Lk_pad/64]
  const float* vscale;  // [H][128]
  const float* vmean;   // [H][128]
  __nv_bfloat16* out;
  int64_t o_ss, o_sh;
  int Lq, Lk, Lq_pad, Lk_pad, H;
  float sl2;  // softmax_scale * log2(e)
  int* status;
  // sequence-parallel output: query rows [dst_start[r], dst_start[r+1]) go to dst_ptr[r] (this GPU's or a peer's
  // memory), addressed relative to the start of the range; n_dst == 0 selects the single buffer `out`
  int n_dst;
  long long dst_start[9];
  __nv_bfloat16* dst_ptr[8];
  // verification hook (DUMP instantiation only): the int32 scores of one 128 x 128 tile go to s_dump [128][128]
  int32_t* s_dump;
  int dump_q_tile, dump_kv_tile, dump_head;
};

struct __align__(8) AttnSmemTail {
  uint64_t q_full;
  uint64_t kv_full[KV_STAGES];
  uint64_t kv_empty[KV_STAGES];
  uint64_t s_full[QG], s_empty[QG], p_full[QG], pv_done[QG];
  uint32_t tmem_base;
  int abort_flag;
};

// Q (2 tiles) | P (2 tiles) | KV ring (K + V^T per stage)
constexpr int ATTN_SMEM_BYTES = (2 * QG + 2 * KV_STAGES) * TILE_BYTES + sizeof(AttnSmemTail) + 1024;

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  uint32_t r;
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
      "mov.b32 %0, {lo, hi};\n\t}"
      : "=r"(r)
      : "f"(a), "f"(b), "f"(c), "f"(d));
  return r;
}

constexpr float kMagic = 12582912.f;            // 1.5 * 2^23: float(kMagic + s) has s in its low mantissa bits
constexpr uint32_t kMagicBits = 0x4B400000u;    // the same value as int32 bits, used to pre-bias S in TMEM
constexpr uint32_t kNegInfBits = 0xFF800000u;

__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {  // two fp32 FMAs in one instruction
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Columns at or beyond `valid` (padding keys of the last tile) become -inf: they lose every max and
// their probability is exactly 0.
__device__ __forceinline__ void mask_tail(uint32_t* r, int col0, int valid) {
#pragma unroll
  for (int i = 0; i < 32; ++i)
    if (col0 + i >= valid) r[i] = kNegInfBits;
}

// Largest raw value (a float 1.5*2^23 + s) of one 32-column chunk, with 3-input max.
__device__ __forceinline__ float chunk_max(const uint32_t* r) {
  float m = max3(__uint_as_float(r[0]), __uint_as_float(r[1]), __uint_as_float(r[2]));
#pragma unroll
  for (int i = 3; i < 31; i += 2) m = max3(m, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
  return fmaxf(m, __uint_as_float(r[31]));
}

// Which exponentials leave the special-function unit. The 32 columns of a chunk are taken four at a time
// (group i = 0..7: columns 4i..4i+3); bit i of the mask sends the SECOND pair of group i (columns 4i+2, 4i+3)
// through the polynomial below on the FMA pipe instead of ex2.approx. 0x55 = four of sixteen pairs = 1/4 of all
// exponentials (measured at L = 36,436, H = 32: mask 0 17.05 ms, 0x11 17.5, 0x55 16.74, 0x33 16.9, 0xAA 16.8, 0xFF
// 17.6). The CPU oracle applies the same mask, so both sides evaluate the same function per column.
#ifndef RH3_ATTN_POLY_MASK
#define RH3_ATTN_POLY_MASK 0x55
#endif
constexpr uint32_t kPolyMask = RH3_ATTN_POLY_MASK;

// 2^t for two values at once without the special-function unit: t is clamped at -60 (2^-60 is nothing against
// a row sum >= 128, and the exponent arithmetic below needs a bounded t), split as t = n + f with n = rint(t)
// taken from the low mantissa bits of t + 1.5*2^23 and f = t - n in [-1/2, 1/2] (exact), 2^f evaluated as a
// cubic in Horner form with fused multiply-adds (relative error 7.5e-5, far inside P's 3-bit mantissa; the
// unrounded value also enters the row sum, where the error alternates in sign over f), and n added to the
// exponent field. Every operation is a correctly rounded fp32 operation, so the result is reproducible bit for
// bit on a CPU.
constexpr float kPolyClamp = -60.f;
constexpr float kPolyC0 = 0x1.fff694p-1f, kPolyC1 = 0x1.62f31ap-1f, kPolyC2 = 0x1.f0ddf6p-3f, kPolyC3 = 0x1.c3f6fp-5f;
__device__ __forceinline__ void exp2_poly2(uint64_t t2, float& pa, float& pb) {
  float ta, tb;
  unpack2(t2, ta, tb);
  const uint64_t tc = pack2(fmaxf(ta, kPolyClamp), fmaxf(tb, kPolyClamp));
  const uint64_t r = add2(tc, pack2(kMagic, kMagic));                        // low mantissa bits = n
  const uint64_t n = add2(r, pack2(-kMagic, -kMagic));                       // n as a float (exact)
  const uint64_t f = fma2(n, pack2(-1.f, -1.f), tc);                         // t - n (exact)
  uint64_t q = fma2(pack2(kPolyC3, kPolyC3), f, pack2(kPolyC2, kPolyC2));
  q = fma2(q, f, pack2(kPolyC1, kPolyC1));
  q = fma2(q, f, pack2(kPolyC0, kPolyC0));
  float ra, rb, qa, qb;
  unpack2(r, ra, rb);
  unpack2(q, qa, qb);
  pa = __uint_as_float(__float_as_uint(qa) + (__float_as_uint(ra) << 23));   // the magic's own bits shift out
  pb = __uint_as_float(__float_as_uint(qb) + (__float_as_uint(rb) << 23));
}

// One 32-column chunk: p = 2^(bits * cc + off) in packed f32x2, e4m3 codes written to 16-byte chunks
// 2k and 2k+1 of the row of P in shared memory (XOR-swizzled), unrounded p added to the sum.
__device__ __forceinline__ void exp_chunk(const uint32_t* r, int k, float cc, float off, uint8_t* p_row, int sw,
                                          uint64_t& lsum2) {
  const uint64_t cc2 = pack2(cc, cc), off2 = pack2(off, off);
  uint32_t w[8];
  uint64_t ls0 = pack2(0.f, 0.f), ls1 = pack2(0.f, 0.f);  // two chains per chunk keep the adds off the critical path
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float pa, pb, pc, pd;
    unpack2(fma2(pack2(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1])), cc2, off2), pa, pb);
    const uint64_t t_cd = fma2(pack2(__uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3])), cc2, off2);
    pa = ex2_approx(pa); pb = ex2_approx(pb);
    if ((kPolyMask >> i) & 1u) {
      exp2_poly2(t_cd, pc, pd);
    } else {
      unpack2(t_cd, pc, pd);
      pc = ex2_approx(pc); pd = ex2_approx(pd);
    }
    if (i & 1) ls1 = add2(ls1, add2(pack2(pa, pb), pack2(pc, pd)));
    else ls0 = add2(ls0, add2(pack2(pa, pb), pack2(pc, pd)));
    w[i] = pack_e4m3x4(pa, pb, pc, pd);
  }
  lsum2 = add2(lsum2, add2(ls0, ls1));
  *reinterpret_cast<uint4*>(p_row + (((2 * k) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
  *reinterpret_cast<uint4*>(p_row + (((2 * k + 1) ^ sw) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
}

// Register reallocation between warp groups (one instruction per warp, all four warps of the group).
// The kernel is compiled for 168 registers per thread (384 threads, one CTA per SM); the service group
// drops to 40 and each softmax thread rises to 232: 128 * 40 + 256 * 232 = 384 * 168 exactly. The two numbers
// must keep that equality: a request for more registers than the CTA's pool holds never returns.
constexpr int REGS_COMPILED = 168, REGS_SERVICE = 40, REGS_SOFTMAX = 232;  // 65536 / 384 rounded down to 8
static_assert(128 * REGS_SERVICE + 256 * REGS_SOFTMAX == ATTN_THREADS * REGS_COMPILED, "register pool must balance");
__device__ __forceinline__ void reg_release_service() { asm volatile("setmaxnreg.dec.sync.aligned.u32 40;"); }
__device__ __forceinline__ void reg_take_softmax() { asm volatile("setmaxnreg.inc.sync.aligned.u32 232;"); }

template <bool DUMP>
__global__ void __launch_bounds__(ATTN_THREADS, 1)
attn_int8_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                 const __grid_constant__ CUtensorMap tma_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                            // [QG] tiles
  uint8_t* sP = smem + QG * TILE_BYTES;          // [QG] tiles
  uint8_t* sKV = smem + 2 * QG * TILE_BYTES;     // stage s: K at +s*2*TILE, V^T at +s*2*TILE + TILE
  AttnSmemTail* tail = reinterpret_cast<AttnSmemTail*>(smem + (2 * QG + 2 * KV_STAGES) * TILE_BYTES);
  volatile int* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_pair = blockIdx.x, h = blockIdx.y;
  const int n_kv = (p.Lk + BKV - 1) / BKV;

  if (threadIdx.x == 0) {
    mbar_init(&tail->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&tail->kv_full[s], 1);
      mbar_init(&tail->kv_empty[s], 1);
    }
    for (int g = 0; g < QG; ++g) {
      mbar_init(&tail->s_full[g], 1);
      mbar_init(&tail->s_empty[g], 4);  // one arrival per softmax warp (128 separate arrivals on one
      mbar_init(&tail->p_full[g], 4);   // barrier word serialise and cost more than the MMAs they gate)
      mbar_init(&tail->pv_done[g], 1);
    }
    tail->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&tail->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tail->tmem_base;

  if (warp < 4) {
    // ============================ service warp group: TMA + MMA issue ============================
    reg_release_service();
    if (warp == 0 && lane == 0) {
      // ------------------------------ TMA producer ------------------------------
      tma_prefetch_desc(&tma_q);
      tma_prefetch_desc(&tma_k);
      tma_prefetch_desc(&tma_v);
      mbar_arrive_expect_tx(&tail->q_full, QG * TILE_BYTES);
      tma_load_2d(sQ, &tma_q, 0, h * p.Lq_pad + q_pair * (QG * BQ), &tail->q_full);
      for (int j = 0; j < n_kv; ++j) {
        const int stage = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait_relaxed(&tail->kv_empty[stage], ph ^ 1, abort_flag, p.status, ST_TIMEOUT_STAGE_EMPTY, 400)) break;
        uint8_t* sk = sKV + stage * 2 * TILE_BYTES;
        mbar_arrive_expect_tx(&tail->kv_full[stage], 2 * TILE_BYTES);
        tma_load_2d(sk, &tma_k, 0, h * p.Lk_pad + j * BKV, &tail->kv_full[stage]);
        tma_load_2d(sk + TILE_BYTES, &tma_v, j * BKV, h * HD, &tail->kv_full[stage]);
      }
    } else if (warp == 1) {
      // ------------------------------ MMA issuer ------------------------------
      // The whole warp runs the loop converged (waits, counters, addresses are warp-uniform and can live in the
      // uniform datapath the MMA instruction reads its operands from); one elected lane issues MMAs and commits.
      constexpr uint32_t idesc_qk = make_idesc(2, 1, 1, BQ, BKV);  // s32 += s8 * s8
      constexpr uint32_t idesc_pv = make_idesc(1, 0, 0, BQ, HD);   // f32 += e4m3 * e4m3
      auto issue_qk = [&](int g, int j) {
        const uint32_t q_addr = smem_u32(sQ + g * TILE_BYTES);
        const uint32_t k_addr = smem_u32(sKV + (j % KV_STAGES) * 2 * TILE_BYTES);
        if (elect_one()) {
          mma4_i8_ss(tmem_base + g * 128, make_desc_k128(q_addr), make_desc_k128(k_addr), idesc_qk, 1);
          mma_commit(&tail->s_full[g]);
        }
        __syncwarp();
      };
      auto all_ok = [](bool ok) { return __all_sync(0xffffffffu, ok) != 0; };
      bool ok = all_ok(mbar_wait(&tail->q_full, 0, abort_flag, p.status, ST_TIMEOUT_TMA_FULL) &&
                       mbar_wait(&tail->kv_full[0], 0, abort_flag, p.status, ST_TIMEOUT_TMA_FULL));
      for (int g = 0; g < QG && ok; ++g) {
        ok = all_ok(mbar_wait(&tail->s_empty[g], 0, abort_flag, p.status, ST_TIMEOUT_ACC_EMPTY));
        if (ok) {
          tc_fence_after();
          issue_qk(g, 0);
        }
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          const int ns = (j + 1) % KV_STAGES;
          ok = all_ok(mbar_wait_relaxed(&tail->kv_full[ns], ((j + 1) / KV_STAGES) & 1, abort_flag, p.status, ST_TIMEOUT_TMA_FULL, 64));
          for (int g = 0; g < QG && ok; ++g) {
            ok = all_ok(mbar_wait_relaxed(&tail->s_empty[g], (j + 1) & 1, abort_flag, p.status, ST_TIMEOUT_ACC_EMPTY, 64));
            if (ok) {
              tc_fence_after();
              issue_qk(g, j + 1);
            }
          }
          if (!ok) break;
        }
        const int stage = j % KV_STAGES;
        const uint32_t v_addr = smem_u32(sKV + stage * 2 * TILE_BYTES + TILE_BYTES);
        for (int g = 0; g < QG && ok; ++g) {
          ok = all_ok(mbar_wait_relaxed(&tail->p_full[g], j & 1, abort_flag, p.status, ST_TIMEOUT_P_READY, 64));
          if (!ok) break;
          tc_fence_after();
          const uint32_t p_addr = smem_u32(sP + g * TILE_BYTES);
          if (elect_one()) {
            mma4_f8_ss(tmem_base + 256 + g * 128, make_desc_k128(p_addr), make_desc_k128(v_addr), idesc_pv, j != 0);
            mma_commit(&tail->pv_done[g]);
          }
          __syncwarp();
        }
        if (ok) {
          if (elect_one()) mma_commit(&tail->kv_empty[stage]);  // both query tiles have read this K / V^T stage
          __syncwarp();
        }
      }
    }
  } else {
    // ============================ softmax warp groups ============================
    // S arrives as raw bits of the float 1.5*2^23 + s (the accumulator is pre-biased, see below), so
    // t = fma(bits, c, off) needs no int->float conversion and the row maximum is a 3-input float max
    // on the raw values. The row is read from TMEM once and S is handed back to the MMA warp right
    // away, so the next Q.K^T of this query tile runs under the whole softmax of the current one.
    reg_take_softmax();
    const int g = (warp >> 2) - 1;     // query tile of this warp group
    const int quad = warp & 3;         // TMEM lane quadrant this warp may access
    const int row = quad * 32 + lane;  // row of the tile = TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_row = tmem_base + g * 128 + lane_off;        // this row of S
    const uint32_t o_row = tmem_base + 256 + g * 128 + lane_off;  // this row of O
    const int64_t q_row = static_cast<int64_t>(q_pair) * (QG * BQ) + g * BQ + row;
    const float c_row = __fmul_rn(p.qs[static_cast<int64_t>(h) * (p.Lq_pad / 64) + (q_row >> 6)], p.sl2);
    const float* ks_h = p.ks + static_cast<int64_t>(h) * (p.Lk_pad / 64);
    uint8_t* p_row = sP + g * TILE_BYTES + row * 128;
    const int sw = row & 7;
    uint64_t* s_full = &tail->s_full[g];
    uint64_t* s_empty = &tail->s_empty[g];
    uint64_t* p_full = &tail->p_full[g];
    uint64_t* pv_done = &tail->pv_done[g];
    float M = 0.f, l = 0.f;
    bool ok = true;

    // bias the accumulator for tile 0
    tmem_st32_splat(t_row, kMagicBits);
    tmem_st32_splat(t_row + 32, kMagicBits);
    tmem_st32_splat(t_row + 64, kMagicBits);
    tmem_st32_splat(t_row + 96, kMagicBits);
    tmem_st_wait();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(s_empty);
    float ks0 = ks_h[0], ks1 = ks_h[1];  // block scales of the tile ahead are fetched one tile early

    for (int j = 0; j < n_kv; ++j) {
      const float c0 = __fmul_rn(c_row, ks0), c1 = __fmul_rn(c_row, ks1);
      if (j + 1 < n_kv) {
        ks0 = ks_h[2 * j + 2];
        ks1 = ks_h[2 * j + 3];
      }
      const float b0 = __fmul_rn(kMagic, c0), b1 = __fmul_rn(kMagic, c1);
      const int valid = min(BKV, p.Lk - j * BKV);
      if (!mbar_wait_relaxed(s_full, j & 1, abort_flag, p.status, ST_TIMEOUT_ACC_FULL, 32)) { ok = false; break; }
      tc_fence_after();
      // ---- the whole row of S (128 raw values) into registers, once ----
      uint32_t r0[32], r1[32], r2[32], r3[32];
      tmem_ld32(t_row, r0);
      tmem_ld32(t_row + 32, r1);
      tmem_ld32(t_row + 64, r2);
      tmem_ld32(t_row + 96, r3);
      tmem_ld_wait_regs(r0);
      tmem_ld_wait_regs(r1);
      tmem_ld_wait_regs(r2);
      tmem_ld_wait_regs(r3);
      if constexpr (DUMP) {
        // raw bits are the float 1.5*2^23 + s, i.e. the integer 0x4B400000 + s for |s| < 2^22
        if (h == p.dump_head && q_pair * QG + g == p.dump_q_tile && j == p.dump_kv_tile) {
          int32_t* d = p.s_dump + row * BKV;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            d[i] = static_cast<int32_t>(r0[i] - kMagicBits);
            d[32 + i] = static_cast<int32_t>(r1[i] - kMagicBits);
            d[64 + i] = static_cast<int32_t>(r2[i] - kMagicBits);
            d[96 + i] = static_cast<int32_t>(r3[i] - kMagicBits);
          }
        }
      }
      // S is in registers: bias it for the next Q.K^T and hand it back
      tmem_st32_splat(t_row, kMagicBits);
      tmem_st32_splat(t_row + 32, kMagicBits);
      tmem_st32_splat(t_row + 64, kMagicBits);
      tmem_st32_splat(t_row + 96, kMagicBits);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty);
      if (valid != BKV) {
        mask_tail(r0, 0, valid);
        mask_tail(r1, 32, valid);
        mask_tail(r2, 64, valid);
        mask_tail(r3, 96, valid);
      }
      // ---- row maximum: 3-input max on the raw values, one multiply-add per 64-key block ----
      const float mx0 = fmaxf(chunk_max(r0), chunk_max(r1)), mx1 = fmaxf(chunk_max(r2), chunk_max(r3));
      const float m = fmaxf(mx0 > 0.f ? fmaf(mx0, c0, -b0) : -INFINITY, mx1 > 0.f ? fmaf(mx1, c1, -b1) : -INFINITY);
      const float M_new = j == 0 ? ceilf(m) : fmaxf(M, ceilf(m));
      const bool grow = j > 0 && M_new > M;
      if (j > 0) {
        // P.V of the previous tile has finished: O is complete up to tile j-1 and the P buffer is free
        if (!mbar_wait_relaxed(pv_done, (j - 1) & 1, abort_flag, p.status, ST_TIMEOUT_PV_DONE, 32)) { ok = false; break; }
        if (__any_sync(0xffffffffu, grow)) {
          tc_fence_after();
          const float f = grow ? ex2_approx(M - M_new) : 1.f;  // exact power of two
#pragma unroll 1
          for (int c = 0; c < 16; ++c) {  // 8 columns at a time: this path is rare and must stay small
            uint32_t r[8];
            tmem_ld8(o_row + c * 8, r);
#pragma unroll
            for (int i = 0; i < 8; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * f);
            tmem_st8(o_row + c * 8, r);
          }
          tmem_st_wait();
          l *= f;
        }
      }
      M = M_new;
      const float off0 = __fsub_rn(__fsub_rn(8.f, M), b0), off1 = __fsub_rn(__fsub_rn(8.f, M), b1);
      // ---- P = e4m3(2^t) into shared memory, l += p ----
      uint64_t lsum2 = pack2(0.f, 0.f);
      exp_chunk(r0, 0, c0, off0, p_row, sw, lsum2);
      exp_chunk(r1, 1, c0, off0, p_row, sw, lsum2);
      exp_chunk(r2, 2, c1, off1, p_row, sw, lsum2);
      exp_chunk(r3, 3, c1, off1, p_row, sw, lsum2);
      float la, lb;
      unpack2(lsum2, la, lb);
      l += la + lb;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue ----
    if (ok && mbar_wait(pv_done, (n_kv - 1) & 1, abort_flag, p.status, ST_TIMEOUT_PV_DONE)) {
      tc_fence_after();
      const float inv_l = __fdiv_rn(1.f, l);
      const float* vs = p.vscale + h * HD;
      const float* vm = p.vmean + h * HD;
      __nv_bfloat16* o;
      if (p.n_dst == 0) {
        o = p.out + q_row * p.o_ss + static_cast<int64_t>(h) * p.o_sh;
      } else {
        int r = 0;
        while (r + 1 < p.n_dst && q_row >= p.dst_start[r + 1]) ++r;
        o = p.dst_ptr[r] + (q_row - p.dst_start[r]) * p.o_ss + static_cast<int64_t>(h) * p.o_sh;
      }
#pragma unroll 1
      for (int c = 0; c < 16; ++c) {
        uint32_t r[8];
        tmem_ld8(o_row + c * 8, r);
        if (q_row < p.Lq) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int d = c * 8 + 2 * i;
            const float a = fmaf(__uint_as_float(r[2 * i]) * inv_l, vs[d], vm[d]);
            const float b = fmaf(__uint_as_float(r[2 * i + 1]) * inv_l, vs[d + 1], vm[d + 1]);
            w[i] = pack_bf16x2(a, b);
          }
          *reinterpret_cast<uint4*>(o + c * 8) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  }

  // ------------------------------ teardown ------------------------------
  __syncwarp();
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace rh3

using namespace rh3;

namespace {
int attn_launch(const void* q8, const float* qs, const void* k8, const float* ks, const void* vt, const float* vscale,
                const float* vmean, int64_t Lq, int64_t Lq_pad, int64_t Lk, int64_t Lk_pad, int64_t H,
                float softmax_scale, void* out, void* const* dst, const int64_t* dst_start, int n_dst, int64_t o_ss,
                int64_t o_sh, cudaStream_t stream, int32_t* s_dump = nullptr, int64_t dump_q_tile = 0,
                int64_t dump_kv_tile = 0, int64_t dump_head = 0) {
  RH3_CHECK_ARG(Lq > 0 && Lk > 0 && H > 0 && H < 65536, "attn_int8: bad shape Lq=%lld Lk=%lld H=%lld", (long long)Lq,
                (long long)Lk, (long long)H);
  RH3_CHECK_ARG(Lq_pad >= Lq && Lk_pad >= Lk && Lq_pad % 256 == 0 && Lk_pad % 128 == 0,
                "attn_int8: Lq_pad must be a multiple of 256 and Lk_pad a multiple of 128, covering Lq / Lk");
  RH3_CHECK_ARG(H * Lq_pad < (1ll << 31) && H * Lk_pad < (1ll << 31), "attn_int8: H * Lpad too large");
  RH3_CHECK_ARG(q8 && qs && k8 && ks && vt && vscale && vmean, "attn_int8: null pointer");
  RH3_CHECK_ARG(aligned16(q8) && aligned16(k8) && aligned16(vt) && o_ss % 8 == 0 && o_sh % 8 == 0,
                "attn_int8: operands must be 16-byte aligned, output strides multiples of 8 elements");
  RH3_CHECK_ARG(softmax_scale > 0.f, "attn_int8: softmax scale must be positive");
  AttnParams p{};
  if (n_dst == 0) {
    RH3_CHECK_ARG(out && aligned16(out), "attn_int8: out must be a 16-byte aligned pointer");
    p.out = static_cast<__nv_bfloat16*>(out);
  } else {
    RH3_CHECK_ARG(n_dst >= 1 && n_dst <= 8 && dst && dst_start, "attn_int8_scatter: 1..8 destinations");
    RH3_CHECK_ARG(dst_start[0] == 0 && dst_start[n_dst] >= Lq, "attn_int8_scatter: ranges must cover [0, Lq)");
    for (int r = 0; r < n_dst; ++r) {
      RH3_CHECK_ARG(dst[r] && aligned16(dst[r]) && dst_start[r + 1] >= dst_start[r],
                    "attn_int8_scatter: destination %d is null, misaligned or its range is negative", r);
      p.dst_ptr[r] = static_cast<__nv_bfloat16*>(dst[r]);
      p.dst_start[r] = dst_start[r];
    }
    p.dst_start[n_dst] = dst_start[n_dst];
    p.n_dst = n_dst;
  }
  CUtensorMap tq, tk, tv;
  if (int e = make_tmap_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q8, HD, H * Lq_pad, HD, HD, QG * BQ,
                           CU_TENSOR_MAP_SWIZZLE_128B))
    return e;
  if (int e = make_tmap_2d(&tk, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k8, HD, H * Lk_pad, HD, HD, BKV,
                           CU_TENSOR_MAP_SWIZZLE_128B))
    return e;
  if (int e = make_tmap_2d(&tv, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, vt, Lk_pad, H * HD, Lk_pad, BKV, HD,
                           CU_TENSOR_MAP_SWIZZLE_128B))
    return e;
  p.qs = qs; p.ks = ks; p.vscale = vscale; p.vmean = vmean;
  p.o_ss = o_ss; p.o_sh = o_sh;
  p.Lq = (int)Lq; p.Lk = (int)Lk; p.Lq_pad = (int)Lq_pad; p.Lk_pad = (int)Lk_pad; p.H = (int)H;
  p.sl2 = static_cast<float>(static_cast<double>(softmax_scale) * 1.4426950408889634);
  p.status = device_status_word();
  const dim3 grid(static_cast<unsigned>((Lq + QG * BQ - 1) / (QG * BQ)), static_cast<unsigned>(H));
  auto kern = s_dump ? attn_int8_kernel<true> : attn_int8_kernel<false>;
  if (s_dump) {
    RH3_CHECK_ARG(dump_head >= 0 && dump_head < H && dump_q_tile >= 0 && dump_q_tile * BQ < Lq_pad && dump_kv_tile >= 0 &&
                      dump_kv_tile * BKV < Lk_pad,
                  "attn_int8_dump_scores: tile (%lld, %lld) of head %lld does not exist", (long long)dump_q_tile,
                  (long long)dump_kv_tile, (long long)dump_head);
    p.s_dump = s_dump;
    p.dump_q_tile = (int)dump_q_tile; p.dump_kv_tile = (int)dump_kv_tile; p.dump_head = (int)dump_head;
  }
  if (int e = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ATTN_SMEM_BYTES),
                         "attn smem attribute"))
    return e;
  kern<<<grid, ATTN_THREADS, ATTN_SMEM_BYTES, stream>>>(tq, tk, tv, p);
  return check_cuda(cudaGetLastError(), "attn_int8 launch");
}
}  // namespace

extern "C" int rh3_attn_int8(const void* q8, const float* qs, const void* k8, const float* ks, const void* vt,
                             const float* vscale, const float* vmean, int64_t Lq, int64_t Lq_pad, int64_t Lk,
                             int64_t Lk_pad, int64_t H, float softmax_scale, void* out, int64_t o_ss, int64_t o_sh,
                             cudaStream_t stream) {
  return attn_launch(q8, qs, k8, ks, vt, vscale, vmean, Lq, Lq_pad, Lk, Lk_pad, H, softmax_scale, out, nullptr, nullptr,
                     0, o_ss, o_sh, stream);
}

// Verification hook: the same launch as rh3_attn_int8, and in addition the exact int32 scores Q8 . K8^T of the 128 x 128
// tile (query tile q_tile, key tile kv_tile) of `head` are written to s_dump [128][128] (rows and keys beyond Lq / Lk
// are the products with the zero padding).
extern "C" int rh3_attn_int8_dump_scores(const void* q8, const float* qs, const void* k8, const float* ks, const void* vt,
                                         const float* vscale, const float* vmean, int64_t Lq, int64_t Lq_pad, int64_t Lk,
                                         int64_t Lk_pad, int64_t H, float softmax_scale, void* out, int64_t o_ss,
                                         int64_t o_sh, int64_t head, int64_t q_tile, int64_t kv_tile, int32_t* s_dump,
                                         cudaStream_t stream) {
  RH3_CHECK_ARG(s_dump != nullptr, "attn_int8_dump_scores: null dump buffer");
  return attn_launch(q8, qs, k8, ks, vt, vscale, vmean, Lq, Lq_pad, Lk, Lk_pad, H, softmax_scale, out, nullptr, nullptr,
                     0, o_ss, o_sh, stream, s_dump, q_tile, kv_tile, head);
}

// The same kernel with its output rows scattered over up to 8 buffers: rows [dst_start[r], dst_start[r+1]) go to
// dst[r] + (row - dst_start[r]) * o_ss + head * o_sh. The buffers may live on peer GPUs (plain stores over NVLink):
// this is the head -> token exchange of sequence parallelism done by the attention epilogue itself.
extern "C" int rh3_attn_int8_scatter(const void* q8, const float* qs, const void* k8, const float* ks, const void* vt,
                                     const float* vscale, const float* vmean, int64_t Lq, int64_t Lq_pad, int64_t Lk,
                                     int64_t Lk_pad, int64_t H, float softmax_scale, void* const* dst,
                                     const int64_t* dst_start, int64_t n_dst, int64_t o_ss, int64_t o_sh,
                                     cudaStream_t stream) {
  RH3_CHECK_ARG(n_dst >= 1 && n_dst <= 8, "attn_int8_scatter: n_dst=%lld must be 1..8", (long long)n_dst);
  return attn_launch(q8, qs, k8, ks, vt, vscale, vmean, Lq, Lq_pad, Lk, Lk_pad, H, softmax_scale, nullptr, dst,
                     dst_start, (int)n_dst, o_ss, o_sh, stream);
}
