// INT8 flash attention with per-token Q / K scales, INT8 V and 8-bit P against each tile's own maximum
// (head_dim 128, non-causal). The arithmetic of the reference's production attention (its "config 80" family:
// custom_nodes/rapid_h3/csrc/README.md "What it computes", csrc/attn_cake/DESIGN.md section 2), laid out for the
// Blackwell tensor cores:
//
//   operands   Q' = H128 . q, K' = H128 . (k - kmean)   (128-point Hadamard rotation, exact for Q.K^T up to the
//              factor 128 folded into the key scales), int8 with ONE SCALE PER TOKEN; V8 = int8((v - vmean)/vscale)
//              per channel, stored transposed
//   S = Q8 . K8^T             int8 x int8 -> int32 in TMEM (tcgen05 kind::i8)
//   t_j = s * kscale_j + kbias_j        kscale_j = (key scale) / 128, kbias_j = 0, or -inf for the padding keys
//   tm = max_j t_j                      the tile's own row maximum
//   P_j = u8(rint(255 * 2^((t_j - tm) * c)))          c = qscale(row) * softmax_scale * log2 e
//   m' = max(m, tm * c),  a = 2^(m - m'),  ts = 2^(tm * c - m')
//   l = ts * sum_j P_j + a * l          row sums from the QUANTIZED P, so numerator and denominator agree
//   A = P . V8                u8 x s8 -> int32 in TMEM, one tile at a time (|A| <= 128 * 255 * 127 < 2^22)
//   O = ts * A + a * O        the per-tile fold, fp32, in registers
//   out = bf16((O / l) * vscale + vmean)
//
// Integers become floats without a conversion instruction: both accumulators are pre-biased with 0x4B400000 (the
// softmax warps store it into TMEM before each tile's MMAs, which then accumulate onto it), so for |x| < 2^22 their
// bits are the float 1.5*2^23 + x, and subtracting 1.5*2^23 from that float is exact. The per-score arithmetic runs
// two values per instruction (fma/add/mul.rn.f32x2).
//
// One CTA = two 128-query tiles of one head, 384 threads: warp 0 = TMA producer (K tile, V^T tile and the 1 KB of
// key scales / biases per step, 3-stage ring), warp 1 = MMA issuer, warps 4..11 = softmax, one query row per
// thread with its 128 fp32 output values in registers (232 registers per softmax thread after the register
// re-split). The scores are read from TMEM twice, 16 columns at a time (maximum, then exponentials), so that the
// output row fits beside them. TMEM (512 columns): S0 | S1 | A0 | A1.
#include <limits.h>

#include "common.cuh"
#include "rapidh3_b200.h"

namespace rh3 {
namespace {

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int QG = 2;
constexpr int TILE_BYTES = 128 * 128;
constexpr int KSB_BYTES = 2 * BKV * 4;                   // per key tile: 128 scales, then 128 biases
constexpr int STAGE_BYTES = 2 * TILE_BYTES + KSB_BYTES;  // K | V^T | scales, biases
constexpr int KV_STAGES = 3;
constexpr int TOK_THREADS = 384;

struct TokParams {
  const float* qs;      // [H][Lq_pad]  one scale per query token
  const float* ksb;     // [H][Lk_pad/128][2][128]
  const float* vscale;  // [H][128]
  const float* vmean;   // [H][128]
  __nv_bfloat16* out;
  int64_t o_ss, o_sh;
  int Lq, Lk, Lq_pad, Lk_pad, H;
  float sl2;
  int* status;
};

struct __align__(8) TokSmemTail {
  uint64_t q_full;
  uint64_t kv_full[KV_STAGES];
  uint64_t kv_empty[KV_STAGES];
  uint64_t s_full[QG], s_empty[QG], p_full[QG], pv_done[QG];
  uint32_t tmem_base;
  int abort_flag;
};

constexpr int TOK_SMEM_BYTES = 2 * QG * TILE_BYTES + KV_STAGES * STAGE_BYTES + sizeof(TokSmemTail) + 1024;

constexpr float kMagic = 12582912.f;          // 1.5 * 2^23
constexpr uint32_t kMagicBits = 0x4B400000u;
constexpr float kLog2_255 = 7.99435343685886f;

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// two fp32 operations per instruction
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// The accumulators are pre-biased with 1.5*2^23 (see the kernel), so their bits ARE the float 1.5*2^23 + x; for
// |x| < 2^22 subtracting the bias is exact: two exact integer values per instruction.
__device__ __forceinline__ uint64_t unbias2(uint32_t lo, uint32_t hi) {
  return add2(pack2(__uint_as_float(lo), __uint_as_float(hi)), pack2(-kMagic, -kMagic));
}
__device__ __forceinline__ void lds4x2(uint32_t addr, uint64_t& a, uint64_t& b) {
  asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "r"(addr));
}
// plain (untiled) bulk copy global -> shared, completion counted on an mbarrier; 16-byte aligned, size % 16 == 0
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

constexpr int REGS_COMPILED = 168, REGS_SERVICE = 40, REGS_SOFTMAX = 232;
static_assert(128 * REGS_SERVICE + 256 * REGS_SOFTMAX == TOK_THREADS * REGS_COMPILED, "register pool must balance");
__device__ __forceinline__ void reg_release_service() { asm volatile("setmaxnreg.dec.sync.aligned.u32 40;"); }
__device__ __forceinline__ void reg_take_softmax() { asm volatile("setmaxnreg.inc.sync.aligned.u32 232;"); }

// t = x * kscale for four columns; on the last key tile (`bias`, uniform over the CTA) the bias is added, which is 0
// for real keys and -inf for the padding keys. rn(x * s) + 0 is the same number as fma(x, s, 0).
__device__ __forceinline__ void scores4(const uint32_t* r, uint32_t ks_addr, uint32_t kb_addr, bool bias, uint64_t& t01,
                                        uint64_t& t23) {
  uint64_t s01, s23;
  lds4x2(ks_addr, s01, s23);
  t01 = mul2(unbias2(r[0], r[1]), s01);
  t23 = mul2(unbias2(r[2], r[3]), s23);
  if (bias) {
    uint64_t b01, b23;
    lds4x2(kb_addr, b01, b23);
    t01 = add2(t01, b01);
    t23 = add2(t23, b23);
  }
}

// Maximum over one 16-column chunk of t.
__device__ __forceinline__ float chunk_tmax(const uint32_t* r, uint32_t ks_addr, uint32_t kb_addr, bool bias, float tm) {
#pragma unroll
  for (int i = 0; i < 16; i += 4) {
    uint64_t t01, t23;
    scores4(r + i, ks_addr + i * 4, kb_addr + i * 4, bias, t01, t23);
    float t0, t1, t2, t3;
    unpack2(t01, t0, t1);
    unpack2(t23, t2, t3);
    tm = fmaxf(fmaxf(tm, fmaxf(t0, t1)), fmaxf(t2, t3));
  }
  return tm;
}

// One 16-column chunk: P = u8(rint(2^(t * c + off))) written to 16-byte chunk k of the row of P in shared memory
// (XOR-swizzled like the TMA tiles), the integer codes added to `rs`.
__device__ __forceinline__ void chunk_p(const uint32_t* r, uint32_t ks_addr, uint32_t kb_addr, bool bias, float c, float off,
                                        int k, uint8_t* p_row, int sw, uint32_t& rs) {
  const uint64_t c2 = pack2(c, c), off2 = pack2(off, off), magic2 = pack2(kMagic, kMagic);
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint64_t t01, t23;
    scores4(r + 4 * i, ks_addr + i * 16, kb_addr + i * 16, bias, t01, t23);
    float e0, e1, e2, e3;
    unpack2(fma2(t01, c2, off2), e0, e1);
    unpack2(fma2(t23, c2, off2), e2, e3);
    // p <= 255 * (1 + 2^-20): adding 1.5*2^23 leaves rint(p) (ties to even) in the low byte
    float p0, p1, p2, p3;
    unpack2(add2(pack2(ex2_approx(e0), ex2_approx(e1)), magic2), p0, p1);
    unpack2(add2(pack2(ex2_approx(e2), ex2_approx(e3)), magic2), p2, p3);
    w[i] = pack_low_bytes(__float_as_uint(p0), __float_as_uint(p1), __float_as_uint(p2), __float_as_uint(p3));
    rs = __dp4a(w[i], 0x01010101u, rs);
  }
  *reinterpret_cast<uint4*>(p_row + ((k ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
}

__global__ void __launch_bounds__(TOK_THREADS, 1)
attn_tok_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                const __grid_constant__ CUtensorMap tma_v, const TokParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sP = smem + QG * TILE_BYTES;
  uint8_t* sKV = smem + 2 * QG * TILE_BYTES;  // stage s at +s*STAGE_BYTES: K, V^T, scales + biases
  TokSmemTail* tail = reinterpret_cast<TokSmemTail*>(sKV + KV_STAGES * STAGE_BYTES);
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
      mbar_init(&tail->s_empty[g], 4);  // one arrival per softmax warp
      mbar_init(&tail->p_full[g], 4);
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
    reg_release_service();
    if (warp == 0 && lane == 0) {
      // ------------------------------ TMA producer ------------------------------
      tma_prefetch_desc(&tma_q);
      tma_prefetch_desc(&tma_k);
      tma_prefetch_desc(&tma_v);
      mbar_arrive_expect_tx(&tail->q_full, QG * TILE_BYTES);
      tma_load_2d(sQ, &tma_q, 0, h * p.Lq_pad + q_pair * (QG * BQ), &tail->q_full);
      const float* ksb_h = p.ksb + static_cast<int64_t>(h) * (p.Lk_pad / BKV) * (2 * BKV);
      for (int j = 0; j < n_kv; ++j) {
        const int stage = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait_relaxed(&tail->kv_empty[stage], ph ^ 1, abort_flag, p.status, ST_TIMEOUT_STAGE_EMPTY, 400)) break;
        uint8_t* sk = sKV + stage * STAGE_BYTES;
        mbar_arrive_expect_tx(&tail->kv_full[stage], STAGE_BYTES);
        tma_load_2d(sk, &tma_k, 0, h * p.Lk_pad + j * BKV, &tail->kv_full[stage]);
        tma_load_2d(sk + TILE_BYTES, &tma_v, j * BKV, h * HD, &tail->kv_full[stage]);
        bulk_load(sk + 2 * TILE_BYTES, ksb_h + static_cast<int64_t>(j) * (2 * BKV), KSB_BYTES, &tail->kv_full[stage]);
      }
    } else if (warp == 1) {
      // ------------------------------ MMA issuer ------------------------------
      // The whole warp runs the loop converged (waits, counters, addresses are warp-uniform and can live in the
      // uniform datapath the MMA instruction reads its operands from); one elected lane issues MMAs and commits.
      constexpr uint32_t idesc_qk = make_idesc(2, 1, 1, BQ, BKV);  // s32 = s8 * s8
      constexpr uint32_t idesc_pv = make_idesc(2, 0, 1, BQ, HD);   // s32 = u8 * s8
      auto all_ok = [](bool ok) { return __all_sync(0xffffffffu, ok) != 0; };
      auto issue_qk = [&](int g, int j) {
        const uint32_t q_addr = smem_u32(sQ + g * TILE_BYTES);
        const uint32_t k_addr = smem_u32(sKV + (j % KV_STAGES) * STAGE_BYTES);
        if (elect_one()) {
          mma4_i8_ss(tmem_base + g * 128, make_desc_k128(q_addr), make_desc_k128(k_addr), idesc_qk, 1);  // onto the bias
          mma_commit(&tail->s_full[g]);
        }
        __syncwarp();
      };
      bool ok = all_ok(mbar_wait(&tail->q_full, 0, abort_flag, p.status, ST_TIMEOUT_TMA_FULL) &&
                       mbar_wait(&tail->kv_full[0], 0, abort_flag, p.status, ST_TIMEOUT_TMA_FULL));
      for (int g = 0; g < QG && ok; ++g) {
        // completion 0 of s_empty: the softmax warps have biased both accumulators of this query tile
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
            // completion j+1 of s_empty: the softmax warps have read the scores of key tile j for the last time and
            // put the bias back
            ok = all_ok(mbar_wait_relaxed(&tail->s_empty[g], (j + 1) & 1, abort_flag, p.status, ST_TIMEOUT_ACC_EMPTY, 64));
            if (ok) {
              tc_fence_after();
              issue_qk(g, j + 1);
            }
          }
          if (!ok) break;
        }
        const int stage = j % KV_STAGES;
        const uint32_t v_addr = smem_u32(sKV + stage * STAGE_BYTES + TILE_BYTES);
        for (int g = 0; g < QG && ok; ++g) {
          // P of tile j is in shared memory, and the same threads have folded the accumulator of tile j-1 before
          ok = all_ok(mbar_wait_relaxed(&tail->p_full[g], j & 1, abort_flag, p.status, ST_TIMEOUT_P_READY, 64));
          if (!ok) break;
          tc_fence_after();
          const uint32_t p_addr = smem_u32(sP + g * TILE_BYTES);
          if (elect_one()) {
            mma4_i8_ss(tmem_base + 256 + g * 128, make_desc_k128(p_addr), make_desc_k128(v_addr), idesc_pv, 1);  // onto the bias
            mma_commit(&tail->pv_done[g]);
          }
          __syncwarp();
        }
        if (ok) {
          if (elect_one()) mma_commit(&tail->kv_empty[stage]);
          __syncwarp();
        }
      }
    }
  } else {
    // ============================ softmax warp groups ============================
    reg_take_softmax();
    const int g = (warp >> 2) - 1;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_row = tmem_base + g * 128 + lane_off;
    const uint32_t a_row = tmem_base + 256 + g * 128 + lane_off;
    const int64_t q_row = static_cast<int64_t>(q_pair) * (QG * BQ) + g * BQ + row;
    const float c_row = __fmul_rn(p.qs[static_cast<int64_t>(h) * p.Lq_pad + q_row], p.sl2);
    uint8_t* p_row = sP + g * TILE_BYTES + row * 128;
    const int sw = row & 7;
    uint64_t* s_full = &tail->s_full[g];
    uint64_t* s_empty = &tail->s_empty[g];
    uint64_t* p_full = &tail->p_full[g];
    uint64_t* pv_done = &tail->pv_done[g];
    float O[HD];   // the output row
#pragma unroll
    for (int i = 0; i < HD; ++i) O[i] = 0.f;
    float m = -INFINITY, l = 0.f, a_prev = 0.f, ts_prev = 0.f;
    bool ok = true;

    auto splat4 = [](uint32_t base) {
      tmem_st32_splat(base, kMagicBits);
      tmem_st32_splat(base + 32, kMagicBits);
      tmem_st32_splat(base + 64, kMagicBits);
      tmem_st32_splat(base + 96, kMagicBits);
    };
    // O = ts * A + a * O for the tile whose P.V has just finished; the accumulator gets its bias back
    auto fold = [&](float a, float ts, bool rebias) {
      tc_fence_after();
      // two register sets: the load of the next 16 columns is in flight while these are folded
      uint32_t ra[16], rb[16];
      tmem_ld16_async(a_row, ra);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t* r = (c & 1) ? rb : ra;
        tmem_ld_wait16(r);
        if (c + 1 < 8) tmem_ld16_async(a_row + (c + 1) * 16, (c & 1) ? ra : rb);
#pragma unroll
        for (int i = 0; i < 16; ++i)
          O[c * 16 + i] = fmaf(ts, __fsub_rn(__uint_as_float(r[i]), kMagic), __fmul_rn(O[c * 16 + i], a));
      }
      if (rebias) {
        splat4(a_row);
        tmem_st_wait();
      }
    };

    // bias both accumulators of this query tile for key tile 0
    splat4(t_row);
    splat4(a_row);
    tmem_st_wait();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(s_empty);

    for (int j = 0; j < n_kv; ++j) {
      const int stage = j % KV_STAGES;
      const uint32_t ks_addr = smem_u32(sKV + stage * STAGE_BYTES + 2 * TILE_BYTES), kb_addr = ks_addr + BKV * 4;
      const bool last = j == n_kv - 1;   // only the last key tile has padding keys (bias -inf)
      // the key scales of this stage came by bulk copy: observe its barrier before reading them
      if (!mbar_wait_relaxed(&tail->kv_full[stage], (j / KV_STAGES) & 1, abort_flag, p.status, ST_TIMEOUT_TMA_FULL, 32)) { ok = false; break; }
      if (!mbar_wait_relaxed(s_full, j & 1, abort_flag, p.status, ST_TIMEOUT_ACC_FULL, 32)) { ok = false; break; }
      tc_fence_after();
      // ---- pass 1: the tile's row maximum ----
      float tm = -INFINITY;
      {
        uint32_t ra[16], rb[16];
        tmem_ld16_async(t_row, ra);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t* r = (c & 1) ? rb : ra;
          tmem_ld_wait16(r);
          if (c + 1 < 8) tmem_ld16_async(t_row + (c + 1) * 16, (c & 1) ? ra : rb);
          tm = chunk_tmax(r, ks_addr + c * 64, kb_addr + c * 64, last, tm);
        }
      }
      const float tmc = __fmul_rn(tm, c_row);
      const float m_new = fmaxf(m, tmc);
      const float a = ex2_approx(__fsub_rn(m, m_new)), ts = ex2_approx(__fsub_rn(tmc, m_new));
      const float off = __fsub_rn(kLog2_255, tmc);
      m = m_new;
      if (j > 0) {
        // P.V of the previous tile has finished: fold its accumulator; the P buffer is free again
        if (!mbar_wait_relaxed(pv_done, (j - 1) & 1, abort_flag, p.status, ST_TIMEOUT_PV_DONE, 32)) { ok = false; break; }
        fold(a_prev, ts_prev, true);
      }
      // ---- pass 2: P into shared memory, integer row sum ----
      uint32_t rs = 0;
      uint32_t ra[16], rb[16];
      tmem_ld16_async(t_row, ra);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t* r = (c & 1) ? rb : ra;
        tmem_ld_wait16(r);
        if (c + 1 < 8) tmem_ld16_async(t_row + (c + 1) * 16, (c & 1) ? ra : rb);
        if (c == 7) {
          // the scores have been read for the last time: bias the accumulator for the next Q.K^T and hand it back
          splat4(t_row);
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(s_empty);
        }
        chunk_p(r, ks_addr + c * 64, kb_addr + c * 64, last, c_row, off, c, p_row, sw, rs);
      }
      l = fmaf(ts, static_cast<float>(rs), __fmul_rn(l, a));
      a_prev = a;
      ts_prev = ts;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue ----
    if (ok && mbar_wait(pv_done, (n_kv - 1) & 1, abort_flag, p.status, ST_TIMEOUT_PV_DONE)) {
      fold(a_prev, ts_prev, false);
      if (q_row < p.Lq) {
        const float inv_l = __fdiv_rn(1.f, l);
        const float* vs = p.vscale + h * HD;
        const float* vm = p.vmean + h * HD;
        __nv_bfloat16* o = p.out + q_row * p.o_ss + static_cast<int64_t>(h) * p.o_sh;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int d = c * 8 + 2 * i;
            w[i] = pack_bf16x2(fmaf(O[d] * inv_l, vs[d], vm[d]), fmaf(O[d + 1] * inv_l, vs[d + 1], vm[d + 1]));
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

extern "C" int rh3_attn_int8_tok(const void* q8, const float* qs, const void* k8, const float* ksb, const void* vt,
                                 const float* vscale, const float* vmean, int64_t Lq, int64_t Lq_pad, int64_t Lk,
                                 int64_t Lk_pad, int64_t H, float softmax_scale, void* out, int64_t o_ss, int64_t o_sh,
                                 cudaStream_t stream) {
  RH3_CHECK_ARG(Lq > 0 && Lk > 0 && H > 0 && H < 65536, "attn_int8_tok: bad shape Lq=%lld Lk=%lld H=%lld", (long long)Lq,
                (long long)Lk, (long long)H);
  RH3_CHECK_ARG(Lq_pad >= Lq && Lk_pad >= Lk && Lq_pad % 256 == 0 && Lk_pad % 128 == 0,
                "attn_int8_tok: Lq_pad must be a multiple of 256 and Lk_pad a multiple of 128, covering Lq / Lk");
  RH3_CHECK_ARG(H * Lq_pad < (1ll << 31) && H * Lk_pad < (1ll << 31), "attn_int8_tok: H * Lpad too large");
  RH3_CHECK_ARG(q8 && qs && k8 && ksb && vt && vscale && vmean && out, "attn_int8_tok: null pointer");
  RH3_CHECK_ARG(aligned16(q8) && aligned16(k8) && aligned16(vt) && aligned16(ksb) && aligned16(out) && o_ss % 8 == 0 &&
                    o_sh % 8 == 0,
                "attn_int8_tok: operands must be 16-byte aligned, output strides multiples of 8 elements");
  RH3_CHECK_ARG(softmax_scale > 0.f, "attn_int8_tok: softmax scale must be positive");
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
  TokParams p{};
  p.qs = qs; p.ksb = ksb; p.vscale = vscale; p.vmean = vmean;
  p.out = static_cast<__nv_bfloat16*>(out); p.o_ss = o_ss; p.o_sh = o_sh;
  p.Lq = (int)Lq; p.Lk = (int)Lk; p.Lq_pad = (int)Lq_pad; p.Lk_pad = (int)Lk_pad; p.H = (int)H;
  p.sl2 = static_cast<float>(static_cast<double>(softmax_scale) * 1.4426950408889634);
  p.status = device_status_word();
  const dim3 grid(static_cast<unsigned>((Lq + QG * BQ - 1) / (QG * BQ)), static_cast<unsigned>(H));
  if (int e = check_cuda(cudaFuncSetAttribute(attn_tok_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TOK_SMEM_BYTES),
                         "attn_tok smem attribute"))
    return e;
  attn_tok_kernel<<<grid, TOK_THREADS, TOK_SMEM_BYTES, stream>>>(tq, tk, tv, p);
  return check_cuda(cudaGetLastError(), "attn_int8_tok launch");
}
