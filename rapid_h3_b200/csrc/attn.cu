// INT8 flash attention for head_dim 128, non-causal, on the Blackwell tensor cores.
//
//   S = Q8 . K8^T            int8 x int8 -> int32 in TMEM (tcgen05 kind::i8), one 128x128 tile at a time
//   t = S * (qs[q block] * ks[k block] * softmax_scale * log2 e)      one scale per 64-token block
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
// One CTA = one 128-query tile of one head, 192 threads, two CTAs per SM (so one CTA's softmax
// overlaps the other's MMAs):
//   warp 0      TMA producer: Q once, then K tile (128 keys x 128 B) + V^T tile (128 ch x 128 keys)
//   warp 1      MMA issuer: QK^T of tile j+1 is issued before P.V of tile j
//   warps 2..5  one query row per thread: two passes over S in TMEM (max, then exp2 + fp8 pack),
//               P written to shared memory in the 128-byte-swizzled K-major layout the MMA reads
// Tensor-core bound: 4 * Lq * Lk * 128 operations per head.
#include <limits.h>

#include "common.cuh"
#include "rapidh3_b200.h"

namespace rh3 {
namespace {

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int TILE_BYTES = 128 * 128;  // every operand tile is 128 rows x 128 bytes
constexpr int KV_STAGES = 2;
constexpr int ATTN_THREADS = 192;

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
};

struct __align__(8) AttnSmemTail {
  uint64_t q_full;
  uint64_t kv_full[KV_STAGES];
  uint64_t kv_empty[KV_STAGES];
  uint64_t s_full, s_empty, p_full, pv_done;
  uint32_t tmem_base;
  int abort_flag;
};

constexpr int ATTN_SMEM_BYTES = (2 + 2 * KV_STAGES) * TILE_BYTES + sizeof(AttnSmemTail) + 1024;

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

__global__ void __launch_bounds__(ATTN_THREADS, 2)
attn_int8_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                 const __grid_constant__ CUtensorMap tma_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sP = smem + TILE_BYTES;
  uint8_t* sKV = smem + 2 * TILE_BYTES;  // stage s: K at +s*2*TILE, V^T at +s*2*TILE + TILE
  AttnSmemTail* tail = reinterpret_cast<AttnSmemTail*>(smem + (2 + 2 * KV_STAGES) * TILE_BYTES);
  volatile int* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tile = blockIdx.x, h = blockIdx.y;
  const int n_kv = (p.Lk + BKV - 1) / BKV;

  if (threadIdx.x == 0) {
    mbar_init(&tail->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&tail->kv_full[s], 1);
      mbar_init(&tail->kv_empty[s], 1);
    }
    mbar_init(&tail->s_full, 1);
    mbar_init(&tail->s_empty, 128);
    mbar_init(&tail->p_full, 128);
    mbar_init(&tail->pv_done, 1);
    tail->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&tail->tmem_base, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tail->tmem_base;
  const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + 128;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tma_q);
      tma_prefetch_desc(&tma_k);
      tma_prefetch_desc(&tma_v);
      mbar_arrive_expect_tx(&tail->q_full, TILE_BYTES);
      tma_load_2d(sQ, &tma_q, 0, h * p.Lq_pad + q_tile * BQ, &tail->q_full);
      for (int j = 0; j < n_kv; ++j) {
        const int stage = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(&tail->kv_empty[stage], ph ^ 1, abort_flag, p.status, ST_TIMEOUT_STAGE_EMPTY)) break;
        uint8_t* sk = sKV + stage * 2 * TILE_BYTES;
        mbar_arrive_expect_tx(&tail->kv_full[stage], 2 * TILE_BYTES);
        tma_load_2d(sk, &tma_k, 0, h * p.Lk_pad + j * BKV, &tail->kv_full[stage]);
        tma_load_2d(sk + TILE_BYTES, &tma_v, j * BKV, h * HD, &tail->kv_full[stage]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(2, 1, 1, BQ, BKV);  // s32 += s8 * s8
      constexpr uint32_t idesc_pv = make_idesc(1, 0, 0, BQ, HD);   // f32 += e4m3 * e4m3
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto issue_qk = [&](int j) {
        const uint32_t k_addr = smem_u32(sKV + (j % KV_STAGES) * 2 * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          mma_i8_ss(tmem_S, make_desc_k128(q_addr + k * 32), make_desc_k128(k_addr + k * 32), idesc_qk, k != 0);
        mma_commit(&tail->s_full);
      };
      bool ok = mbar_wait(&tail->q_full, 0, abort_flag, p.status, ST_TIMEOUT_TMA_FULL) &&
                mbar_wait(&tail->kv_full[0], 0, abort_flag, p.status, ST_TIMEOUT_TMA_FULL);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          const int ns = (j + 1) % KV_STAGES;
          if (!mbar_wait(&tail->kv_full[ns], ((j + 1) / KV_STAGES) & 1, abort_flag, p.status, ST_TIMEOUT_TMA_FULL) ||
              !mbar_wait(&tail->s_empty, j & 1, abort_flag, p.status, ST_TIMEOUT_ACC_EMPTY)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_qk(j + 1);
        }
        if (!mbar_wait(&tail->p_full, j & 1, abort_flag, p.status, ST_TIMEOUT_P_READY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const int stage = j % KV_STAGES;
        const uint32_t v_addr = smem_u32(sKV + stage * 2 * TILE_BYTES + TILE_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          mma_f8_ss(tmem_O, make_desc_k128(p_addr + k * 32), make_desc_k128(v_addr + k * 32), idesc_pv,
                    (j | k) != 0);
        mma_commit(&tail->kv_empty[stage]);
        mma_commit(&tail->pv_done);
      }
    }
  } else {
    // ------------------------------ softmax / correction / epilogue ------------------------------
    const int quad = warp & 3;
    const int row = quad * 32 + lane;  // row of the tile = TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const int64_t q_row = static_cast<int64_t>(q_tile) * BQ + row;
    const float c_row = __fmul_rn(p.qs[static_cast<int64_t>(h) * (p.Lq_pad / 64) + (q_row >> 6)], p.sl2);
    const float* ks_h = p.ks + static_cast<int64_t>(h) * (p.Lk_pad / 64);
    uint8_t* p_row = sP + row * 128;
    const int sw = row & 7;
    float Mi = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait(&tail->s_full, j & 1, abort_flag, p.status, ST_TIMEOUT_ACC_FULL)) { ok = false; break; }
      tc_fence_after();
      const float c0 = __fmul_rn(c_row, ks_h[2 * j]), c1 = __fmul_rn(c_row, ks_h[2 * j + 1]);
      const int valid = min(BKV, p.Lk - j * BKV);
      // ---- pass 1: row maximum in scaled units ----
      float mloc = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_S + lane_off + c * 32, r);
        tmem_ld_wait();
        int imax = INT_MIN;
        if (valid == BKV) {
#pragma unroll
          for (int i = 0; i < 32; ++i) imax = max(imax, static_cast<int>(r[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < valid) imax = max(imax, static_cast<int>(r[i]));
        }
        if (imax != INT_MIN) mloc = fmaxf(mloc, __fmul_rn(__int2float_rn(imax), c < 2 ? c0 : c1));
      }
      const float Mi_new = fmaxf(Mi, ceilf(mloc));
      const bool grow = Mi_new > Mi;
      if (j > 0) {
        // P.V of the previous tile has finished: O is complete up to tile j-1 and the P buffer is free
        if (!mbar_wait(&tail->pv_done, (j - 1) & 1, abort_flag, p.status, ST_TIMEOUT_PV_DONE)) { ok = false; break; }
        if (__any_sync(0xffffffffu, grow)) {
          tc_fence_after();
          const float f = grow ? ex2_approx(Mi - Mi_new) : 1.f;  // exact power of two
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld32(tmem_O + lane_off + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * f);
            tmem_st32(tmem_O + lane_off + c * 32, r);
          }
          tmem_st_wait();
          l *= f;
        }
      }
      Mi = Mi_new;
      const float off = 8.f - Mi;
      // ---- pass 2: P = e4m3(2^(t - M + 8)) into shared memory, l += p ----
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_S + lane_off + c * 32, r);
        tmem_ld_wait();
        if (c == 3) {  // S has been read completely: the next Q.K^T may overwrite it
          tc_fence_before();
          mbar_arrive(&tail->s_empty);
        }
        const float cc = c < 2 ? c0 : c1;
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e = ex2_approx(fmaf(__int2float_rn(static_cast<int>(r[i])), cc, off));
          if (valid != BKV && c * 32 + i >= valid) e = 0.f;
          pv[i] = e;
          l += e;
        }
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = pack_e4m3x4(pv[4 * i], pv[4 * i + 1], pv[4 * i + 2], pv[4 * i + 3]);
        *reinterpret_cast<uint4*>(p_row + (((2 * c) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(p_row + (((2 * c + 1) ^ sw) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&tail->p_full);
    }
    // ---- epilogue ----
    if (ok && mbar_wait(&tail->pv_done, (n_kv - 1) & 1, abort_flag, p.status, ST_TIMEOUT_PV_DONE)) {
      tc_fence_after();
      const float inv_l = __fdiv_rn(1.f, l);
      const float* vs = p.vscale + h * HD;
      const float* vm = p.vmean + h * HD;
      __nv_bfloat16* o = p.out + q_row * p.o_ss + static_cast<int64_t>(h) * p.o_sh;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_O + lane_off + c * 32, r);
        tmem_ld_wait();
        if (q_row < p.Lq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int d = c * 32 + g * 8 + 2 * i;
              const float a = fmaf(__uint_as_float(r[g * 8 + 2 * i]) * inv_l, vs[d], vm[d]);
              const float b = fmaf(__uint_as_float(r[g * 8 + 2 * i + 1]) * inv_l, vs[d + 1], vm[d + 1]);
              w[i] = pack_bf16x2(a, b);
            }
            *reinterpret_cast<uint4*>(o + c * 32 + g * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
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
    tmem_dealloc(tmem_base, 256);
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace rh3

using namespace rh3;

extern "C" int rh3_attn_int8(const void* q8, const float* qs, const void* k8, const float* ks, const void* vt,
                             const float* vscale, const float* vmean, int64_t Lq, int64_t Lq_pad, int64_t Lk,
                             int64_t Lk_pad, int64_t H, float softmax_scale, void* out, int64_t o_ss, int64_t o_sh,
                             cudaStream_t stream) {
  RH3_CHECK_ARG(Lq > 0 && Lk > 0 && H > 0 && H < 65536, "attn_int8: bad shape Lq=%lld Lk=%lld H=%lld", (long long)Lq,
                (long long)Lk, (long long)H);
  RH3_CHECK_ARG(Lq_pad >= Lq && Lk_pad >= Lk && Lq_pad % 128 == 0 && Lk_pad % 128 == 0,
                "attn_int8: padded lengths must be multiples of 128 and cover Lq / Lk");
  RH3_CHECK_ARG(H * Lq_pad < (1ll << 31) && H * Lk_pad < (1ll << 31), "attn_int8: H * Lpad too large");
  RH3_CHECK_ARG(q8 && qs && k8 && ks && vt && vscale && vmean && out, "attn_int8: null pointer");
  RH3_CHECK_ARG(aligned16(q8) && aligned16(k8) && aligned16(vt) && aligned16(out) && o_ss % 8 == 0 && o_sh % 8 == 0,
                "attn_int8: operands must be 16-byte aligned, output strides multiples of 8 elements");
  RH3_CHECK_ARG(softmax_scale > 0.f, "attn_int8: softmax scale must be positive");
  CUtensorMap tq, tk, tv;
  if (int e = make_tmap_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q8, HD, H * Lq_pad, HD, HD, BQ,
                           CU_TENSOR_MAP_SWIZZLE_128B))
    return e;
  if (int e = make_tmap_2d(&tk, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k8, HD, H * Lk_pad, HD, HD, BKV,
                           CU_TENSOR_MAP_SWIZZLE_128B))
    return e;
  if (int e = make_tmap_2d(&tv, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, vt, Lk_pad, H * HD, Lk_pad, BKV, HD,
                           CU_TENSOR_MAP_SWIZZLE_128B))
    return e;
  AttnParams p{};
  p.qs = qs; p.ks = ks; p.vscale = vscale; p.vmean = vmean;
  p.out = static_cast<__nv_bfloat16*>(out); p.o_ss = o_ss; p.o_sh = o_sh;
  p.Lq = (int)Lq; p.Lk = (int)Lk; p.Lq_pad = (int)Lq_pad; p.Lk_pad = (int)Lk_pad; p.H = (int)H;
  p.sl2 = static_cast<float>(static_cast<double>(softmax_scale) * 1.4426950408889634);
  p.status = device_status_word();
  if (int e = check_cuda(cudaFuncSetAttribute(attn_int8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              ATTN_SMEM_BYTES),
                         "attn smem attribute"))
    return e;
  const dim3 grid(static_cast<unsigned>((Lq + BQ - 1) / BQ), static_cast<unsigned>(H));
  attn_int8_kernel<<<grid, ATTN_THREADS, ATTN_SMEM_BYTES, stream>>>(tq, tk, tv, p);
  return check_cuda(cudaGetLastError(), "attn_int8 launch");
}
