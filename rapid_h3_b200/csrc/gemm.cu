// Row-wise-scaled W8A8 GEMM on the Blackwell tensor cores.
//
//   acc[m, n] = sum_k xq[m, k] * wq[n, k]          int8 x int8 -> int32 (tcgen05 kind::i8), or
//                                                   e4m3 x e4m3 -> fp32 (tcgen05 kind::f8f6f4)
//   EPI_PLAIN : out[m, n]   = bf16(((float(acc) * xs[m]) * ws[n]) + bias[n])
//   EPI_GATED : resid[m, n] = bf16(fma(bf16((float(acc) * xs[m]) * ws[n]), gate[n], resid[m, n]))   (in place)
//   EPI_SWIGLU: columns come in groups of 8 = [g 4j..4j+3 | u 4j..4j+3];
//               out[m, n/2] = bf16(silu(bf16(g)) * bf16(u)), half-width store
// (reference: custom_nodes/rapid_h3/csrc/fp8_rowwise.cu:294-304 plain epilogue, :333-336 gated
//  residual, :74-93 SwiGLU store; PyTorch emulation custom_nodes/rapid_h3/kernels.py:129-137).
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: 128x128-byte A tile + 256x128-byte B tile per stage, 4-stage ring
//   warp 1      MMA issuer: 4 x tcgen05.mma (M128 N256 K32) per stage into a TMEM accumulator;
//               two 256-column accumulators so the epilogue of tile i overlaps the main loop of i+1
//   warps 2..5  epilogue: tcgen05.ld 32 columns at a time, dequantize, fused epilogue, 64-byte
//               contiguous bf16 stores per thread-row
// Tensor-core bound: 2*M*N*K operations per call.

#include <atomic>

#include "common.cuh"
#include "rapidh3_b200.h"

namespace rh3 {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;  // bytes (= elements for 8-bit operands) along K per stage
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK;
constexpr int B_BYTES = BN * BK;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;
#ifndef RH3_GEMM_GROUP_M
#define RH3_GEMM_GROUP_M 16
#endif
constexpr int GROUP_M = RH3_GEMM_GROUP_M;  // tile rasterisation: GROUP_M row-tiles share each column-tile in L2

enum { EPI_PLAIN = 0, EPI_GATED = 1, EPI_SWIGLU = 2, EPI_F16 = 3, EPI_SWIGLU_F16 = 4 };

struct GemmParams {
  int M, N, K;
  const float* xs;
  const float* ws;
  const __nv_bfloat16* bias;  // EPI_PLAIN, optional
  __nv_bfloat16* out;         // EPI_PLAIN / EPI_SWIGLU
  int64_t ldo;
  int32_t* acc_dump;          // optional raw accumulator dump [M, N] (int32, or fp32 bits for fp8)
  const __nv_bfloat16* gate;  // EPI_GATED
  __nv_bfloat16* resid;       // EPI_GATED
  int64_t ldr;
  // fp16 epilogues of the VAE transformer decoder (EPI_F16 / EPI_SWIGLU_F16)
  const __half* bias_h;    // [N]
  const __half* rscale_h;  // [N] or null (EPI_F16 with residual)
  const __half* resid_h;   // [M, N] row stride ldr, or null
  __half* out_h;           // row stride ldo
  int wide;                // bf16 output (and gated residual) rows are 32-byte aligned: 32-byte accesses in the epilogue
  int* status;
};

struct __align__(8) GemmSmemTail {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  float ws[BN];
  float aux[BN];   // bias or gate as fp32
  float aux2[BN];  // residual scale as fp32 (EPI_F16)
};

constexpr int GEMM_SMEM_BYTES = STAGES * STAGE_BYTES + sizeof(GemmSmemTail) + 1024;  // +1024 alignment slack

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& m_blk, int& n_blk) {
  const int per_group = GROUP_M * num_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gsize = min(GROUP_M, num_m - first_m);
  const int t = tile - g * per_group;
  m_blk = first_m + t % gsize;
  n_blk = t / gsize;
}

// The epilogue of one accumulator row: 256 columns, 32 at a time from TMEM, dequantized and stored through the fused
// epilogue EPI. `t_row` = TMEM address of this thread's row (lane) at the accumulator's first column.
// The residual row of an epilogue that adds one (gated residual, fp16 residual): its BN columns are asked into L2
// while the tile's MMAs still run, so the epilogue's loads do not wait on HBM (the residual of a step is far
// larger than L2 and cold by the time its tile comes up).
template <int EPI>
__device__ __forceinline__ void prefetch_residual(const GemmParams& p, int row, bool row_ok, int n0) {
  if (!row_ok) return;
  if (EPI == EPI_GATED) {
    const __nv_bfloat16* r = p.resid + static_cast<int64_t>(row) * p.ldr + n0;
#pragma unroll
    for (int c = 0; c < BN; c += 64)
      if (n0 + c < p.N) prefetch_l2(r + c);
  } else if (EPI == EPI_F16) {
    if (p.resid_h) {
      const __half* r = p.resid_h + static_cast<int64_t>(row) * p.ldr + n0;
#pragma unroll
      for (int c = 0; c < BN; c += 64)
        if (n0 + c < p.N) prefetch_l2(r + c);
    }
  }
}

// 32 bf16 outputs of one row (four 16-byte groups) to o: 32-byte stores where the row allows it, 16-byte stores for
// what remains in range otherwise.
__device__ __forceinline__ void store_chunk_bf16(__nv_bfloat16* o, const uint4* w4, int col0, int N, int wide) {
#pragma unroll
  for (int g = 0; g < 4; g += 2) {
    if (wide && col0 + g * 8 + 16 <= N) {
      st_global_32(o + g * 8, w4[g], w4[g + 1]);
    } else {
      if (col0 + g * 8 + 8 <= N) *reinterpret_cast<uint4*>(o + g * 8) = w4[g];
      if (col0 + g * 8 + 16 <= N) *reinterpret_cast<uint4*>(o + g * 8 + 8) = w4[g + 1];
    }
  }
}

// The gated residual's values of chunks c and c + 1 of a row (eight 16-byte pieces; zeros off the edge).
__device__ __forceinline__ void load_gated_residual(const GemmParams& p, int row, bool row_ok, int n0, int c, uint4* dst) {
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const int col0 = n0 + (c + q) * 32;
    const __nv_bfloat16* o = p.resid + static_cast<int64_t>(row) * p.ldr + col0;
#pragma unroll
    for (int g = 0; g < 4; g += 2) {
      if (p.wide && row_ok && col0 + g * 8 + 16 <= p.N) {
        ld_global_32(o + g * 8, dst[q * 4 + g], dst[q * 4 + g + 1]);
      } else {
        dst[q * 4 + g] = (row_ok && col0 + g * 8 + 8 <= p.N) ? *reinterpret_cast<const uint4*>(o + g * 8) : make_uint4(0, 0, 0, 0);
        dst[q * 4 + g + 1] = (row_ok && col0 + g * 8 + 16 <= p.N) ? *reinterpret_cast<const uint4*>(o + g * 8 + 8) : make_uint4(0, 0, 0, 0);
      }
    }
  }
}

template <int KIND_F8, int EPI>
__device__ __forceinline__ void epilogue_row(const GemmParams& p, const GemmSmemTail* tail, uint32_t t_row, int row,
                                             bool row_ok, float xs, int n0, const uint4* res0) {
  // two 32-column chunks are loaded per wait, so a tile costs four TMEM round trips instead of eight; `old4` = the
  // chunk's residual values (gated residual only), loaded one round trip ahead
  auto chunk = [&](const uint32_t* r, int c, const uint4* old4) {
    const int col0 = n0 + c * 32;
    if (row_ok && col0 < p.N) {
      if (p.acc_dump) {
        int32_t* d = p.acc_dump + static_cast<int64_t>(row) * p.N + col0;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          if (col0 + j + 4 <= p.N) *reinterpret_cast<uint4*>(d + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
      }
      float y[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float a = KIND_F8 ? __uint_as_float(r[j]) : __int2float_rn(static_cast<int>(r[j]));
        y[j] = __fmul_rn(__fmul_rn(a, xs), tail->ws[c * 32 + j]);
      }
      if (EPI == EPI_PLAIN) {
        __nv_bfloat16* o = p.out + static_cast<int64_t>(row) * p.ldo + col0;
        uint4 w4[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int e = g * 8 + 2 * j;
            w[j] = pack_bf16x2(__fadd_rn(y[e], tail->aux[c * 32 + e]), __fadd_rn(y[e + 1], tail->aux[c * 32 + e + 1]));
          }
          w4[g] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        store_chunk_bf16(o, w4, col0, p.N, p.wide);
      } else if (EPI == EPI_GATED) {
        __nv_bfloat16* o = p.resid + static_cast<int64_t>(row) * p.ldr + col0;
        uint4 w4[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint4 old = old4[g];
          const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int e = g * 8 + 2 * j;
            const float v0 = fmaf(bf16_round(y[e]), tail->aux[c * 32 + e], bf16_lo(ow[j]));
            const float v1 = fmaf(bf16_round(y[e + 1]), tail->aux[c * 32 + e + 1], bf16_hi(ow[j]));
            w[j] = pack_bf16x2(v0, v1);
          }
          w4[g] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        store_chunk_bf16(o, w4, col0, p.N, p.wide);
      } else if (EPI == EPI_F16) {
        // y1 = fp16(y + bias); with a residual: out = fp16(float(y1) * rscale + resid), two separate roundings
        __half* o = p.out_h + static_cast<int64_t>(row) * p.ldo + col0;
        const __half* rs = p.resid_h ? p.resid_h + static_cast<int64_t>(row) * p.ldr + col0 : nullptr;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          if (col0 + g * 8 + 8 <= p.N) {
            uint4 old = make_uint4(0, 0, 0, 0);
            if (rs) old = *reinterpret_cast<const uint4*>(rs + g * 8);
            const __half2* oh = reinterpret_cast<const __half2*>(&old);
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int e = g * 8 + 2 * j;
              float v0 = __half2float(__float2half_rn(__fadd_rn(y[e], tail->aux[c * 32 + e])));
              float v1 = __half2float(__float2half_rn(__fadd_rn(y[e + 1], tail->aux[c * 32 + e + 1])));
              if (rs) {
                const float2 r2 = __half22float2(oh[j]);
                v0 = __fadd_rn(__fmul_rn(v0, tail->aux2[c * 32 + e]), r2.x);
                v1 = __fadd_rn(__fmul_rn(v1, tail->aux2[c * 32 + e + 1]), r2.y);
              }
              const __half2 h2 = __floats2half2_rn(v0, v1);
              w[j] = *reinterpret_cast<const uint32_t*>(&h2);
            }
            *reinterpret_cast<uint4*>(o + g * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      } else if (EPI == EPI_SWIGLU_F16) {
        // columns in groups of 8 = [g0..g3 | u0..u3]; g, u = fp16(y + bias); out = fp16(g / (1 + e^-g) * u)
        __half* o = p.out_h + static_cast<int64_t>(row) * p.ldo + (col0 >> 1);
#pragma unroll
        for (int hgrp = 0; hgrp < 2; ++hgrp) {
          if (col0 + hgrp * 16 + 16 <= p.N) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const int b = hgrp * 16 + q * 8;
              float h[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float gv = __half2float(__float2half_rn(__fadd_rn(y[b + j], tail->aux[c * 32 + b + j])));
                const float uv = __half2float(__float2half_rn(__fadd_rn(y[b + 4 + j], tail->aux[c * 32 + b + 4 + j])));
                h[j] = gv / (1.f + __expf(-gv)) * uv;
              }
              const __half2 h01 = __floats2half2_rn(h[0], h[1]), h23 = __floats2half2_rn(h[2], h[3]);
              w[q * 2] = *reinterpret_cast<const uint32_t*>(&h01);
              w[q * 2 + 1] = *reinterpret_cast<const uint32_t*>(&h23);
            }
            *reinterpret_cast<uint4*>(o + hgrp * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      } else {  // EPI_SWIGLU: 32 columns = 4 groups of [g0..g3 | u0..u3] -> 16 outputs
        __nv_bfloat16* o = p.out + static_cast<int64_t>(row) * p.ldo + (col0 >> 1);
        uint4 w4[2];
#pragma unroll
        for (int hgrp = 0; hgrp < 2; ++hgrp) {  // 16 columns -> 8 outputs -> 16 bytes
          {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 2; ++q) {  // one group of 8 columns -> 4 outputs
              const int b = hgrp * 16 + q * 8;
              float h[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float gv = bf16_round(y[b + j]);
                const float uv = bf16_round(y[b + 4 + j]);
                h[j] = __fdividef(gv, 1.f + __expf(-gv)) * uv;
              }
              w[q * 2] = pack_bf16x2(h[0], h[1]);
              w[q * 2 + 1] = pack_bf16x2(h[2], h[3]);
            }
            w4[hgrp] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
        if (p.wide && col0 + 32 <= p.N) {
          st_global_32(o, w4[0], w4[1]);
        } else {
          if (col0 + 16 <= p.N) *reinterpret_cast<uint4*>(o) = w4[0];
          if (col0 + 32 <= p.N) *reinterpret_cast<uint4*>(o + 8) = w4[1];
        }
      }
    }
  };
  if (EPI == EPI_GATED) {
    // the residual of the next two chunks is fetched while the current two are computed (the loads of a row are
    // 16 bytes each from a cold 8 KB-strided row: waiting for them chunk by chunk was most of this epilogue's time)
    // (the first two chunks' values, `res0`, were fetched by the caller before it waited for the accumulator)
    uint4 res[2][8];
    auto load_res = [&](uint4* dst, int c) { load_gated_residual(p, row, row_ok, n0, c, dst); };
#pragma unroll
    for (int i = 0; i < 8; ++i) res[0][i] = res0[i];
#pragma unroll
    for (int it = 0; it < BN / 64; ++it) {
      const int c = it * 2;
      uint32_t ra[32], rb[32];
      tmem_ld32(t_row + c * 32, ra);
      tmem_ld32(t_row + c * 32 + 32, rb);
      if (it + 1 < BN / 64) load_res(res[(it + 1) & 1], c + 2);
      tmem_ld_wait_regs(ra);
      tmem_ld_wait_regs(rb);
      chunk(ra, c, res[it & 1]);
      chunk(rb, c + 1, res[it & 1] + 4);
    }
    return;
  }
#pragma unroll 1
  for (int c = 0; c < BN / 32; c += 2) {
    uint32_t ra[32], rb[32];
    tmem_ld32(t_row + c * 32, ra);
    tmem_ld32(t_row + c * 32 + 32, rb);
    tmem_ld_wait_regs(ra);
    tmem_ld_wait_regs(rb);
    chunk(ra, c, nullptr);
    chunk(rb, c + 1, nullptr);
  }
}

template <int KIND_F8, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_w8a8_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  GemmSmemTail* tail = reinterpret_cast<GemmSmemTail*>(smem + STAGES * STAGE_BYTES);
  volatile int* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&tail->full[s], 1);
      mbar_init(&tail->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tail->acc_full[b], 1);
      mbar_init(&tail->acc_empty[b], 4);  // one arrival per epilogue warp
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

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(tile, num_m, num_n, m_blk, n_blk);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&tail->empty[stage], phase ^ 1, abort_flag, p.status, ST_TIMEOUT_STAGE_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_arrive_expect_tx(&tail->full[stage], STAGE_BYTES);
          tma_load_2d(sa, &tma_a, kb * BK, m_blk * BM, &tail->full[stage]);
          tma_load_2d(sb, &tma_b, kb * BK, n_blk * BN, &tail->full[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    // The whole warp runs the loop, converged: waits, counters, addresses and descriptors are then warp-uniform
    // values the compiler can keep in the uniform datapath, where the MMA instruction takes its operands from; one
    // elected lane (the same every time) issues the MMAs and the commits. On the bare issue pattern of this loop
    // (rh3_selftest_mma_rate, patterns 1 and 3) a single lane in the loop reaches 3.2 POP/s and the converged warp
    // 4.5; in this kernel the two forms measure the same (2.7 POP/s at K = 4096), so the issuing thread is not what
    // holds the tensor pipe at 70 % here.
    constexpr uint32_t idesc = KIND_F8 ? make_idesc(1, 0, 0, BM, BN) : make_idesc(2, 1, 1, BM, BN);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      ok = __all_sync(0xffffffffu, mbar_wait(&tail->acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, ST_TIMEOUT_ACC_EMPTY));
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = 0; kb < num_kb; ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(&tail->full[stage], phase, abort_flag, p.status, ST_TIMEOUT_TMA_FULL));
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
        const uint32_t b_addr = a_addr + A_BYTES;
        if (elect_one()) {
          if (KIND_F8) mma4_f8_ss(d_tmem, make_desc_k128(a_addr), make_desc_k128(b_addr), idesc, kb != 0);
          else mma4_i8_ss(d_tmem, make_desc_k128(a_addr), make_desc_k128(b_addr), idesc, kb != 0);
          mma_commit(&tail->empty[stage]);  // the stage is free once these MMAs have read it
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      if (elect_one()) mma_commit(&tail->acc_full[acc]);
      __syncwarp();
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  } else {
    // ------------------------------ epilogue (warps 2..5) ------------------------------
    const int quad = warp & 3;           // TMEM lane quadrant this warp may read
    const int et = threadIdx.x - 64;     // 0..127
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int m_blk, n_blk;
      tile_coords(tile, num_m, num_n, m_blk, n_blk);
      const int n0 = n_blk * BN;
      // stage the per-column scale (and bias / gate) of this tile in shared memory
      asm volatile("bar.sync 1, 128;" ::: "memory");  // previous tile's readers are done
      for (int c = et; c < BN; c += 128) {
        const int n = n0 + c;
        tail->ws[c] = n < p.N ? p.ws[n] : 0.f;
        if (EPI == EPI_PLAIN) tail->aux[c] = (p.bias && n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
        if (EPI == EPI_GATED) tail->aux[c] = n < p.N ? __bfloat162float(p.gate[n]) : 0.f;
        if (EPI == EPI_F16 || EPI == EPI_SWIGLU_F16) tail->aux[c] = n < p.N ? __half2float(p.bias_h[n]) : 0.f;
        if (EPI == EPI_F16) tail->aux2[c] = (p.rscale_h && n < p.N) ? __half2float(p.rscale_h[n]) : 0.f;
      }
      const int row = m_blk * BM + quad * 32 + lane;
      const bool row_ok = row < p.M;
      if (tile == static_cast<int>(blockIdx.x)) prefetch_residual<EPI>(p, row, row_ok, n0);
      if (tile + static_cast<int>(gridDim.x) < num_tiles) {   // the next tile's residual, a whole epilogue ahead
        int m2, n2;
        tile_coords(tile + gridDim.x, num_m, num_n, m2, n2);
        const int row2 = m2 * BM + quad * 32 + lane;
        prefetch_residual<EPI>(p, row2, row2 < p.M, n2 * BN);
      }
      uint4 res0[8];
      if (EPI == EPI_GATED) load_gated_residual(p, row, row_ok, n0, 0, res0);
      // the four warps leave together: a warp that gave up its wait takes the others with it at this barrier
      // (which also publishes the staged columns), so none of them waits at the next tile's barrier alone
      const bool got = mbar_wait(&tail->acc_full[acc], acc_phase, abort_flag, p.status, ST_TIMEOUT_ACC_FULL);
      if (bar_sync_or(1, 128, !got)) break;
      tc_fence_after();
      const float xs = row_ok ? p.xs[row] : 0.f;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
      epilogue_row<KIND_F8, EPI>(p, tail, t_row, row, row_ok, xs, n0, res0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tail->acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ------------------------------ teardown ------------------------------
  __syncwarp();
  if (*abort_flag && threadIdx.x == 0) {
    // give copies that may still be in flight time to land before shared memory is released
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
// The same GEMM on CTA pairs (thread-block clusters of two, tcgen05 cta_group::2): a pair computes a 256 x 256 tile.
// CTA r of the pair loads A rows [128 r, 128 r + 128) and B rows (output columns) [128 r, 128 r + 128) of the tile
// into its own shared memory (32 KB per stage instead of 48: what an SM has to take in per 512 tensor cycles is
// what bounds the single-CTA kernel), one thread of the even CTA issues MMAs of 256 x 256 x 32 that read both CTAs'
// tiles, and each CTA's TMEM receives its 128 rows x 256 columns, which its own epilogue warps drain as before.
// Barriers: the TMA loads of both CTAs count their bytes on the even CTA's `full`; stage release and accumulator
// hand-over are commits to the barrier of each CTA in turn (no multicast form anywhere); the epilogue warps of both
// CTAs arrive on the even CTA's `acc_empty`. Every wait is bounded as in the single-CTA kernel; the two cluster-wide
// barriers (after set-up, before tear-down) are reached by every thread on every path.
// ---------------------------------------------------------------------------------------------
constexpr int P_STAGES = 6;
constexpr int P_B_BYTES = 128 * BK;                 // this CTA's half of B
constexpr int P_STAGE_BYTES = A_BYTES + P_B_BYTES;  // 32 KB

struct __align__(8) PairSmemTail {
  uint64_t full[P_STAGES];
  uint64_t empty[P_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  GemmSmemTail cols;   // ws / aux / aux2 staging of the epilogue (its barrier fields are unused here)
};
constexpr int PAIR_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + sizeof(PairSmemTail) + 1024;

template <int KIND_F8, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  PairSmemTail* tail = reinterpret_cast<PairSmemTail*>(smem + P_STAGES * P_STAGE_BYTES);
  volatile int* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();          // 0 = the even CTA of the pair: it issues the MMAs
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_m = (p.M + 2 * BM - 1) / (2 * BM), num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&tail->full[s], 1);     // the even CTA's: one arrive.expect_tx for the bytes of both CTAs
      mbar_init(&tail->empty[s], 1);    // one commit per CTA
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tail->acc_full[b], 1);
      mbar_init(&tail->acc_empty[b], 8);  // the even CTA's: one arrival per epilogue warp of both CTAs
    }
    tail->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(&tail->tmem_base, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers exist before anything arrives on them from the other side
  tc_fence_after();
  const uint32_t tmem_base = tail->tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (elect_one()) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
    }
    __syncwarp();
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      int m_blk, n_blk;
      tile_coords(tile, num_m, num_n, m_blk, n_blk);
      const int row0 = m_blk * 2 * BM + static_cast<int>(rank) * BM, col0 = n_blk * BN + static_cast<int>(rank) * 128;
      for (int kb = 0; kb < num_kb; ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(&tail->empty[stage], phase ^ 1, abort_flag, p.status, ST_TIMEOUT_STAGE_EMPTY));
        if (!ok) break;
        uint8_t* sa = smem + stage * P_STAGE_BYTES;
        const uint32_t leader_full = cluster_addr(&tail->full[stage], 0);
        if (elect_one()) {
          if (rank == 0) mbar_arrive_expect_tx(&tail->full[stage], 2 * P_STAGE_BYTES);
          tma_load_2d_pair(sa, &tma_a, kb * BK, row0, leader_full);
          tma_load_2d_pair(sa + A_BYTES, &tma_b, kb * BK, col0, leader_full);
        }
        __syncwarp();
        if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA only; converged warp, one elected lane) ------------------------------
    if (rank == 0) {
      constexpr uint32_t idesc = KIND_F8 ? make_idesc(1, 0, 0, 2 * BM, BN) : make_idesc(2, 1, 1, 2 * BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        ok = __all_sync(0xffffffffu, mbar_wait(&tail->acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, ST_TIMEOUT_ACC_EMPTY));
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = __all_sync(0xffffffffu, mbar_wait(&tail->full[stage], phase, abort_flag, p.status, ST_TIMEOUT_TMA_FULL));
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * P_STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
          const uint32_t empty0 = cluster_addr(&tail->empty[stage], 0), empty1 = cluster_addr(&tail->empty[stage], 1);
          if (elect_one()) {
            if (KIND_F8) mma4_f8_pair(d_tmem, make_desc_k128(a_addr), make_desc_k128(b_addr), idesc, kb != 0);
            else mma4_i8_pair(d_tmem, make_desc_k128(a_addr), make_desc_k128(b_addr), idesc, kb != 0);
            mma_commit_pair(empty0);   // the stage is free in both CTAs once these MMAs have read it
            mma_commit_pair(empty1);
          }
          __syncwarp();
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        const uint32_t full0 = cluster_addr(&tail->acc_full[acc], 0), full1 = cluster_addr(&tail->acc_full[acc], 1);
        if (elect_one()) {
          mma_commit_pair(full0);
          mma_commit_pair(full1);
        }
        __syncwarp();
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------ epilogue (warps 2..5 of both CTAs) ------------------------------
    const int quad = warp & 3;
    const int et = threadIdx.x - 64;
    GemmSmemTail* cols = &tail->cols;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs) {
      int m_blk, n_blk;
      tile_coords(tile, num_m, num_n, m_blk, n_blk);
      const int n0 = n_blk * BN;
      asm volatile("bar.sync 1, 128;" ::: "memory");  // previous tile's readers are done
      for (int c = et; c < BN; c += 128) {
        const int n = n0 + c;
        cols->ws[c] = n < p.N ? p.ws[n] : 0.f;
        if (EPI == EPI_PLAIN) cols->aux[c] = (p.bias && n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
        if (EPI == EPI_GATED) cols->aux[c] = n < p.N ? __bfloat162float(p.gate[n]) : 0.f;
        if (EPI == EPI_F16 || EPI == EPI_SWIGLU_F16) cols->aux[c] = n < p.N ? __half2float(p.bias_h[n]) : 0.f;
        if (EPI == EPI_F16) cols->aux2[c] = (p.rscale_h && n < p.N) ? __half2float(p.rscale_h[n]) : 0.f;
      }
      const int row = m_blk * 2 * BM + static_cast<int>(rank) * BM + quad * 32 + lane;
      const bool row_ok = row < p.M;
      if (tile == pair) prefetch_residual<EPI>(p, row, row_ok, n0);
      if (tile + num_pairs < num_tiles) {   // the next tile's residual, a whole epilogue ahead
        int m2, n2;
        tile_coords(tile + num_pairs, num_m, num_n, m2, n2);
        const int row2 = m2 * 2 * BM + static_cast<int>(rank) * BM + quad * 32 + lane;
        prefetch_residual<EPI>(p, row2, row2 < p.M, n2 * BN);
      }
      uint4 res0[8];
      if (EPI == EPI_GATED) load_gated_residual(p, row, row_ok, n0, 0, res0);
      const bool got = mbar_wait(&tail->acc_full[acc], acc_phase, abort_flag, p.status, ST_TIMEOUT_ACC_FULL);
      if (bar_sync_or(1, 128, !got)) break;
      tc_fence_after();
      const float xs = row_ok ? p.xs[row] : 0.f;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
      epilogue_row<KIND_F8, EPI>(p, cols, t_row, row, row_ok, xs, n0, res0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(&tail->acc_empty[acc], 0);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ------------------------------ teardown ------------------------------
  __syncwarp();
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // nothing of the other CTA is in flight towards this CTA's shared memory or barriers any more
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

std::atomic<int> g_use_pairs{1};

template <int KIND_F8, int EPI>
int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
  auto kern = gemm_pair_kernel<KIND_F8, EPI>;
  if (int e = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES),
                         "gemm pair smem attribute"))
    return e;
  const int num_tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + BN - 1) / BN);
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
  cfg.stream = stream;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  // as many pairs as can be resident at once (one CTA per SM), never more than there are tiles
  cfg.gridDim = dim3(2 * (device_sm_count() / 2));
  int max_clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess || max_clusters < 1)
    return set_error(RH3_ARG_ERROR, "gemm pair: no cluster of two CTAs can be resident");
  const int pairs = num_tiles < max_clusters ? num_tiles : max_clusters;
  cfg.gridDim = dim3(2 * pairs);
  if (int e = check_cuda(cudaLaunchKernelEx(&cfg, kern, ta, tb, p), "gemm pair launch")) return e;
  return check_cuda(cudaGetLastError(), "gemm pair launch");
}

template <int KIND_F8, int EPI>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb_pair, const GemmParams& p,
                cudaStream_t stream) {
  // pairs need more than one 128-row tile to be worth their 256-row tiles
  if (g_use_pairs.load(std::memory_order_relaxed) && p.M > BM && p.N > 128)
    return launch_gemm_pair<KIND_F8, EPI>(ta, tb_pair, p, stream);
  auto kern = gemm_w8a8_kernel<KIND_F8, EPI>;
  if (int e = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES),
                         "gemm smem attribute"))
    return e;
  const int num_tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  const int grid = num_tiles < device_sm_count() ? num_tiles : device_sm_count();
  kern<<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, stream>>>(ta, tb, p);
  return check_cuda(cudaGetLastError(), "gemm launch");
}

int gemm_common(const void* xq, int64_t lda, const void* wq, const float* xs, const float* ws, int64_t M, int64_t N,
                int64_t K, int kind, CUtensorMap* ta, CUtensorMap* tb, CUtensorMap* tb_pair) {
  RH3_CHECK_ARG(kind == RH3_KIND_I8 || kind == RH3_KIND_F8, "gemm_w8a8: kind must be RH3_KIND_I8 or RH3_KIND_F8");
  RH3_CHECK_ARG(M >= 0 && N > 0 && K > 0 && M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31),
                "gemm_w8a8: bad shape M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
  RH3_CHECK_ARG(K % 16 == 0, "gemm_w8a8: K=%lld must be a multiple of 16", (long long)K);
  RH3_CHECK_ARG(N % 8 == 0, "gemm_w8a8: N=%lld must be a multiple of 8", (long long)N);
  RH3_CHECK_ARG(lda >= K && lda % 16 == 0, "gemm_w8a8: xq row stride must be >= K and a multiple of 16");
  if (M == 0) return 0;
  RH3_CHECK_ARG(xq && wq && xs && ws, "gemm_w8a8: null pointer");
  RH3_CHECK_ARG((reinterpret_cast<uintptr_t>(xq) & 15) == 0 && (reinterpret_cast<uintptr_t>(wq) & 15) == 0,
                "gemm_w8a8: xq and wq must be 16-byte aligned");
  if (int e = make_tmap_2d(ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, K, M, lda, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B))
    return e;
  if (int e = make_tmap_2d(tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, K, N, K, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B))
    return e;
  // the CTA-pair kernel loads B in halves of 128 rows
  if (int e = make_tmap_2d(tb_pair, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, K, N, K, BK, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return e;
  return 0;
}

}  // namespace
int pairs_enabled() { return g_use_pairs.load(std::memory_order_relaxed); }
}  // namespace rh3

using namespace rh3;

// Selects the kernel the GEMM entries launch: 0 = one CTA per 128 x 256 tile, 1 (default) = CTA pairs on 256 x 256
// tiles (gemm_pair_kernel) for every call with more than 128 rows and more than 128 columns. Returns the previous
// setting. Results are identical (int32 accumulators, same epilogue). The convolution follows the same switch
// (conv3d_pair_kernel: fp32 accumulation in the same order, identical results).
extern "C" int rh3_gemm_use_pairs(int on) { return g_use_pairs.exchange(on ? 1 : 0); }

extern "C" int rh3_gemm_w8a8(const void* xq, int64_t lda, const void* wq, const float* xs, const float* ws,
                             const void* bias, int64_t M, int64_t N, int64_t K, int kind, void* out, int64_t ldo,
                             int32_t* acc_dump, cudaStream_t stream) {
  CUtensorMap ta, tb, tbp;
  if (int e = gemm_common(xq, lda, wq, xs, ws, M, N, K, kind, &ta, &tb, &tbp)) return e;
  if (M == 0) return 0;
  RH3_CHECK_ARG(out && ldo >= N && ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
                "gemm_w8a8: out must be 16-byte aligned with a row stride >= N that is a multiple of 8");
  RH3_CHECK_ARG(!acc_dump || (reinterpret_cast<uintptr_t>(acc_dump) & 15) == 0, "gemm_w8a8: acc_dump misaligned");
  GemmParams p{};
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.xs = xs; p.ws = ws;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.out = static_cast<__nv_bfloat16*>(out); p.ldo = ldo; p.acc_dump = acc_dump; p.status = device_status_word();
  p.wide = (reinterpret_cast<uintptr_t>(out) & 31) == 0 && ldo % 16 == 0;
  return kind == RH3_KIND_F8 ? launch_gemm<1, EPI_PLAIN>(ta, tb, tbp, p, stream) : launch_gemm<0, EPI_PLAIN>(ta, tb, tbp, p, stream);
}

extern "C" int rh3_gemm_w8a8_gated_residual(const void* xq, int64_t lda, const void* wq, const float* xs,
                                            const float* ws, const void* gate, void* resid, int64_t ldr, int64_t M,
                                            int64_t N, int64_t K, int kind, cudaStream_t stream) {
  CUtensorMap ta, tb, tbp;
  if (int e = gemm_common(xq, lda, wq, xs, ws, M, N, K, kind, &ta, &tb, &tbp)) return e;
  if (M == 0) return 0;
  RH3_CHECK_ARG(gate && resid && ldr >= N && ldr % 8 == 0 && (reinterpret_cast<uintptr_t>(resid) & 15) == 0,
                "gemm_w8a8_gated_residual: resid must be 16-byte aligned with a row stride >= N, multiple of 8");
  GemmParams p{};
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.xs = xs; p.ws = ws;
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.resid = static_cast<__nv_bfloat16*>(resid); p.ldr = ldr; p.status = device_status_word();
  p.wide = (reinterpret_cast<uintptr_t>(resid) & 31) == 0 && ldr % 16 == 0;
  return kind == RH3_KIND_F8 ? launch_gemm<1, EPI_GATED>(ta, tb, tbp, p, stream) : launch_gemm<0, EPI_GATED>(ta, tb, tbp, p, stream);
}

extern "C" int rh3_gemm_w8a8_swiglu(const void* xq, int64_t lda, const void* wq, const float* xs, const float* ws,
                                    int64_t M, int64_t N, int64_t K, int kind, void* out, int64_t ldo,
                                    cudaStream_t stream) {
  CUtensorMap ta, tb, tbp;
  if (int e = gemm_common(xq, lda, wq, xs, ws, M, N, K, kind, &ta, &tb, &tbp)) return e;
  RH3_CHECK_ARG(N % 16 == 0, "gemm_w8a8_swiglu: N=%lld must be a multiple of 16", (long long)N);
  if (M == 0) return 0;
  RH3_CHECK_ARG(out && ldo >= N / 2 && ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
                "gemm_w8a8_swiglu: out must be 16-byte aligned with a row stride >= N/2 that is a multiple of 8");
  GemmParams p{};
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.xs = xs; p.ws = ws;
  p.out = static_cast<__nv_bfloat16*>(out); p.ldo = ldo; p.status = device_status_word();
  p.wide = (reinterpret_cast<uintptr_t>(out) & 31) == 0 && ldo % 16 == 0;
  return kind == RH3_KIND_F8 ? launch_gemm<1, EPI_SWIGLU>(ta, tb, tbp, p, stream) : launch_gemm<0, EPI_SWIGLU>(ta, tb, tbp, p, stream);
}

// ---- fp16 epilogues: the reference's VAE transformer-decoder GEMMs (custom_nodes/rapid_h3/csrc/vae_ops.cu:150-227
// plain + bias and residual addcmul, :228-345 w1 + SwiGLU) ----
extern "C" int rh3_vae_gemm(const void* xq, int64_t lda, const void* wq, const float* xs, const float* ws,
                            const void* bias_f16, const void* rscale_f16, const void* resid_f16, int64_t ldr,
                            int64_t M, int64_t N, int64_t K, void* out_f16, int64_t ldo, cudaStream_t stream) {
  CUtensorMap ta, tb, tbp;
  if (int e = gemm_common(xq, lda, wq, xs, ws, M, N, K, RH3_KIND_I8, &ta, &tb, &tbp)) return e;
  if (M == 0) return 0;
  RH3_CHECK_ARG(bias_f16, "vae_gemm: bias is required (pass zeros for none)");
  RH3_CHECK_ARG(out_f16 && ldo >= N && ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(out_f16) & 15) == 0,
                "vae_gemm: out must be 16-byte aligned with a row stride >= N that is a multiple of 8");
  RH3_CHECK_ARG((rscale_f16 == nullptr) == (resid_f16 == nullptr), "vae_gemm: rscale and resid come together");
  RH3_CHECK_ARG(!resid_f16 || (ldr >= N && ldr % 8 == 0 && (reinterpret_cast<uintptr_t>(resid_f16) & 15) == 0),
                "vae_gemm: resid must be 16-byte aligned with a row stride >= N that is a multiple of 8");
  GemmParams p{};
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.xs = xs; p.ws = ws;
  p.bias_h = static_cast<const __half*>(bias_f16); p.rscale_h = static_cast<const __half*>(rscale_f16);
  p.resid_h = static_cast<const __half*>(resid_f16); p.ldr = ldr;
  p.out_h = static_cast<__half*>(out_f16); p.ldo = ldo; p.status = device_status_word();
  return launch_gemm<0, EPI_F16>(ta, tb, tbp, p, stream);
}

extern "C" int rh3_vae_gemm_swiglu(const void* xq, int64_t lda, const void* wq, const float* xs, const float* ws,
                                   const void* bias_f16, int64_t M, int64_t N, int64_t K, void* out_f16, int64_t ldo,
                                   cudaStream_t stream) {
  CUtensorMap ta, tb, tbp;
  if (int e = gemm_common(xq, lda, wq, xs, ws, M, N, K, RH3_KIND_I8, &ta, &tb, &tbp)) return e;
  RH3_CHECK_ARG(N % 16 == 0, "vae_gemm_swiglu: N=%lld must be a multiple of 16", (long long)N);
  if (M == 0) return 0;
  RH3_CHECK_ARG(bias_f16, "vae_gemm_swiglu: bias is required (pass zeros for none)");
  RH3_CHECK_ARG(out_f16 && ldo >= N / 2 && ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(out_f16) & 15) == 0,
                "vae_gemm_swiglu: out must be 16-byte aligned with a row stride >= N/2 that is a multiple of 8");
  GemmParams p{};
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.xs = xs; p.ws = ws;
  p.bias_h = static_cast<const __half*>(bias_f16);
  p.out_h = static_cast<__half*>(out_f16); p.ldo = ldo; p.status = device_status_word();
  return launch_gemm<0, EPI_SWIGLU_F16>(ta, tb, tbp, p, stream);
}
