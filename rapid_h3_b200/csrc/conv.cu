// Causal 3x3x3 convolution of the VAE decoder as an implicit GEMM on the Blackwell tensor cores, plus
// the GroupNorm + SiLU kernels that sit between convolutions.
//
//   x   [N, T, H, W, Cin]  bf16 channels-last          w [Cout, 27, Cin] bf16 (tap = (dt*3 + dh)*3 + dw)
//   out [N, T, H, W, Cout] bf16 = bf16( sum_{tap, ci} x[n, t+dt-2, h+dh-1, w+dw-1, ci] * w[co, tap, ci]
//                                      + bias[co] (+ residual[n, t, h, w, co]) )
//   zero padding: one pixel around H and W, two frames BEFORE t = 0 (causal: no frame after t is read).
//
// There is no im2col buffer: for every tap the A operand of the GEMM is a shifted box of the input,
// fetched by a 5-D TMA tensor copy whose out-of-range coordinates are filled with zeros (that is the
// padding). One output tile = bh x bw sites of one frame (bh * bw <= 128 rows of the MMA) x BN output
// channels; the K loop runs over 27 taps x Cin/64 channel chunks (64 bf16 = one 128-byte swizzled row).
// Same warp roles and double-buffered TMEM accumulators as the W8A8 GEMM; the ring has as many stages as fit in
// shared memory (4 of 48 KB at 256 output channels per tile, up to 12 for narrow tiles): a stage of a narrow tile
// holds few tensor cycles of work, and the ring has to cover the L2 latency with them.
// The epilogue also emits per-tile partial sums (sum, sum of squares of the rounded outputs) per
// GroupNorm group, so the statistics of the next GroupNorm cost no extra pass over the activations.
//
// No counterpart exists in the reference repository (its VAE fast path is a transformer decoder,
// custom_nodes/rapid_h3/vae_fast.py:430-437); the CPU oracle (oracle/vae.py) defines the arithmetic.
// Tensor-core bound: 2 * sites * Cout * Cin * 27 operations per call.
#include "common.cuh"
#include "rapidh3_b200.h"

namespace rh3 {
namespace {

constexpr int CBM = 128;        // MMA rows (output sites per tile, bh * bw of them used)
constexpr int CBK = 64;         // channels per K chunk (128 bytes of bf16)
constexpr int CA_BYTES = CBM * 128;
constexpr int CMAX_STAGES = 12;       // ring depth: as many stages of CA_BYTES + (weight rows) * 128 bytes as fit
constexpr int CTAIL_BYTES = 2048;     // barriers and the staged bias, in front of the ring
constexpr int CRING_MAX_BYTES = 227 * 1024 - 1024 - CTAIL_BYTES;   // what the ring may take (1 KB of alignment slack)
constexpr int CONV_THREADS = 192;
constexpr int GN_GROUPS = 32;

struct ConvParams {
  int N, T, H, W, Cin, Cout;
  int halo;            // frames that precede output frame 0 inside x (0: causal zero padding, 2: a time shard's halo)
  int bh, bw;          // tile of output sites inside a frame
  int tiles_h, tiles_w;
  int BN;              // output channels per tile (multiple of 16, <= 256)
  const __nv_bfloat16* bias;      // [Cout] or null
  const __nv_bfloat16* residual;  // [N,T,H,W,Cout] or null
  __nv_bfloat16* out;
  float* gn_part;      // [num_m_tiles * 4][32][2] partial (sum, sumsq) per GroupNorm group, or null
  int stages, stage_bytes;   // ring: stage_bytes = kch * chunk_bytes
  int wide;                  // out (and residual) rows are 32-byte aligned: 32-byte accesses in the epilogue
  int kch, chunk_bytes;      // K chunks per stage (one barrier round trip each), CA_BYTES + (weight rows a CTA loads) * 128
  int* status;
};

struct __align__(8) ConvSmemTail {
  uint64_t full[CMAX_STAGES];
  uint64_t empty[CMAX_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  float bias[256];
};

static_assert(sizeof(ConvSmemTail) <= CTAIL_BYTES, "tail does not fit");

struct TileCoord {
  int n, t, h0, w0, n_blk;
};

__device__ __forceinline__ TileCoord conv_tile(int tile, const ConvParams& p, int num_n) {
  // column tiles fastest: the CTAs running together share the same input boxes through L2
  TileCoord c;
  c.n_blk = tile % num_n;
  int m = tile / num_n;
  c.w0 = (m % p.tiles_w) * p.bw;
  m /= p.tiles_w;
  c.h0 = (m % p.tiles_h) * p.bh;
  m /= p.tiles_h;
  c.t = m % p.T;
  c.n = m / p.T;
  return c;
}

// GroupNorm partials of a warp's 32 rows over one 32-column chunk: the GS channels of a group are summed per row
// (in channel order), the 32 rows by an xor butterfly; lane 0 writes (sum, sum of squares) of every group the chunk
// holds. GS is a template parameter so that every index into y[] is static (a run-time group width sends the array
// to local memory, which made this loop the slowest part of the kernel).
template <int GS>
__device__ __forceinline__ void gn_partials_chunk(const float* y, float* part, int col0, int Cout, int lane) {
#pragma unroll
  for (int j0 = 0; j0 < 32; j0 += GS) {
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = j0; j < j0 + GS; ++j) {
      s1 += y[j];
      s2 += y[j] * y[j];
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      s1 += __shfl_xor_sync(0xffffffffu, s1, o);
      s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    const int grp = (col0 + j0) / GS;
    if (lane == 0 && col0 + j0 < Cout) {
      part[grp * 2] = s1;
      part[grp * 2 + 1] = s2;
    }
  }
}

// The residual values of a thread's output site are asked into L2 while the tile's MMAs still run.
__device__ __forceinline__ void conv_prefetch_residual(const ConvParams& p, const TileCoord& c, int n0, bool tile_ok,
                                                       int quad, int lane) {
  if (!p.residual || !tile_ok) return;
  const int m = quad * 32 + lane;
  const int hh = m / p.bw, ww = m - hh * p.bw;
  const int h = c.h0 + hh, w = c.w0 + ww;
  if (m >= p.bh * p.bw || h >= p.H || w >= p.W) return;
  const int64_t site = ((static_cast<int64_t>(c.n) * p.T + c.t) * p.H + h) * p.W + w;
  const __nv_bfloat16* r = p.residual + site * p.Cout + n0;
  for (int cb = 0; cb < p.BN && n0 + cb < p.Cout; cb += 64) prefetch_l2(r + cb);
}

// The epilogue of one output tile for one thread (= one output site): BN columns, 32 at a time from TMEM, bias and
// residual added, bf16 stored, GroupNorm partials of the warp's 32 rows. `acc_tmem` = TMEM address of the
// accumulator's first column; `tile_ok` false = this CTA has no tile here (the odd tile of a pair): nothing is stored.
__device__ __forceinline__ void conv_epilogue_tile(const ConvParams& p, const float* bias_s, uint32_t acc_tmem,
                                                   const TileCoord& c, int n0, int m_tile, bool tile_ok, int quad, int lane) {
  const int gs = p.Cout / GN_GROUPS;  // channels per GroupNorm group (used only when gn_part != null)
  const int m = quad * 32 + lane;
  const int hh = m / p.bw, ww = m - hh * p.bw;
  const int h = c.h0 + hh, w = c.w0 + ww;
  const bool row_ok = tile_ok && m < p.bh * p.bw && h < p.H && w < p.W;
  const int64_t site = ((static_cast<int64_t>(c.n) * p.T + c.t) * p.H + h) * p.W + w;
  const uint32_t t_row = acc_tmem + (static_cast<uint32_t>(quad * 32) << 16);
  float* part = (p.gn_part && tile_ok) ? p.gn_part + (static_cast<int64_t>(m_tile) * 4 + quad) * GN_GROUPS * 2 : nullptr;
  // the residual of a chunk is loaded one chunk ahead (zeros where there is none), so its latency is spent under the
  // previous chunk's arithmetic and the TMEM round trip instead of in front of the additions
  const bool has_res = p.residual && row_ok;
  uint4 res_next[4];
  auto load_res = [&](int cb, uint4* dst) {
    const int col0 = n0 + cb;
    const __nv_bfloat16* rs = p.residual + site * p.Cout + col0;
#pragma unroll
    for (int g = 0; g < 4; g += 2) {
      if (p.wide && has_res && cb < p.BN && col0 + g * 8 + 16 <= p.Cout) {
        ld_global_32(rs + g * 8, dst[g], dst[g + 1]);
      } else {
        dst[g] = (has_res && cb < p.BN && col0 + g * 8 + 8 <= p.Cout) ? *reinterpret_cast<const uint4*>(rs + g * 8)
                                                                       : make_uint4(0, 0, 0, 0);
        dst[g + 1] = (has_res && cb < p.BN && col0 + g * 8 + 16 <= p.Cout) ? *reinterpret_cast<const uint4*>(rs + g * 8 + 8)
                                                                            : make_uint4(0, 0, 0, 0);
      }
    }
  };
  load_res(0, res_next);
#pragma unroll 1
  for (int cb = 0; cb < p.BN; cb += 32) {
    uint32_t r[32];
    tmem_ld32(t_row + cb, r);
    uint4 res[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) res[g] = res_next[g];
    load_res(cb + 32, res_next);
    tmem_ld_wait_regs(r);
    const int col0 = n0 + cb;
    float y[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) y[j] = __uint_as_float(r[j]) + bias_s[cb + j];
    if (has_res) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        if (col0 + g * 8 + 8 <= p.Cout) {
          const uint4 v = res[g];
          const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            y[g * 8 + 2 * j] += bf16_lo(vw[j]);
            y[g * 8 + 2 * j + 1] += bf16_hi(vw[j]);
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) y[j] = row_ok ? bf16_round(y[j]) : 0.f;  // what is stored; rows off the edge add 0
    if (row_ok) {
      __nv_bfloat16* o = p.out + site * p.Cout + col0;
      uint4 w4[4];
#pragma unroll
      for (int g = 0; g < 4; ++g)
        w4[g] = make_uint4(pack_bf16x2(y[g * 8], y[g * 8 + 1]), pack_bf16x2(y[g * 8 + 2], y[g * 8 + 3]),
                           pack_bf16x2(y[g * 8 + 4], y[g * 8 + 5]), pack_bf16x2(y[g * 8 + 6], y[g * 8 + 7]));
#pragma unroll
      for (int g = 0; g < 4; g += 2) {
        if (p.wide && col0 + g * 8 + 16 <= p.Cout) {
          st_global_32(o + g * 8, w4[g], w4[g + 1]);
        } else {
          if (col0 + g * 8 + 8 <= p.Cout) *reinterpret_cast<uint4*>(o + g * 8) = w4[g];
          if (col0 + g * 8 + 16 <= p.Cout) *reinterpret_cast<uint4*>(o + g * 8 + 8) = w4[g + 1];
        }
      }
    }
    if (part) {
      // the group width is uniform over the launch; one instantiation per width keeps y[] in registers
      switch (gs) {
        case 1: gn_partials_chunk<1>(y, part, col0, p.Cout, lane); break;
        case 2: gn_partials_chunk<2>(y, part, col0, p.Cout, lane); break;
        case 4: gn_partials_chunk<4>(y, part, col0, p.Cout, lane); break;
        case 8: gn_partials_chunk<8>(y, part, col0, p.Cout, lane); break;
        case 16: gn_partials_chunk<16>(y, part, col0, p.Cout, lane); break;
        default: gn_partials_chunk<32>(y, part, col0, p.Cout, lane); break;
      }
    }
  }
}

template <int KCH>   // K chunks per ring stage
__global__ void __launch_bounds__(CONV_THREADS, 1)
conv3d_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_w,
              const ConvParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  ConvSmemTail* tail = reinterpret_cast<ConvSmemTail*>(smem);
  smem += CTAIL_BYTES;
  const int CSTAGES = p.stages, CSTAGE_BYTES = p.stage_bytes;
  volatile int* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_n = (p.Cout + p.BN - 1) / p.BN;
  const int num_m = p.N * p.T * p.tiles_h * p.tiles_w;
  const int num_tiles = num_m * num_n;
  const int chunks = p.Cin / CBK;
  const int num_kb = 27 * chunks;
  const uint32_t a_bytes = static_cast<uint32_t>(p.bh * p.bw) * 128u;
  const uint32_t b_bytes = static_cast<uint32_t>(p.BN) * 128u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < CSTAGES; ++s) {
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
      tma_prefetch_desc(&tma_x);
      tma_prefetch_desc(&tma_w);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TileCoord c = conv_tile(tile, p, num_n);
        for (int kb = 0; kb < num_kb; kb += KCH) {
          if (!mbar_wait(&tail->empty[stage], phase ^ 1, abort_flag, p.status, ST_TIMEOUT_STAGE_EMPTY)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&tail->full[stage], (a_bytes + b_bytes) * KCH);
#pragma unroll
          for (int q = 0; q < KCH; ++q) {
            const int tap = (kb + q) / chunks, cc = kb + q - tap * chunks;
            const int dt = tap / 9, dh = (tap / 3) % 3, dw = tap % 3;
            uint8_t* sa = smem + stage * CSTAGE_BYTES + q * p.chunk_bytes;
            // out-of-range coordinates (negative or past the edge) read zeros: spatial and causal padding
            tma_load_5d(sa, &tma_x, cc * CBK, c.w0 + dw - 1, c.h0 + dh - 1, c.t + dt - 2 + p.halo, c.n, &tail->full[stage]);
            tma_load_2d(sa + CA_BYTES, &tma_w, tap * p.Cin + cc * CBK, c.n_blk * p.BN, &tail->full[stage]);
          }
          if (++stage == CSTAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    // the whole warp runs the loop converged (waits, counters and addresses are warp-uniform); one elected lane, the
    // same every time, issues the MMAs and the commits
    const uint32_t idesc = make_idesc(1, 1, 1, CBM, p.BN);  // f32 += bf16 * bf16
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      ok = __all_sync(0xffffffffu, mbar_wait(&tail->acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, ST_TIMEOUT_ACC_EMPTY));
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * 256;
      for (int kb = 0; kb < num_kb; kb += KCH) {
        ok = __all_sync(0xffffffffu, mbar_wait(&tail->full[stage], phase, abort_flag, p.status, ST_TIMEOUT_TMA_FULL));
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + stage * CSTAGE_BYTES);
        if (elect_one()) {
          // per K chunk four MMAs of 16 bf16 (32 bytes) each along K; one commit for the whole stage
#pragma unroll
          for (int q = 0; q < KCH; ++q) {
            const uint32_t aq = a_addr + q * p.chunk_bytes;
            mma4_f16_ss(d_tmem, make_desc_k128(aq), make_desc_k128(aq + CA_BYTES), idesc, (kb + q) != 0);
          }
          mma_commit(&tail->empty[stage]);
        }
        __syncwarp();
        if (++stage == CSTAGES) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      if (elect_one()) mma_commit(&tail->acc_full[acc]);
      __syncwarp();
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  } else {
    // ------------------------------ epilogue (warps 2..5) ------------------------------
    const int quad = warp & 3;
    const int et = threadIdx.x - 64;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const TileCoord c = conv_tile(tile, p, num_n);
      const int n0 = c.n_blk * p.BN;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      for (int i = et; i < p.BN; i += 128)
        tail->bias[i] = (p.bias && n0 + i < p.Cout) ? __bfloat162float(p.bias[n0 + i]) : 0.f;
      // the four warps leave together: a warp that gave up its wait takes the others with it at this barrier
      // (which also publishes the staged bias), so none of them waits at the next tile's barrier alone
      if (tile == static_cast<int>(blockIdx.x)) conv_prefetch_residual(p, c, n0, true, quad, lane);
      if (tile + static_cast<int>(gridDim.x) < num_tiles) {   // the next tile's residual, a whole epilogue ahead
        const TileCoord c2 = conv_tile(tile + gridDim.x, p, num_n);
        conv_prefetch_residual(p, c2, c2.n_blk * p.BN, true, quad, lane);
      }
      const bool got = mbar_wait(&tail->acc_full[acc], acc_phase, abort_flag, p.status, ST_TIMEOUT_ACC_FULL);
      if (bar_sync_or(1, 128, !got)) break;
      tc_fence_after();
      conv_epilogue_tile(p, tail->bias, tmem_base + acc * 256, c, n0, tile / num_n, true, quad, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tail->acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

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

// ---------------------------------------------------------------------------------------------
// The same convolution on CTA pairs (clusters of two, tcgen05 cta_group::2). A pair computes two neighbouring site
// tiles (m = 2 * pair_m + rank) x BN output channels with MMAs of 256 rows: every CTA fetches the shifted input box of
// its own site tile and HALF of the BN weight rows (rank r: rows [r * BN/2, (r+1) * BN/2) of the column tile), so an
// SM takes in 16 KB + BN/2 * 128 B per K chunk instead of 16 KB + BN * 128 B: the single-CTA kernel is bound by that
// ingest, not by the tensor pipe. Each CTA's TMEM receives its own 128 sites x BN channels and its own epilogue
// warps drain them exactly as in the single-CTA kernel (same fp32 accumulation order: results are identical).
// When the number of site tiles is odd, the odd CTA of the last pair loads the last valid tile again and stores nothing.
// Barriers as in the GEMM's pair kernel: both CTAs' loads count on the even CTA's `full`; stage release and
// accumulator hand-over are one commit per CTA; every wait is bounded; the two cluster barriers are reached by all.
// ---------------------------------------------------------------------------------------------

struct __align__(8) ConvPairSmemTail {
  uint64_t full[CMAX_STAGES];
  uint64_t empty[CMAX_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  float bias[256];
};
static_assert(sizeof(ConvPairSmemTail) <= CTAIL_BYTES, "tail does not fit");

// site tile m and column tile of pair-tile index `tile` for CTA `rank`: column tiles fastest, then pairs of site tiles
__device__ __forceinline__ void conv_pair_tile(int tile, int rank, int num_m, int num_n, int& m, int& n_blk, bool& ok) {
  n_blk = tile % num_n;
  m = (tile / num_n) * 2 + rank;
  ok = m < num_m;
  if (!ok) m = num_m - 1;
}

template <int KCH>   // K chunks per ring stage
__global__ void __launch_bounds__(CONV_THREADS, 1)
conv3d_pair_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_w,
                   const ConvParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  ConvPairSmemTail* tail = reinterpret_cast<ConvPairSmemTail*>(smem);
  smem += CTAIL_BYTES;
  const int CP_STAGES = p.stages, CP_STAGE_BYTES = p.stage_bytes;
  volatile int* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_cta_rank());   // 0 = the even CTA: it issues the MMAs
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_n = (p.Cout + p.BN - 1) / p.BN;
  const int num_m = p.N * p.T * p.tiles_h * p.tiles_w;
  const int num_tiles = ((num_m + 1) >> 1) * num_n;
  const int chunks = p.Cin / CBK;
  const int num_kb = 27 * chunks;
  const int half_n = p.BN >> 1;
  const uint32_t stage_tx = 2u * (static_cast<uint32_t>(p.bh * p.bw) * 128u + static_cast<uint32_t>(half_n) * 128u);

  if (threadIdx.x == 0) {
    for (int s = 0; s < CP_STAGES; ++s) {
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
      tma_prefetch_desc(&tma_x);
      tma_prefetch_desc(&tma_w);
    }
    __syncwarp();
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      int m, n_blk;
      bool tile_ok;
      conv_pair_tile(tile, rank, num_m, num_n, m, n_blk, tile_ok);
      const TileCoord c = conv_tile(m * num_n + n_blk, p, num_n);
      const int wrow0 = n_blk * p.BN + rank * half_n;
      for (int kb = 0; kb < num_kb; kb += KCH) {
        ok = __all_sync(0xffffffffu, mbar_wait(&tail->empty[stage], phase ^ 1, abort_flag, p.status, ST_TIMEOUT_STAGE_EMPTY));
        if (!ok) break;
        const uint32_t leader_full = cluster_addr(&tail->full[stage], 0);
        if (elect_one()) {
          if (rank == 0) mbar_arrive_expect_tx(&tail->full[stage], stage_tx * KCH);
#pragma unroll
          for (int q = 0; q < KCH; ++q) {
            const int tap = (kb + q) / chunks, cc = kb + q - tap * chunks;
            const int dt = tap / 9, dh = (tap / 3) % 3, dw = tap % 3;
            uint8_t* sa = smem + stage * CP_STAGE_BYTES + q * p.chunk_bytes;
            tma_load_5d_pair(sa, &tma_x, cc * CBK, c.w0 + dw - 1, c.h0 + dh - 1, c.t + dt - 2 + p.halo, c.n, leader_full);
            tma_load_2d_pair(sa + CA_BYTES, &tma_w, tap * p.Cin + cc * CBK, wrow0, leader_full);
          }
        }
        __syncwarp();
        if (++stage == CP_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA only; converged warp, one elected lane) ------------------------------
    if (rank == 0) {
      const uint32_t idesc = make_idesc(1, 1, 1, 2 * CBM, p.BN);  // f32 += bf16 * bf16, 256 rows over the pair
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        ok = __all_sync(0xffffffffu, mbar_wait(&tail->acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, ST_TIMEOUT_ACC_EMPTY));
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * 256;
        for (int kb = 0; kb < num_kb; kb += KCH) {
          ok = __all_sync(0xffffffffu, mbar_wait(&tail->full[stage], phase, abort_flag, p.status, ST_TIMEOUT_TMA_FULL));
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * CP_STAGE_BYTES);
          const uint32_t empty0 = cluster_addr(&tail->empty[stage], 0), empty1 = cluster_addr(&tail->empty[stage], 1);
          if (elect_one()) {
  #pragma unroll
          for (int q = 0; q < KCH; ++q) {
              const uint32_t aq = a_addr + q * p.chunk_bytes;
              mma4_f16_pair(d_tmem, make_desc_k128(aq), make_desc_k128(aq + CA_BYTES), idesc, (kb + q) != 0);
            }
            mma_commit_pair(empty0);   // the stage is free in both CTAs once these MMAs have read it
            mma_commit_pair(empty1);
          }
          __syncwarp();
          if (++stage == CP_STAGES) { stage = 0; phase ^= 1; }
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
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs) {
      int m, n_blk;
      bool tile_ok;
      conv_pair_tile(tile, rank, num_m, num_n, m, n_blk, tile_ok);
      const TileCoord c = conv_tile(m * num_n + n_blk, p, num_n);
      const int n0 = n_blk * p.BN;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      for (int i = et; i < p.BN; i += 128)
        tail->bias[i] = (p.bias && n0 + i < p.Cout) ? __bfloat162float(p.bias[n0 + i]) : 0.f;
      if (tile == pair) conv_prefetch_residual(p, c, n0, tile_ok, quad, lane);
      if (tile + num_pairs < num_tiles) {   // the next tile's residual, a whole epilogue ahead
        int m2, nb2;
        bool ok2;
        conv_pair_tile(tile + num_pairs, rank, num_m, num_n, m2, nb2, ok2);
        conv_prefetch_residual(p, conv_tile(m2 * num_n + nb2, p, num_n), nb2 * p.BN, ok2, quad, lane);
      }
      const bool got = mbar_wait(&tail->acc_full[acc], acc_phase, abort_flag, p.status, ST_TIMEOUT_ACC_FULL);
      if (bar_sync_or(1, 128, !got)) break;
      tc_fence_after();
      conv_epilogue_tile(p, tail->bias, tmem_base + acc * 256, c, n0, m, tile_ok, quad, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(&tail->acc_empty[acc], 0);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

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

// ---------------------------------------------------------------------------------------------
// GroupNorm statistics from the convolution's partials, GroupNorm + SiLU, causal 2x upsampling
// ---------------------------------------------------------------------------------------------
// sums[n][g] = (sum, sum of squares) over all row blocks of sample n, added in a fixed order in fp64.
__global__ void __launch_bounds__(256) gn_reduce_kernel(const float* __restrict__ part, int64_t rows_per_sample,
                                                        double* __restrict__ sums) {
  __shared__ double red[2][256];
  const int n = blockIdx.x / GN_GROUPS, g = blockIdx.x % GN_GROUPS;
  const float* p = part + (static_cast<int64_t>(n) * rows_per_sample * GN_GROUPS + g) * 2;
  double s1 = 0.0, s2 = 0.0;
  for (int64_t r = threadIdx.x; r < rows_per_sample; r += 256) {
    s1 += p[r * GN_GROUPS * 2];
    s2 += p[r * GN_GROUPS * 2 + 1];
  }
  red[0][threadIdx.x] = s1;
  red[1][threadIdx.x] = s2;
  __syncthreads();
  for (int o = 128; o; o >>= 1) {
    if (threadIdx.x < o) {
      red[0][threadIdx.x] += red[0][threadIdx.x + o];
      red[1][threadIdx.x] += red[1][threadIdx.x + o];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    sums[blockIdx.x * 2] = red[0][0];
    sums[blockIdx.x * 2 + 1] = red[1][0];
  }
}

// y = silu((x - mean[g]) * rstd[g] * gamma[c] + beta[c]). A thread keeps one group of 8 channels for the whole
// launch (the block's 256 threads cover 256 / (C/8) sites per iteration), so the per-channel scale
// a = rstd * gamma and offset b = beta - mean * a are computed once and the loop body is one FMA and the SiLU
// per value: silu(t) = t / (1 + 2^(-t * log2 e)) with the hardware exponential and reciprocal (both good to
// about 1e-7 relative, far inside the bf16 rounding of the result; the hyperbolic-tangent form with its 2^-11
// error flipped too many of those roundings). Launched as (blocks, N); C/8 <= 256 (threads beyond the last
// whole site of the block idle).
__device__ __forceinline__ float silu_fast(float t) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
  return t * r;
}
__global__ void __launch_bounds__(256) gn_silu_kernel(const __nv_bfloat16* __restrict__ x,
                                                      const float* __restrict__ mean_rstd,  // [N][32][2]
                                                      const __nv_bfloat16* __restrict__ gamma,
                                                      const __nv_bfloat16* __restrict__ beta, int64_t sites_per_sample,
                                                      int C, __nv_bfloat16* __restrict__ y) {
  const int vps = C >> 3;                       // 16-byte vectors per site
  const int lane_vec = threadIdx.x % vps;       // this thread's vector inside a site
  const int site_in_block = threadIdx.x / vps;
  const int sites_per_iter = 256 / vps;
  if (site_in_block >= sites_per_iter) return;
  const int n = blockIdx.y;
  const int c0 = lane_vec << 3;
  const int gs = C / GN_GROUPS;
  float a[8], b[8];
  {
    const uint4 gr = __ldg(reinterpret_cast<const uint4*>(gamma + c0));
    const uint4 br = __ldg(reinterpret_cast<const uint4*>(beta + c0));
    const uint32_t gw[4] = {gr.x, gr.y, gr.z, gr.w}, bw[4] = {br.x, br.y, br.z, br.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float2 mr = *reinterpret_cast<const float2*>(mean_rstd + (static_cast<int64_t>(n) * GN_GROUPS + (c0 + j) / gs) * 2);
      const float gv = (j & 1) ? bf16_hi(gw[j >> 1]) : bf16_lo(gw[j >> 1]);
      const float bv = (j & 1) ? bf16_hi(bw[j >> 1]) : bf16_lo(bw[j >> 1]);
      a[j] = mr.y * gv;
      b[j] = fmaf(-mr.x, a[j], bv);
    }
  }
  const __nv_bfloat16* xs = x + static_cast<int64_t>(n) * sites_per_sample * C;
  __nv_bfloat16* ys = y + static_cast<int64_t>(n) * sites_per_sample * C;
  for (int64_t site = static_cast<int64_t>(blockIdx.x) * sites_per_iter + site_in_block; site < sites_per_sample;
       site += static_cast<int64_t>(gridDim.x) * sites_per_iter) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(xs + site * C + c0));
    const uint32_t xw[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float t0 = fmaf(bf16_lo(xw[j]), a[2 * j], b[2 * j]);
      const float t1 = fmaf(bf16_hi(xw[j]), a[2 * j + 1], b[2 * j + 1]);
      o[j] = pack_bf16x2(silu_fast(t0), silu_fast(t1));
    }
    *reinterpret_cast<uint4*>(ys + site * C + c0) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// out[n, u, yy, xx, :] = in[n, (u + 1) / 2, yy / 2, xx / 2, :]: nearest 2x in space, causal 2x in time
// (the first frame is not repeated: T frames become 2T - 1).
__global__ void __launch_bounds__(256) upsample_kernel(const __nv_bfloat16* __restrict__ x, int T, int H, int W, int C,
                                                       int64_t total_vec, __nv_bfloat16* __restrict__ y) {
  const int64_t v = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (v >= total_vec) return;
  const int vec_per_site = C >> 3;
  int64_t s = v / vec_per_site;
  const int c0 = static_cast<int>(v - s * vec_per_site) << 3;
  const int T2 = 2 * T - 1, H2 = 2 * H, W2 = 2 * W;
  const int xx = static_cast<int>(s % W2);
  s /= W2;
  const int yy = static_cast<int>(s % H2);
  s /= H2;
  const int u = static_cast<int>(s % T2);
  const int64_t n = s / T2;
  const int64_t src = ((n * T + (u + 1) / 2) * H + yy / 2) * W + xx / 2;
  *reinterpret_cast<uint4*>(y + (v / vec_per_site) * C + c0) = __ldg(reinterpret_cast<const uint4*>(x + src * C + c0));
}

// tile of output sites inside a frame: bh * bw <= 128, chosen to waste as few MMA rows as possible
void choose_tile(int H, int W, int* bh, int* bw) {
  double best = -1.0;
  for (int w = 1; w <= 128 && w <= 256; ++w) {
    const int h = 128 / w;
    if (h < 1) break;
    const int hh = h < H ? h : H, ww = w < W ? w : W;
    const double eff = static_cast<double>(H) * W / (static_cast<double>((H + hh - 1) / hh) * ((W + ww - 1) / ww) * 128.0);
    if (eff > best + 1e-9) {
      best = eff;
      *bh = hh;
      *bw = ww;
    }
  }
}

// K chunks per ring stage. A stage costs one barrier round trip in the producer and in the MMA issuer, a few hundred
// cycles that a narrow tile's four MMAs per chunk (2 * BN tensor cycles) do not cover: narrow tiles put two or four
// chunks behind one barrier; the pair kernel (32 KB per chunk at most) also does so for full-width tiles, where it
// still gains 4-5 %. The count divides the 27 * chunks_per_tap chunks of a tile.
int choose_kch(int bn, int chunks_per_tap, bool pair) {
  int want = bn > 128 ? (pair ? 2 : 1) : (bn > 64 ? 2 : 4);
  while (want > 1 && chunks_per_tap % want != 0) want >>= 1;
  return want;
}

bool a16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace rh3

using namespace rh3;

extern "C" int64_t rh3_conv3d_gn_part_rows(int64_t N, int64_t T, int64_t H, int64_t W) {
  int bh = 1, bw = 1;
  choose_tile((int)H, (int)W, &bh, &bw);
  return N * T * ((H + bh - 1) / bh) * ((W + bw - 1) / bw) * 4;
}

extern "C" int rh3_conv3d_causal(const void* x, const void* w, const void* bias, const void* residual, void* out,
                                 float* gn_part, int64_t N, int64_t T, int64_t H, int64_t W, int64_t Cin,
                                 int64_t Cout, int64_t halo_frames, cudaStream_t stream) {
  RH3_CHECK_ARG(N > 0 && T > 0 && H > 0 && W > 0 && N * T * H * W < (1ll << 31), "conv3d_causal: bad shape");
  RH3_CHECK_ARG(halo_frames == 0 || halo_frames == 2, "conv3d_causal: halo_frames must be 0 or 2");
  RH3_CHECK_ARG(Cin > 0 && Cin % 64 == 0, "conv3d_causal: Cin=%lld must be a multiple of 64", (long long)Cin);
  RH3_CHECK_ARG(Cout > 0 && Cout % 16 == 0, "conv3d_causal: Cout=%lld must be a multiple of 16", (long long)Cout);
  RH3_CHECK_ARG(!gn_part || (Cout % GN_GROUPS == 0 && 32 % (Cout / GN_GROUPS) == 0),
                "conv3d_causal: GroupNorm partials need Cout/32 in {1,2,4,8,16,32}");
  RH3_CHECK_ARG(x && w && out && a16(x) && a16(w) && a16(out) && (!residual || a16(residual)),
                "conv3d_causal: null or misaligned pointer");
  ConvParams p{};
  p.N = (int)N; p.T = (int)T; p.H = (int)H; p.W = (int)W; p.Cin = (int)Cin; p.Cout = (int)Cout;
  p.halo = (int)halo_frames;
  choose_tile(p.H, p.W, &p.bh, &p.bw);
  p.tiles_h = (p.H + p.bh - 1) / p.bh;
  p.tiles_w = (p.W + p.bw - 1) / p.bw;
  // output channels per tile: the whole width when it fits one accumulator, else an even split. The epilogue walks
  // a tile in 32-column chunks, so a split tile is a multiple of 32 wide: a chunk must never reach into the columns
  // of the next tile (weight rows past Cout are zero-filled by TMA and their stores are skipped).
  const int splits = (p.Cout + 255) / 256;
  p.BN = ((p.Cout + splits - 1) / splits + 15) / 16 * 16;
  if (splits > 1) p.BN = (p.BN + 31) / 32 * 32;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.gn_part = gn_part;
  p.status = device_status_word();
  p.wide = (reinterpret_cast<uintptr_t>(out) & 31) == 0 && (!residual || (reinterpret_cast<uintptr_t>(residual) & 31) == 0);
  CUtensorMap tx, tw;
  const uint64_t Tin = (uint64_t)(T + halo_frames);  // frames held by x
  const uint64_t dims[5] = {(uint64_t)Cin, (uint64_t)W, (uint64_t)H, Tin, (uint64_t)N};
  const uint64_t strides[4] = {(uint64_t)Cin * 2, (uint64_t)W * Cin * 2, (uint64_t)H * W * Cin * 2,
                               Tin * H * W * Cin * 2};
  const uint32_t box[5] = {CBK, (uint32_t)p.bw, (uint32_t)p.bh, 1, 1};
  if (int e = make_tmap_nd(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, 5, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
    return e;
  if (int e = make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, 27 * Cin, Cout, 27 * Cin * 2, CBK, p.BN,
                           CU_TENSOR_MAP_SWIZZLE_128B))
    return e;
  const int64_t num_m = N * T * p.tiles_h * p.tiles_w, num_n = (Cout + p.BN - 1) / p.BN;
  // CTA pairs: two site tiles per pair and BN/2 weight rows per CTA (a multiple of 16, so every MMA shape is legal)
  if (pairs_enabled() && num_m >= 2 && p.BN % 32 == 0) {
    CUtensorMap twp;
    if (int e = make_tmap_2d(&twp, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, 27 * Cin, Cout, 27 * Cin * 2, CBK, p.BN / 2,
                             CU_TENSOR_MAP_SWIZZLE_128B))
      return e;
    p.chunk_bytes = CA_BYTES + p.BN / 2 * 128;
    p.kch = choose_kch(p.BN, (int)(Cin / CBK), true);
    p.stage_bytes = p.kch * p.chunk_bytes;
    p.stages = CRING_MAX_BYTES / p.stage_bytes < CMAX_STAGES ? CRING_MAX_BYTES / p.stage_bytes : CMAX_STAGES;
    const int CONV_PAIR_SMEM_BYTES = 1024 + CTAIL_BYTES + p.stages * p.stage_bytes;
    auto launch_pair = [&](auto kern) -> int {
      if (int e = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, CONV_PAIR_SMEM_BYTES),
                             "conv3d pair smem attribute"))
        return e;
      cudaLaunchConfig_t cfg{};
      cudaLaunchAttribute attr{};
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.blockDim = dim3(CONV_THREADS);
      cfg.dynamicSmemBytes = CONV_PAIR_SMEM_BYTES;
      cfg.stream = stream;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      cfg.gridDim = dim3(2 * (device_sm_count() / 2));
      int max_clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess || max_clusters < 1)
        return set_error(RH3_ARG_ERROR, "conv3d pair: no cluster of two CTAs can be resident");
      const int64_t pair_tiles = (num_m + 1) / 2 * num_n;
      cfg.gridDim = dim3(2 * static_cast<unsigned>(pair_tiles < max_clusters ? pair_tiles : max_clusters));
      return check_cuda(cudaLaunchKernelEx(&cfg, kern, tx, twp, p), "conv3d pair launch");
    };
    if (int e = p.kch == 4 ? launch_pair(conv3d_pair_kernel<4>) : p.kch == 2 ? launch_pair(conv3d_pair_kernel<2>)
                                                                            : launch_pair(conv3d_pair_kernel<1>))
      return e;
    return check_cuda(cudaGetLastError(), "conv3d pair launch");
  }
  p.chunk_bytes = CA_BYTES + p.BN * 128;
  p.kch = choose_kch(p.BN, (int)(Cin / CBK), false);
  p.stage_bytes = p.kch * p.chunk_bytes;
  p.stages = CRING_MAX_BYTES / p.stage_bytes < CMAX_STAGES ? CRING_MAX_BYTES / p.stage_bytes : CMAX_STAGES;
  const int CONV_SMEM_BYTES = 1024 + CTAIL_BYTES + p.stages * p.stage_bytes;
  const int64_t tiles = num_m * num_n;
  const int grid = tiles < device_sm_count() ? (int)tiles : device_sm_count();
  auto launch_single = [&](auto kern) -> int {
    if (int e = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, CONV_SMEM_BYTES),
                           "conv3d smem attribute"))
      return e;
    kern<<<grid, CONV_THREADS, CONV_SMEM_BYTES, stream>>>(tx, tw, p);
    return 0;
  };
  if (int e = p.kch == 4 ? launch_single(conv3d_kernel<4>) : p.kch == 2 ? launch_single(conv3d_kernel<2>)
                                                                        : launch_single(conv3d_kernel<1>))
    return e;
  return check_cuda(cudaGetLastError(), "conv3d_causal launch");
}

extern "C" int rh3_gn_reduce(const float* gn_part, int64_t rows_per_sample, int64_t N, double* sums,
                             cudaStream_t stream) {
  RH3_CHECK_ARG(gn_part && sums && rows_per_sample > 0 && N > 0 && N * GN_GROUPS < (1ll << 31), "gn_reduce: bad argument");
  gn_reduce_kernel<<<static_cast<unsigned>(N * GN_GROUPS), 256, 0, stream>>>(gn_part, rows_per_sample, sums);
  return check_cuda(cudaGetLastError(), "gn_reduce launch");
}

extern "C" int rh3_gn_silu_apply(const void* x, const float* mean_rstd, const void* gamma, const void* beta, int64_t N,
                                 int64_t sites_per_sample, int64_t C, void* y, cudaStream_t stream) {
  RH3_CHECK_ARG(x && mean_rstd && gamma && beta && y && a16(x) && a16(y) && a16(gamma) && a16(beta),
                "gn_silu_apply: null or misaligned pointer");
  RH3_CHECK_ARG(N > 0 && sites_per_sample > 0 && C > 0 && C % 8 == 0 && C % GN_GROUPS == 0, "gn_silu_apply: bad shape");
  RH3_CHECK_ARG(C / 8 <= 256, "gn_silu_apply: C=%lld is larger than 2048", (long long)C);
  RH3_CHECK_ARG(N < 65536, "gn_silu_apply: too many samples");
  const int64_t sites_per_iter = 256 / (C / 8);
  const int64_t want = (sites_per_sample + sites_per_iter - 1) / sites_per_iter;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 16;  // a few waves of resident blocks, grid-stride beyond
  const dim3 grid(static_cast<unsigned>(want < cap ? want : cap), static_cast<unsigned>(N));
  gn_silu_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), mean_rstd,
                                          static_cast<const __nv_bfloat16*>(gamma),
                                          static_cast<const __nv_bfloat16*>(beta), sites_per_sample, (int)C,
                                          static_cast<__nv_bfloat16*>(y));
  return check_cuda(cudaGetLastError(), "gn_silu_apply launch");
}

// Depth-to-space by 8 of the decoder head: y [N, T, H, W, 3*8*8] (channel = (ch*8 + dy)*8 + dx) ->
// rgb [N, 3, T, 8H, 8W]. One thread moves the 8 pixels of one (site, ch, dy): 16 bytes in, 16 bytes out; threads
// run along the output row so the stores are contiguous.
__global__ void __launch_bounds__(256) depth_to_space8_kernel(const __nv_bfloat16* __restrict__ y, int T, int H, int W,
                                                              int64_t total, __nv_bfloat16* __restrict__ rgb) {
  const int64_t v = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;  // index over [N][3][T][8H][W]
  if (v >= total) return;
  const int w = static_cast<int>(v % W);
  int64_t r = v / W;
  const int Y = static_cast<int>(r % (8 * H));
  r /= 8 * H;
  const int t = static_cast<int>(r % T);
  r /= T;
  const int ch = static_cast<int>(r % 3);
  const int64_t n = r / 3;
  const int h = Y >> 3, dy = Y & 7;
  const int64_t src = (((n * T + t) * H + h) * W + w) * 192 + (ch * 8 + dy) * 8;
  *reinterpret_cast<uint4*>(rgb + v * 8) = __ldg(reinterpret_cast<const uint4*>(y + src));
}

extern "C" int rh3_upsample_causal2x(const void* x, void* y, int64_t N, int64_t T, int64_t H, int64_t W, int64_t C,
                                     cudaStream_t stream) {
  RH3_CHECK_ARG(x && y && a16(x) && a16(y) && N > 0 && T > 0 && H > 0 && W > 0 && C > 0 && C % 8 == 0,
                "upsample_causal2x: bad argument");
  const int64_t total_vec = N * (2 * T - 1) * 2 * H * 2 * W * (C / 8);
  RH3_CHECK_ARG((total_vec + 255) / 256 < (1ll << 31), "upsample_causal2x: tensor too large");
  upsample_kernel<<<static_cast<unsigned>((total_vec + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), (int)T, (int)H, (int)W, (int)C, total_vec, static_cast<__nv_bfloat16*>(y));
  return check_cuda(cudaGetLastError(), "upsample_causal2x launch");
}

extern "C" int rh3_depth_to_space8(const void* y, void* rgb, int64_t N, int64_t T, int64_t H, int64_t W,
                                   cudaStream_t stream) {
  RH3_CHECK_ARG(y && rgb && a16(y) && a16(rgb) && N > 0 && T > 0 && H > 0 && W > 0, "depth_to_space8: bad argument");
  const int64_t total = N * 3 * T * 8 * H * W;
  RH3_CHECK_ARG((total + 255) / 256 < (1ll << 31), "depth_to_space8: tensor too large");
  depth_to_space8_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(y), (int)T, (int)H, (int)W, total, static_cast<__nv_bfloat16*>(rgb));
  return check_cuda(cudaGetLastError(), "depth_to_space8 launch");
}
