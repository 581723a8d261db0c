// Shared device/host helpers for the sm_100a kernels of librapidh3_b200.
//
// Everything here is inline PTX for Blackwell (tcgen05 tensor cores with TMEM accumulators,
// TMA tensor copies, mbarriers) plus the status/error plumbing the C-ABI uses.
//
// Rules kept by every kernel built on these helpers:
//   * every wait (mbarrier) is bounded: after a limit the waiter raises the CTA-wide abort
//     flag, records a code in the caller's status word and every role leaves its loop;
//   * TMA loads are plain CTA-local loads (no cluster-wide broadcast forms are used anywhere);
//   * no fast-math: expressions whose rounding the CPU oracle mirrors use __fmul_rn/__fadd_rn/
//     __fdiv_rn so the compiler cannot contract them into FMAs.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rh3 {

// ---------------------------------------------------------------------------------------------
// status codes written into the device status word (0 = ok)
// ---------------------------------------------------------------------------------------------
enum : int {
  ST_OK = 0,
  ST_TIMEOUT_TMA_FULL = 101,    // consumer waited too long for a TMA stage
  ST_TIMEOUT_STAGE_EMPTY = 102, // producer waited too long for a free stage
  ST_TIMEOUT_ACC_FULL = 103,    // epilogue/softmax waited too long for the tensor core
  ST_TIMEOUT_ACC_EMPTY = 104,   // MMA issuer waited too long for a free accumulator
  ST_TIMEOUT_P_READY = 105,     // attention: MMA issuer waited too long for P
  ST_TIMEOUT_PV_DONE = 106,     // attention: softmax waited too long for P.V
  ST_TIMEOUT_SELFTEST = 190,    // rh3_selftest_wait_expiry: the wait that is meant to run out did
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
// true in exactly one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
  uint32_t is_elected;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(is_elected));
  return is_elected != 0;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait. `abort_flag` is a CTA-shared int that any role sets when it gives up; every
// waiter polls it so the whole CTA drains instead of hanging. Returns true when the phase
// completed, false when the wait was abandoned (the caller must then leave its loop).
// The limit is generous (seconds): a healthy wait finishes in microseconds.
__device__ __forceinline__ bool mbar_wait_polls(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                int* status, int code, uint32_t max_polls) {
  for (uint32_t it = 0; it < max_polls; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 64) {
      if (*abort_flag) return false;
      if (it > 4096) __nanosleep(128);
    }
  }
  *abort_flag = 1;
  if (status) atomicCAS(status, 0, code);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
  return mbar_wait_polls(bar, parity, abort_flag, status, code, 1u << 24);
}

// The same bounded wait for roles that share a scheduler with busy compute warps (a TMA producer, an MMA issuer):
// between polls the thread sleeps `ns` nanoseconds, so its polling does not take issue slots from those warps.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                                  int code, unsigned ns) {
  for (uint32_t it = 0; it < (1u << 24); ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(ns);
    if (it > 64 && *abort_flag) return false;
  }
  *abort_flag = 1;
  if (status) atomicCAS(status, 0, code);
  return false;
}

// Named barrier `id` over `nthreads` threads that also ORs a predicate: every participant gets true when any of
// them passed true. The epilogue warps use it to agree on leaving their tile loop after a wait was abandoned, so
// that no warp goes on to a barrier the others will never reach.
__device__ __forceinline__ bool bar_sync_or(int id, int nthreads, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "bar.red.or.pred q, %2, %3, p;\n\t"
      "selp.b32 %0, 1, 0, q;\n\t"
      "}\n"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(pred)), "r"(id), "r"(nthreads)
      : "memory");
  return r != 0;
}

// ---------------------------------------------------------------------------------------------
// TMA (cp.async.bulk.tensor), CTA-local destination, completion on an mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, int x, int y, int z,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_5d(void* smem_dst, const CUtensorMap* m, int c0, int c1, int c2, int c3,
                                            int c4, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], "
      "[%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
// 32-byte global accesses (one full sector per thread; the address must be 32-byte aligned)
__device__ __forceinline__ void st_global_32(void* p, const uint4& a, const uint4& b) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w),
               "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
               : "memory");
}
__device__ __forceinline__ void ld_global_32(const void* p, uint4& a, uint4& b) {
  asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w)
               : "l"(p)
               : "memory");
}
// asks L2 for the 128-byte line that holds `p` (no register, no wait): an epilogue that will read a residual row
// issues these before it waits for its accumulator, so the reads that follow hit L2 instead of HBM
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}
// generic-proxy writes to smem that an async-proxy reader (tcgen05.mma, TMA store) will consume
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05: TMEM allocation, MMA issue, commit, loads
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {  // whole warp
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// ---- CTA pairs (thread-block clusters of two, tcgen05 cta_group::2) ----
// The same warp index of BOTH CTAs of the pair executes alloc / relinquish / dealloc.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {  // whole warp, both CTAs
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// all threads of both CTAs
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address, in the cluster's shared-memory window, of this CTA's shared-memory location `p` as seen in CTA `rank`
__device__ __forceinline__ uint32_t cluster_addr(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
// arrive on the barrier at this offset in CTA `rank` of the cluster
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t rank) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr(bar, rank)) : "memory");
}
// TMA tile load into THIS CTA's shared memory whose bytes are counted on the barrier at the same offset in the pair's
// even CTA (`leader_bar` = cluster_addr(bar, 0)); every CTA fetches its own tile
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, int x, int y, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_5d_pair(void* smem_dst, const CUtensorMap* m, int c0, int c1, int c2, int c3,
                                                 int c4, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], "
      "[%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(leader_bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
// all MMAs issued so far by this thread arrive, when they retire, on the barrier at the given cluster address
__device__ __forceinline__ void mma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; one thread issues.
__device__ __forceinline__ void mma_i8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Four MMAs over one 128-byte K slab (4 x 32 bytes) in a single instruction sequence: the issuing thread
// is one lane, so every scalar instruction between two MMAs costs tensor-pipe time. The descriptors of
// the K steps differ only by +2 in the 16-byte start-address field, so the whole slab costs six adds.
// `acc_first` = 0 makes the first MMA overwrite D; the other three always accumulate.
#define RH3_DEFINE_MMA4(NAME, KIND)                                                                            \
  __device__ __forceinline__ void NAME(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,       \
                                       uint32_t acc_first) {                                                    \
    asm volatile(                                                                                              \
        "{\n\t"                                                                                                \
        ".reg .pred p, q;\n\t"                                                                                 \
        ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"                                                                \
        "setp.ne.b32 p, %4, 0;\n\t"                                                                            \
        "setp.eq.b32 q, 0, 0;\n\t"                                                                             \
        "add.u64 a1, %1, 2;\n\t"                                                                               \
        "add.u64 b1, %2, 2;\n\t"                                                                               \
        "add.u64 a2, %1, 4;\n\t"                                                                               \
        "add.u64 b2, %2, 4;\n\t"                                                                               \
        "add.u64 a3, %1, 6;\n\t"                                                                               \
        "add.u64 b3, %2, 6;\n\t"                                                                               \
        "tcgen05.mma.cta_group::1.kind::" KIND " [%0], %1, %2, %3, p;\n\t"                                     \
        "tcgen05.mma.cta_group::1.kind::" KIND " [%0], a1, b1, %3, q;\n\t"                                     \
        "tcgen05.mma.cta_group::1.kind::" KIND " [%0], a2, b2, %3, q;\n\t"                                     \
        "tcgen05.mma.cta_group::1.kind::" KIND " [%0], a3, b3, %3, q;\n\t"                                     \
        "}\n" ::"r"(d_tmem),                                                                                   \
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc_first)                                                   \
        : "memory");                                                                                           \
  }
RH3_DEFINE_MMA4(mma4_i8_ss, "i8")
// The same four MMAs issued for a CTA pair (256 rows: 128 from each CTA's A tile; B's N rows split between the two
// CTAs' tiles; each CTA's TMEM receives its 128 rows). Issued by one thread of the pair's even CTA.
#define RH3_DEFINE_MMA4_PAIR(NAME, KIND)                                                                       \
  __device__ __forceinline__ void NAME(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,       \
                                       uint32_t acc_first) {                                                    \
    asm volatile(                                                                                              \
        "{\n\t"                                                                                                \
        ".reg .pred p, q;\n\t"                                                                                 \
        ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"                                                                \
        "setp.ne.b32 p, %4, 0;\n\t"                                                                            \
        "setp.eq.b32 q, 0, 0;\n\t"                                                                             \
        "add.u64 a1, %1, 2;\n\t"                                                                               \
        "add.u64 b1, %2, 2;\n\t"                                                                               \
        "add.u64 a2, %1, 4;\n\t"                                                                               \
        "add.u64 b2, %2, 4;\n\t"                                                                               \
        "add.u64 a3, %1, 6;\n\t"                                                                               \
        "add.u64 b3, %2, 6;\n\t"                                                                               \
        "tcgen05.mma.cta_group::2.kind::" KIND " [%0], %1, %2, %3, p;\n\t"                                     \
        "tcgen05.mma.cta_group::2.kind::" KIND " [%0], a1, b1, %3, q;\n\t"                                     \
        "tcgen05.mma.cta_group::2.kind::" KIND " [%0], a2, b2, %3, q;\n\t"                                     \
        "tcgen05.mma.cta_group::2.kind::" KIND " [%0], a3, b3, %3, q;\n\t"                                     \
        "}\n" ::"r"(d_tmem),                                                                                   \
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc_first)                                                   \
        : "memory");                                                                                           \
  }
RH3_DEFINE_MMA4_PAIR(mma4_i8_pair, "i8")
RH3_DEFINE_MMA4_PAIR(mma4_f8_pair, "f8f6f4")
RH3_DEFINE_MMA4_PAIR(mma4_f16_pair, "f16")
#undef RH3_DEFINE_MMA4_PAIR
RH3_DEFINE_MMA4(mma4_f8_ss, "f8f6f4")
RH3_DEFINE_MMA4(mma4_f16_ss, "f16")
#undef RH3_DEFINE_MMA4

// all previously issued MMAs of this thread arrive on `bar` when they retire
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets row (lane base + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x 8 consecutive columns (small-footprint variants for rarely taken paths)
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n\t"
               "tcgen05.wait::ld.sync.aligned;"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
// 32 lanes x 16 consecutive columns without the wait (pair with tmem_ld_wait16 on the same registers)
__device__ __forceinline__ void tmem_ld16_async(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr)
               : "memory");
}
// wait for every TMEM load issued so far; tied to 16 destination registers so that no use of them moves above it
__device__ __forceinline__ void tmem_ld_wait16(uint32_t* r) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
// store the same 32-bit value to 32 lanes x 32 consecutive columns (one source register)
__device__ __forceinline__ void tmem_st32_splat(uint32_t taddr, uint32_t v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, "
      "%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr),
      "r"(v)
      : "memory");
}
// Same wait, tied to the 32 destination registers of an earlier tmem_ld32 so that the compiler cannot
// move arithmetic on them above the wait (the load delivers its registers asynchronously).
__device__ __forceinline__ void tmem_ld_wait_regs(uint32_t* r) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]),
                 "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]),
                 "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// descriptors
// ---------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a K-major operand tile whose rows are exactly 128 bytes,
// stored with the 128-byte swizzle TMA produces (16-byte chunk c of row r lives at chunk
// c ^ (r & 7)); groups of 8 rows are 1024 bytes apart. The tile base must be 1024-byte aligned;
// stepping along K inside the 128-byte row is done by adding the byte offset to the start address.
__device__ __forceinline__ uint64_t make_desc_k128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);  // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;                     // leading byte offset (unused for swizzled K-major)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;             // stride byte offset between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;                     // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                     // 128-byte swizzle
  return d;
}

// Instruction descriptor (dense, no negate, K-major A and B).
//   c_format: 1 = f32, 2 = s32;  a/b_format: kind::i8 -> 1 = signed 8-bit; kind::f8f6f4 -> 0 = e4m3;
//   kind::f16 -> 1 = bf16
__host__ __device__ constexpr uint32_t make_idesc(uint32_t c_format, uint32_t a_format, uint32_t b_format,
                                                  uint32_t m, uint32_t n) {
  return (c_format << 4) | (a_format << 7) | (b_format << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------
// small numeric helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// fixed-order butterfly sum: every lane ends with the same value; the CPU oracle mirrors the order
__device__ __forceinline__ float warp_sum_xor(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---------------------------------------------------------------------------------------------
// exact quantizer steps without the conversion unit
// ---------------------------------------------------------------------------------------------
// int8 code of round_half_even(y / s) (|y / s| <= 127 by construction of s), returned in the low byte.
// t = fma(y, 1/s, 1.5 * 2^23) rounds the exact product P = y * (1/s) to the integer r = t - 1.5 * 2^23; d = fma(y, 1/s, -r)
// is P's distance from r. P and the rounded quotient fl(y / s) each differ from the true quotient by at most
// 127 * 2^-24 = 7.6e-6, so they can round to different integers only when |d| > 0.5 - 2^-14; only then is the exact
// IEEE quotient computed. The code therefore always equals the one a true division would give.
__device__ __forceinline__ uint32_t quant_code_i8(float y, float s, float inv) {
  const float kMagic = 12582912.f;
  float t = fmaf(y, inv, kMagic);
  const float d = fmaf(y, inv, -__fsub_rn(t, kMagic));
  if (fabsf(d) > 0.5f - 6.103515625e-5f) t = __fadd_rn(__fdiv_rn(y, s), kMagic);
  return __float_as_uint(t);  // low byte = two's complement code
}
// e4m3 code of clamp(y / s, +-448) rounded to nearest even. The fast path converts y * (1/s); the exact
// quotient is used when the product is within 16 fp32 ulps of an e4m3 rounding tie or in e4m3's subnormal
// range, where the two could round differently.
__device__ __forceinline__ uint32_t quant_code_e4m3(float y, float s, float inv) {
  float yq = fminf(fmaxf(__fmul_rn(y, inv), -448.f), 448.f);
  const uint32_t drop = __float_as_uint(yq) & 0xFFFFFu;
  if (fabsf(yq) < 0.015625f || (drop - 0x7FFF0u) < 0x20u) yq = fminf(fmaxf(__fdiv_rn(y, s), -448.f), 448.f);
  return static_cast<uint32_t>(__nv_cvt_float_to_fp8(yq, __NV_SATFINITE, __NV_E4M3)) & 0xFFu;
}
// Eight int8 codes at once (bytes 0..7 of the result in memory order). Same arithmetic as quant_code_i8,
// but the "near a tie" tests of the eight values are OR-ed into one predicate, so the exact-division path is
// a single rarely taken branch per 8 values instead of one per value. Recomputing all eight exactly is
// harmless: away from a tie the fast and the exact code agree.
__device__ __forceinline__ uint2 quant8_i8(const float* y, float s, float inv) {
  const float kMagic = 12582912.f;
  float t[8];
  bool near = false;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    t[j] = fmaf(y[j], inv, kMagic);
    // the product's distance from the integer it rounded to; a wider window than 2^-14 below a tie would send most
    // warps down the division path (any of 256 values triggers it)
    near |= fabsf(fmaf(y[j], inv, -__fsub_rn(t[j], kMagic))) > 0.5f - 6.103515625e-5f;
  }
  if (near) {
#pragma unroll  // static indices: a rolled loop would push the caller's register array to local memory
    for (int j = 0; j < 8; ++j) t[j] = __fadd_rn(__fdiv_rn(y[j], s), kMagic);
  }
  uint2 o;
  o.x = __byte_perm(__byte_perm(__float_as_uint(t[0]), __float_as_uint(t[1]), 0x0040),
                    __byte_perm(__float_as_uint(t[2]), __float_as_uint(t[3]), 0x0040), 0x5410);
  o.y = __byte_perm(__byte_perm(__float_as_uint(t[4]), __float_as_uint(t[5]), 0x0040),
                    __byte_perm(__float_as_uint(t[6]), __float_as_uint(t[7]), 0x0040), 0x5410);
  return o;
}
// Eight e4m3 codes at once; the arithmetic of quant_code_e4m3 with one shared exact path per 8 values and the
// two-at-a-time hardware conversion (which saturates at +-448 itself).
__device__ __forceinline__ uint2 quant8_e4m3(const float* y, float s, float inv) {
  float yq[8];
  bool near = false;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    yq[j] = __fmul_rn(y[j], inv);
    const uint32_t drop = __float_as_uint(yq[j]) & 0xFFFFFu;
    near |= (fabsf(yq[j]) < 0.015625f) | ((drop - 0x7FFF0u) < 0x20u);
  }
  if (near) {
#pragma unroll
    for (int j = 0; j < 8; ++j) yq[j] = __fdiv_rn(y[j], s);
  }
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint16_t h;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(h) : "f"(yq[2 * j]), "f"(yq[2 * j + 1]));
    w[j] = h;
  }
  return make_uint2(w[0] | (w[1] << 16), w[2] | (w[3] << 16));
}
// The same for eight values that each have their own scale (a row of V against per-channel scales).
__device__ __forceinline__ uint2 quant8_e4m3_per_channel(const float* y, const float* s, const float* inv) {
  float yq[8];
  bool near = false;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    yq[j] = __fmul_rn(y[j], inv[j]);
    const uint32_t drop = __float_as_uint(yq[j]) & 0xFFFFFu;
    near |= (fabsf(yq[j]) < 0.015625f) | ((drop - 0x7FFF0u) < 0x20u);
  }
  if (near) {
#pragma unroll
    for (int j = 0; j < 8; ++j) yq[j] = __fdiv_rn(y[j], s[j]);
  }
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint16_t h;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(h) : "f"(yq[2 * j]), "f"(yq[2 * j + 1]));
    w[j] = h;
  }
  return make_uint2(w[0] | (w[1] << 16), w[2] | (w[3] << 16));
}
// pack the low bytes of four words into one word (a -> byte 0 ... d -> byte 3)
__device__ __forceinline__ uint32_t pack_low_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

}  // namespace rh3

// ---------------------------------------------------------------------------------------------
// host side: error reporting shared by all translation units (defined in api.cu)
// ---------------------------------------------------------------------------------------------
extern "C" const char* rh3_last_error_string(void);
namespace rh3 {
int set_error(int code, const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);
// Encode a 2-D row-major byte/element tensor map: dims {inner, outer}, box {box_inner, box_outer}.
int make_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, uint32_t elem_bytes, const void* base, uint64_t inner,
                 uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                 CUtensorMapSwizzle swz);
int make_tmap_nd(CUtensorMap* out, CUtensorMapDataType dt, uint32_t elem_bytes, const void* base, int rank,
                 const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz);
int device_sm_count();
// 1 when the GEMM and convolution entries launch their CTA-pair kernels (rh3_gemm_use_pairs)
int pairs_enabled();
// device status word (one int per device, lazily allocated at library load / first use)
int* device_status_word();
int read_and_clear_status(cudaStream_t stream, int* out);
}  // namespace rh3

#define RH3_ARG_ERROR (-1)
#define RH3_CHECK_ARG(cond, ...)                          \
  do {                                                    \
    if (!(cond)) return rh3::set_error(RH3_ARG_ERROR, __VA_ARGS__); \
  } while (0)
