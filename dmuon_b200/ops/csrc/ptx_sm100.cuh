// Thin inline-PTX wrappers for the sm_100a features the kernels in this
// directory use: mbarrier, TMA bulk-tensor loads (never with cluster
// multicast), tcgen05 MMA / TMEM allocation / TMEM loads, and bounded waits.
//
// Every wait in this file has a deadline.  A wait that runs out records a
// code in a status word and lets the kernel return; nothing here can spin
// forever or trap.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace dmuon {

// Status codes written to the int status word a kernel receives.
enum : int {
  kStatusOk = 0,
  kStatusTimeoutProducer = 1,   // TMA producer waited too long for a free stage
  kStatusTimeoutMma = 2,        // MMA issuer waited too long for data or TMEM
  kStatusTimeoutEpilogue = 3,   // epilogue waited too long for an accumulator
  kStatusTimeoutPeerFlag = 4,   // a flag another GPU or CTA should set never came
  kStatusBadArgument = 5,
};

// ~2 s at 1.9 GHz; far above any legitimate wait inside one kernel.
__device__ constexpr long long kWaitBudgetCycles = 4000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait on an mbarrier phase.  Returns false if the deadline passed or
// another role of this CTA already gave up (abort_flag != 0).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitBudgetCycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// Same with a caller-chosen budget (kernels whose progress depends on another
// GPU wait as long as the cross-GPU flag waits do).
__device__ __forceinline__ bool mbar_wait_long(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                               long long budget_cycles) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > budget_cycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// --- TMA (cp.async.bulk.tensor), 3-D tiled load, no multicast -------------
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const void* tmap, uint32_t bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// --- tcgen05 / TMEM ---------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], issued by ONE thread.
__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// mbarrier arrives once all MMAs issued so far by this thread have finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread t of the warp gets lane
// (warp%4)*32+t, registers 0..31 are columns col..col+31.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for tcgen05.mma (sm_100 format: version 1
// in bits 46-47, 3-bit layout type in bits 61-63, 2 = 128-byte swizzle).
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;   // descriptor version for Blackwell
  d |= static_cast<uint64_t>(2) << 61;   // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16 with fp32 accumulation.
__device__ __forceinline__ uint32_t make_idesc_f16(int m, int n, bool ab_is_fp16, bool a_mn_major,
                                                   bool b_mn_major) {
  uint32_t d = 0;
  d |= 1u << 4;                                   // accumulator format: f32
  d |= (ab_is_fp16 ? 0u : 1u) << 7;               // A format: f16 / bf16
  d |= (ab_is_fp16 ? 0u : 1u) << 10;              // B format
  d |= (a_mn_major ? 1u : 0u) << 15;
  d |= (b_mn_major ? 1u : 0u) << 16;
  d |= static_cast<uint32_t>(n >> 3) << 17;
  d |= static_cast<uint32_t>(m >> 4) << 24;
  return d;
}

// --- CTA pairs (cluster of 2, tcgen05 cta_group::2) ---------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// shared::cluster address of the same shared-memory offset in CTA `rank`
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// Tiled load issued by either CTA of a pair; the transaction bytes are counted
// on the mbarrier of the pair's leader (even rank).  No multicast.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t smem_dst, const void* tmap, uint32_t leader_bar,
                                                 int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_dst), "l"(tmap), "r"(leader_bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// 256 x N x 16 MMA over both CTAs of the pair, issued by one thread of the leader.
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive on ONE mbarrier (any CTA of the cluster) when the pair's MMAs so far are done.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar)
               : "memory");
}

// --- operand forwarding between CTAs of one cluster (distributed shared memory) ---
// shared memory of this CTA -> shared memory of another CTA of the cluster; the
// bytes are counted on an mbarrier of the RECEIVING CTA.  Both addresses 16-byte
// aligned, size a multiple of 16.  This is a copy between two SMs' shared
// memories: no global memory and no multicast is involved.
__device__ __forceinline__ void bulk_copy_s2cluster(uint32_t dst_cluster, uint32_t src_cta, uint32_t bytes,
                                                    uint32_t mbar_cluster) {
  asm volatile(
      "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(dst_cluster), "r"(src_cta), "r"(bytes), "r"(mbar_cluster)
      : "memory");
}

// A 32-bit progress counter in another CTA's shared memory (monotonic, so a
// reader can never confuse two rounds the way a one-bit phase could).
__device__ __forceinline__ void st_release_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.release.cluster.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_cluster_u32(uint32_t cta_addr) {
  uint32_t v;
  asm volatile("ld.acquire.cluster.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(cta_addr) : "memory");
  return v;
}

// Spin until the counter at `cta_addr` (this CTA's shared memory, written by a
// peer CTA) reaches `want`; gives up like mbar_wait_bounded.
__device__ __forceinline__ bool counter_wait_bounded(uint32_t cta_addr, uint32_t want, volatile int* abort_flag) {
  if (ld_acquire_cluster_u32(cta_addr) >= want) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (ld_acquire_cluster_u32(cta_addr) >= want) return true;
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitBudgetCycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// --- untiled bulk copies (16-byte aligned addresses, size a multiple of 16) ---
// global (this GPU's or a peer's memory) -> shared, completion on an mbarrier
__device__ __forceinline__ void bulk_load_g2s(uint32_t smem_dst, const void* gsrc, uint32_t bytes,
                                              uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar)
      : "memory");
}

// shared -> global, tracked by the bulk async-group of the issuing thread
__device__ __forceinline__ void bulk_store_s2g(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// all but the newest `N` groups have finished READING their shared-memory source
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// all but the newest `N` groups have completed (their global writes are done)
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

__device__ __forceinline__ void red_add_release_gpu(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// --- peer / flag helpers ----------------------------------------------------
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// --- NVSwitch multicast (NVLS): one address that stands for the same offset in
// every rank's buffer.  A reduce-load returns the element-wise sum over all
// ranks, formed inside the switch (fp32 accumulation for 16-bit types, result
// rounded to the element type); a store is replicated to every rank.  These are
// plain loads and stores on a multicast mapping -- not TMA, not cluster multicast.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}

__device__ __forceinline__ uint4 multimem_ld_reduce_f16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}

__device__ __forceinline__ uint4 multimem_ld_reduce_f32x4(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}

// 16 bytes to the same offset of every rank's buffer
__device__ __forceinline__ void multimem_st_16B(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// Spin until *flag >= want (system scope), at most budget_cycles.  Returns
// false when the budget ran out.
__device__ __forceinline__ bool wait_flag_ge_sys(const int* flag, int want, long long budget_cycles) {
  if (ld_acquire_sys(flag) >= want) return true;
  const long long t0 = clock64();
  while (true) {
    if (ld_acquire_sys(flag) >= want) return true;
    if (clock64() - t0 > budget_cycles) return false;
    __nanosleep(64);
  }
}

__device__ __forceinline__ bool wait_flag_ge_gpu(const int* flag, int want, long long budget_cycles) {
  if (ld_acquire_gpu(flag) >= want) return true;
  const long long t0 = clock64();
  while (true) {
    if (ld_acquire_gpu(flag) >= want) return true;
    if (clock64() - t0 > budget_cycles) return false;
    __nanosleep(32);
  }
}

}  // namespace dmuon
