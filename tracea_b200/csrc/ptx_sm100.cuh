// Thin inline-PTX wrappers for the sm_100a features the conv kernel uses:
// mbarrier (bounded waits), TMA tiled + im2col loads, tcgen05 alloc / mma / commit / ld.
//
// Every wait in here is bounded: a wait that runs out returns false so the caller can record
// an error code and unwind, instead of spinning for ever on a shared GPU.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb200 {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------ CTA pairs (cluster of 2)
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Barrier over every thread of both CTAs of the cluster (all threads must call it).
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_cluster(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// ------------------------------------------------------------------ programmatic dependent launch
// A kernel launched with the programmatic-stream-serialization attribute may start while the kernel before it on
// the stream is still running. `griddep_wait` returns once that earlier kernel has completed and its writes are
// visible (at once when there is no such dependency); nothing the earlier kernel wrote may be read, and nothing it
// reads may be overwritten, before it. `griddep_launch_dependents` lets the NEXT kernel on the stream be scheduled
// as soon as every CTA of this grid has called it (or exited).
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n"
      "selp.u32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking probe. Its result takes a couple of hundred cycles to come back, so the single-thread
// roles issue the probe for the NEXT stage before working on the current one and only read the
// answer afterwards.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n"
      "selp.u32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. `abort_flag` is a CTA-shared word any role sets when it gives up; every waiter
// polls it so that one failed wait unwinds the whole CTA. `limit_cycles` bounds this wait alone.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  volatile uint32_t* abort_flag,
                                                  long long limit_cycles) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0x3ffu) == 0) {
      if (*abort_flag != 0u) return false;
      if (clock64() - t0 > limit_cycles) return false;
    }
  }
}

// The same wait for a whole warp: lane 0 polls (optionally with a short sleep between polls), the other lanes park
// at the shuffle that hands them the answer -- a value the compiler knows to be the same in every lane, so the code
// that follows stays in uniform control flow. Callers follow with tcgen05.fence::after_thread_sync before touching
// TMEM.
template <bool kSleep = true>
__device__ __forceinline__ bool mbar_wait_bounded_warp(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                       long long limit_cycles, int lane) {
  uint32_t ok = 1u;
  if (lane == 0 && !mbar_try_wait(bar, parity)) {
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (true) {
      if constexpr (kSleep) __nanosleep(64);
      if (mbar_try_wait(bar, parity)) break;
      if ((++spins & 0x3fu) == 0) {
        if (*abort_flag != 0u || clock64() - t0 > limit_cycles) {
          ok = 0u;
          break;
        }
      }
    }
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0u;
}

// Bounded wait of a whole converged warp in uniform control flow: every lane polls (one broadcast access), every
// branch is taken on a warp vote, so the compiler can keep treating what follows as warp-uniform. That matters for
// the MMA-issuing warp: after a wait with a lane-0-only polling loop the very same MMA loop was measured to issue
// at 97 instead of 43 cycles per MMA.
__device__ __forceinline__ bool mbar_wait_bounded_uniform(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                          long long limit_cycles) {
  if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
    if ((++spins & 0x7u) == 0) {   // a failed try_wait has already slept for a while
      if (__any_sync(0xffffffffu, *abort_flag != 0u || clock64() - t0 > limit_cycles)) return false;
    }
  }
}

// One lane of a converged warp, as a 0 / 1 word (elect.sync).
__device__ __forceinline__ uint32_t elect_one_lane() {
  uint32_t pred;
  asm volatile("{\n.reg .pred P;\nelect.sync _|P, 0xffffffff;\nselp.u32 %0, 1, 0, P;\n}\n" : "=r"(pred));
  return pred;
}

// ------------------------------------------------------------------ TMA loads (no multicast)
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// Tiled 2-D load: coordinates {c0 (innermost), c1}.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// im2col-mode 4-D load over an NHWC tensor: coordinates {c, w, h, n} give the first base pixel
// (already including the negative padding corner), {off_w, off_h} the filter-tap offset.
__device__ __forceinline__ void tma_load_im2col_4d(uint32_t dst, const void* tmap, uint32_t bar,
                                                   int c, int w, int h, int n, uint16_t off_w,
                                                   uint16_t off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n),
        "h"(off_w), "h"(off_h)
      : "memory");
}

// Same im2col box, but only pulled into L2 (no shared-memory destination, no barrier): used to run the
// HBM fetch of the activations several k-steps ahead of the shared-memory ring.
__device__ __forceinline__ void tma_prefetch_im2col_4d(const void* tmap, int c, int w, int h, int n, uint16_t off_w,
                                                       uint16_t off_h) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.im2col [%0, {%1, %2, %3, %4}], {%5, %6};"
               :
               : "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
               : "memory");
}

// Tiled 2-D store shared -> global (bulk-group completion). Rows / columns outside the tensor are
// clipped by the TMA unit, which is what handles the M and K_out tails.
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(tmap)), "r"(src), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// At most N of this thread's most recent bulk groups may still be reading shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// All bulk groups of this thread are complete (writes performed).
__device__ __forceinline__ void bulk_wait_group0() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
// Acquire load at GPU scope: used to poll a counter another CTA increments after a __threadfence().
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Release increment at GPU scope: everything this thread wrote, and everything it has observed (the other lanes'
// stores, after a warp barrier), is visible to whoever sees the new count with an acquire load.
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ float4 ld_shared_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// ------------------------------------------------------------------ tcgen05 / TMEM
template <uint32_t kCols>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(kCols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <uint32_t kCols>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(kCols)
               : "memory");
}
// cta_group::2 forms: the TMEM columns are allocated in both CTAs of the pair; each CTA's MMA warp calls these.
template <uint32_t kCols>
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(kCols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <uint32_t kCols>
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(kCols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// One pipeline stage of the MMA issuer as a single block: probe the NEXT stage's full barrier, issue
// the four MMAs of this stage, commit them to this stage's empty barrier, and only then read the
// probe's predicate -- so the probe's latency is spent under the MMA issue instead of stalling the
// in-order thread in front of it. Returns whether the next stage was already full.
template <bool kTf32, bool kFirstAccumulates>
__device__ __forceinline__ bool mma_stage4_probe(uint32_t tmem_d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3,
                                                 uint32_t desc_hi, uint32_t idesc, uint32_t empty_bar,
                                                 uint32_t next_full_bar, uint32_t next_parity) {
  uint32_t ready;
#define TB200_MMA_STAGE(KIND)                                                                   \
  asm volatile(                                                                                  \
      "{\n"                                                                                      \
      ".reg .pred pn, p0, p1;\n"                                                                 \
      ".reg .b64 da, db;\n"                                                                      \
      "mbarrier.test_wait.parity.shared::cta.b64 pn, [%13], %14;\n"                              \
      "setp.ne.b32 p0, %15, 0;\n"                                                                \
      "setp.eq.b32 p1, 0, 0;\n"                                                                  \
      "mov.b64 da, {%2, %10};\n"                                                                 \
      "mov.b64 db, {%6, %10};\n"                                                                 \
      "tcgen05.mma.cta_group::1.kind::" KIND " [%1], da, db, %11, p0;\n"                         \
      "mov.b64 da, {%3, %10};\n"                                                                 \
      "mov.b64 db, {%7, %10};\n"                                                                 \
      "tcgen05.mma.cta_group::1.kind::" KIND " [%1], da, db, %11, p1;\n"                         \
      "mov.b64 da, {%4, %10};\n"                                                                 \
      "mov.b64 db, {%8, %10};\n"                                                                 \
      "tcgen05.mma.cta_group::1.kind::" KIND " [%1], da, db, %11, p1;\n"                         \
      "mov.b64 da, {%5, %10};\n"                                                                 \
      "mov.b64 db, {%9, %10};\n"                                                                 \
      "tcgen05.mma.cta_group::1.kind::" KIND " [%1], da, db, %11, p1;\n"                         \
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%12];\n"           \
      "selp.u32 %0, 1, 0, pn;\n"                                                                 \
      "}\n"                                                                                      \
      : "=r"(ready)                                                                              \
      : "r"(tmem_d), "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(b2), "r"(b3),     \
        "r"(desc_hi), "r"(idesc), "r"(empty_bar), "r"(next_full_bar), "r"(next_parity),          \
        "n"(kFirstAccumulates ? 1 : 0)                                                           \
      : "memory")
  if constexpr (kTf32) {
    TB200_MMA_STAGE("tf32");
  } else {
    TB200_MMA_STAGE("f16");
  }
#undef TB200_MMA_STAGE
  return ready != 0;
}

// The same stage for a CTA pair: issued by the leader CTA only; each MMA spans both SMs (M = 256: 128 rows of
// A and half of B's rows come from each CTA's shared memory at the same offsets) and the commit arrives on
// the `empty` barrier at the same offset in BOTH CTAs (multicast arrive, mask 0b11).
template <bool kTf32, bool kFirstAccumulates>
__device__ __forceinline__ bool mma_stage4_probe_pair(uint32_t tmem_d, uint32_t a0, uint32_t a1, uint32_t a2,
                                                      uint32_t a3, uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3,
                                                      uint32_t desc_hi, uint32_t idesc, uint32_t empty_bar,
                                                      uint32_t next_full_bar, uint32_t next_parity) {
  uint32_t ready;
#define TB200_MMA_STAGE2(KIND)                                                                  \
  asm volatile(                                                                                  \
      "{\n"                                                                                      \
      ".reg .pred pn, p0, p1;\n"                                                                 \
      ".reg .b64 da, db;\n"                                                                      \
      ".reg .b16 msk;\n"                                                                         \
      "mov.b16 msk, 3;\n"                                                                        \
      "mbarrier.test_wait.parity.shared::cta.b64 pn, [%13], %14;\n"                              \
      "setp.ne.b32 p0, %15, 0;\n"                                                                \
      "setp.eq.b32 p1, 0, 0;\n"                                                                  \
      "mov.b64 da, {%2, %10};\n"                                                                 \
      "mov.b64 db, {%6, %10};\n"                                                                 \
      "tcgen05.mma.cta_group::2.kind::" KIND " [%1], da, db, %11, p0;\n"                         \
      "mov.b64 da, {%3, %10};\n"                                                                 \
      "mov.b64 db, {%7, %10};\n"                                                                 \
      "tcgen05.mma.cta_group::2.kind::" KIND " [%1], da, db, %11, p1;\n"                         \
      "mov.b64 da, {%4, %10};\n"                                                                 \
      "mov.b64 db, {%8, %10};\n"                                                                 \
      "tcgen05.mma.cta_group::2.kind::" KIND " [%1], da, db, %11, p1;\n"                         \
      "mov.b64 da, {%5, %10};\n"                                                                 \
      "mov.b64 db, {%9, %10};\n"                                                                 \
      "tcgen05.mma.cta_group::2.kind::" KIND " [%1], da, db, %11, p1;\n"                         \
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%12], msk;\n" \
      "selp.u32 %0, 1, 0, pn;\n"                                                                 \
      "}\n"                                                                                      \
      : "=r"(ready)                                                                              \
      : "r"(tmem_d), "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(b2), "r"(b3),     \
        "r"(desc_hi), "r"(idesc), "r"(empty_bar), "r"(next_full_bar), "r"(next_parity),          \
        "n"(kFirstAccumulates ? 1 : 0)                                                           \
      : "memory")
  if constexpr (kTf32) {
    TB200_MMA_STAGE2("tf32");
  } else {
    TB200_MMA_STAGE2("f16");
  }
#undef TB200_MMA_STAGE2
  return ready != 0;
}
// Arrive on `bar` (same offset in both CTAs of the pair) once every MMA issued so far has retired.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  asm volatile(
      "{\n"
      ".reg .b16 msk;\n"
      "mov.b16 msk, 3;\n"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], msk;\n"
      "}\n" ::"r"(bar)
      : "memory");
}

// Producer stage of a CTA pair: both CTAs issue their own copies (their 128 pixels of A, their half of B's
// rows) into their own shared memory, all signalling the LEADER's full barrier (`full_bar_leader`, a
// shared::cluster address). No multicast: each CTA fetches what it needs itself. `expect_bytes` is the whole
// stage of both CTAs for the leader and 0 for the follower (which then skips the arrive).
__device__ __forceinline__ bool tma_stage_probe_pair(uint32_t a_dst, uint32_t b_dst, uint32_t full_bar_local,
                                                     uint32_t full_bar_leader, uint32_t expect_bytes,
                                                     const void* tmap_x, int c, int w, int h, int n, uint16_t off_w,
                                                     uint16_t off_h, const void* tmap_w, int k0, int n0,
                                                     uint32_t next_empty_bar, uint32_t next_parity) {
  uint32_t free_next;
  asm volatile(
      "{\n"
      ".reg .pred pn, pl;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 pn, [%16], %17;\n"
      "setp.ne.b32 pl, %4, 0;\n"
      "@pl mbarrier.arrive.expect_tx.shared::cta.b64 _, [%3], %4;\n"
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
      " [%1], [%6, {%7, %8, %9, %10}], [%5], {%11, %12};\n"
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%2], [%13, {%14, %15}], [%5];\n"
      "selp.u32 %0, 1, 0, pn;\n"
      "}\n"
      : "=r"(free_next)
      : "r"(a_dst), "r"(b_dst), "r"(full_bar_local), "r"(expect_bytes), "r"(full_bar_leader),
        "l"(reinterpret_cast<uint64_t>(tmap_x)), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h),
        "l"(reinterpret_cast<uint64_t>(tmap_w)), "r"(k0), "r"(n0), "r"(next_empty_bar), "r"(next_parity)
      : "memory");
  return free_next != 0;
}

// One pipeline stage of the TMA producer as a single block, same idea: probe the NEXT slot's empty
// barrier first, then arm this slot's full barrier and issue the im2col copy of A and the tiled copy
// of B, then read the probe.
__device__ __forceinline__ bool tma_stage_probe(uint32_t a_dst, uint32_t b_dst, uint32_t full_bar, uint32_t stage_bytes,
                                                const void* tmap_x, int c, int w, int h, int n, uint16_t off_w,
                                                uint16_t off_h, const void* tmap_w, int k0, int n0,
                                                uint32_t next_empty_bar, uint32_t next_parity) {
  uint32_t free_next;
  asm volatile(
      "{\n"
      ".reg .pred pn;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 pn, [%15], %16;\n"
      "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%3], %4;\n"
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
      " [%1], [%5, {%6, %7, %8, %9}], [%3], {%10, %11};\n"
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%2], [%12, {%13, %14}], [%3];\n"
      "selp.u32 %0, 1, 0, pn;\n"
      "}\n"
      : "=r"(free_next)
      : "r"(a_dst), "r"(b_dst), "r"(full_bar), "r"(stage_bytes), "l"(reinterpret_cast<uint64_t>(tmap_x)), "r"(c),
        "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h), "l"(reinterpret_cast<uint64_t>(tmap_w)), "r"(k0), "r"(n0),
        "r"(next_empty_bar), "r"(next_parity)
      : "memory");
  return free_next != 0;
}

// Producer stage of a two-row-block tile: two im2col copies of A (pixels 0..127 and 128..255 of the tile,
// each with its own start pixel) and one tiled copy of B.
__device__ __forceinline__ bool tma_stage_probe_rows2(uint32_t a0_dst, uint32_t a1_dst, uint32_t b_dst,
                                                      uint32_t full_bar, uint32_t stage_bytes, const void* tmap_x,
                                                      int c, int w0, int h0, int n0i, int w1, int h1, int n1i,
                                                      uint16_t off_w, uint16_t off_h, const void* tmap_w, int k0,
                                                      int ncol, uint32_t next_empty_bar, uint32_t next_parity) {
  uint32_t free_next;
  asm volatile(
      "{\n"
      ".reg .pred pn;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 pn, [%19], %20;\n"
      "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%4], %5;\n"
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
      " [%1], [%6, {%7, %8, %9, %10}], [%4], {%14, %15};\n"
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
      " [%2], [%6, {%7, %11, %12, %13}], [%4], {%14, %15};\n"
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%3], [%16, {%17, %18}], [%4];\n"
      "selp.u32 %0, 1, 0, pn;\n"
      "}\n"
      : "=r"(free_next)
      : "r"(a0_dst), "r"(a1_dst), "r"(b_dst), "r"(full_bar), "r"(stage_bytes), "l"(reinterpret_cast<uint64_t>(tmap_x)),
        "r"(c), "r"(w0), "r"(h0), "r"(n0i), "r"(w1), "r"(h1), "r"(n1i), "h"(off_w), "h"(off_h),
        "l"(reinterpret_cast<uint64_t>(tmap_w)), "r"(k0), "r"(ncol), "r"(next_empty_bar), "r"(next_parity)
      : "memory");
  return free_next != 0;
}

// Arrive on `bar` once every tcgen05.mma issued so far by this thread has retired.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (thread i = lane i).
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
// The reverse: 32 registers per thread -> 32 lanes x 32 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ------------------------------------------------------------------ descriptors
// Shared-memory matrix descriptor (64-bit) for tcgen05.mma operands; the kernel assembles it from a
// precomputed low word (address + leading-dimension offset) and a constant high word.
//   [0,14)  start address >> 4      [16,30) leading-dim byte offset >> 4
//   [32,46) stride-dim byte offset >> 4   [46,48) descriptor version (1 on sm_100)
//   [49,52) base offset (0: stage buffers are 1024-B aligned)   [61,64) swizzle mode
// Swizzle modes: 0 none, 2 = 128 B, 4 = 64 B, 6 = 32 B.
// Instruction descriptor (32-bit) for kind::f16 / kind::tf32, dense, fp32 accumulate,
// both operands K-major.
//   [4,6) D format (1 = f32)   [7,10) A format   [10,13) B format
//   (kind::f16: 0 = f16, 1 = bf16; kind::tf32: 2 = tf32)
//   [15] A major, [16] B major (0 = K-major)   [17,23) N >> 3   [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc(uint32_t ab_format, uint32_t m, uint32_t n) {
  return (1u << 4) | (ab_format << 7) | (ab_format << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

}  // namespace ptx
}  // namespace tb200
