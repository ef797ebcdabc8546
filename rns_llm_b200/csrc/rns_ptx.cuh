// PTX wrappers and small device helpers shared by the sm_100a GEMM kernels:
// mbarriers, TMA / bulk copies, tensor memory, tcgen05.mma, bounded waits.
#pragma once

#include <cuda.h>
#include <cstdint>

namespace rns {

constexpr long long kWaitLimitCycles = 4000000000ll;  // about 2 s of SM clock

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
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
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking test of a phase (never suspends the thread).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t holder_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem),
                 "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
                 : "memory");
}
// True in exactly one lane of a fully active warp (the same lane every time).
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                        uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t holder_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem),
                 "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                             uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the barrier at this shared-memory offset in BOTH CTAs of the pair
// once the MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"((uint16_t)3)
        : "memory");
}
// Arrive on the barrier at the same offset in another CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar, uint32_t cta_rank) {
    asm volatile(
        "{\n\t.reg .b32 remote;\n\t"
        "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [remote];\n\t}"
        ::"r"(bar), "r"(cta_rank)
        : "memory");
}
// The same without the cluster-scope release (which costs the arriving thread more than a
// thousand cycles): for data that lives in the arriving CTA's shared memory and whose writes
// the arriving thread has already seen complete through a CTA-scope acquire or a warp barrier.
__device__ __forceinline__ void mbar_arrive_remote_relaxed(uint32_t bar, uint32_t cta_rank) {
    asm volatile(
        "{\n\t.reg .b32 remote;\n\t"
        "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
        "mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [remote];\n\t}"
        ::"r"(bar), "r"(cta_rank)
        : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int (&v)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major operand tile with 64- or 128-byte swizzle: rows of tile_k bytes,
// groups of 8 rows 8*tile_k bytes apart.  Fields as in the sm_100 matrix
// descriptor: start>>4 [0,14), leading offset [16,30) (unused for swizzled
// K-major, set to 1), stride offset>>4 [32,46), version=1 [46,48), swizzle
// mode [61,64) (2 = 128B, 4 = 64B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t tile_k) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)((8u * tile_k) >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(tile_k == 128 ? 2 : 4) << 61;
    return d;
}
// Instruction descriptor: S32 accumulate [4,6)=2, signed 8-bit A [7,10)=1 and
// B [10,13)=1, both K-major, N>>3 at [17,23), M>>4 at [24,29).
__device__ __forceinline__ uint32_t make_idesc(uint32_t m, uint32_t n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Waits for `parity` of `bar`; false (and *abort set) when the time limit passes
// or another thread of the CTA already gave up.  `where` names the wait (role and
// pipeline stage, see wait_code); the first wait of a CTA that expires leaves it in
// *abort, and the kernel's teardown reports it to the host.
// SPIN: poll with test_wait instead of the suspending try_wait; for the single
// threads whose wake-up latency is on the critical path of every K block.
template <bool CLUSTER = false, bool SPIN = false>
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort, int where = 1) {
    auto poll = [&]() {
        return CLUSTER ? mbar_try_wait_cluster(bar, parity)
                       : (SPIN ? mbar_test_wait(bar, parity) : mbar_try_wait(bar, parity));
    };
    // Fast path: no clock is read unless the wait keeps failing (reading the global
    // timer costs hundreds of cycles, which every blocked wait would otherwise pay).
#ifndef RNS_SPIN_SLEEP_NS
#define RNS_SPIN_SLEEP_NS 20   // back-off between polls of a spinning lane: frees issue slots for the encoders
#endif
    for (int i = 0; i < 64; ++i) {
        if (poll()) return true;
        if (SPIN && RNS_SPIN_SLEEP_NS > 0 && i >= 4) __nanosleep(RNS_SPIN_SLEEP_NS);
    }
    long long t0 = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (poll()) return true;
        if (SPIN && RNS_SPIN_SLEEP_NS > 0) __nanosleep(RNS_SPIN_SLEEP_NS);
        if ((spin & 255u) == 0) {
            if (*abort) return false;
            if (clock64() - t0 > kWaitLimitCycles) {
                if (*abort == 0) *abort = where;
                return false;
            }
        }
    }
}
// Code of one wait: which role gave up (1 raw-tile producer, 2 plane producer, 3/4 pair
// relay on operands/planes, 5/6/7 MMA issuer on operands/planes/peer, 8/9 encoders on a
// released operand slot, 10 encoders on raw tiles, 11 epilogue on the accumulators) and
// at which pipeline stage.  Never zero.
__device__ __forceinline__ int wait_code(int role, int stage) { return (role << 20) | (stage & 0xfffff); }

// The same for a whole (converged) warp, with a warp-uniform result.
#ifndef RNS_LANE0_POLL
#define RNS_LANE0_POLL 0   // measured: all lanes polling is faster than one lane + shuffle
#endif
template <bool CLUSTER = false, bool SPIN = false>
__device__ __forceinline__ bool warp_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort, int where = 1) {
#if RNS_LANE0_POLL
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = wait_bounded<CLUSTER, SPIN>(bar, parity, abort, where) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
#else
    return __all_sync(0xffffffffu, wait_bounded<CLUSTER, SPIN>(bar, parity, abort, where));
#endif
}

// Registers -> tensor memory: 16 consecutive 32-bit columns of this warp's 32 lanes.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, "
        "%13, %14, %15, %16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (128 rows x 32 bytes of K) is read
// from tensor memory, 8 columns per call.
__device__ __forceinline__ void umma_i8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                           uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Stores through an NVLink multicast address (NVLS): the switch delivers the bytes to the same
// offset of every GPU bound to the multicast object.  16 bytes, and one 32-bit word.
__device__ __forceinline__ void multimem_store16(void* mc_addr, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(mc_addr), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
                   "f"(__uint_as_float(v.w))
                 : "memory");
}
__device__ __forceinline__ void multimem_store_u32(void* mc_addr, uint32_t v) {
    asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(mc_addr), "r"(v) : "memory");
}

}  // namespace rns
