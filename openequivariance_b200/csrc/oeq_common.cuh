// Device-side building blocks shared by the sm_100a kernels: compile-time loops,
// mbarrier / bulk-copy (TMA) wrappers with bounded waits, named group barriers.
//
// The kernels are compiled at run time (NVRTC) against a small generated
// "problem descriptor" (namespace oeqd) that holds only constexpr tables; all
// kernel bodies live in these hand-written headers.
#pragma once

namespace oeq {

template <int V>
struct IC {
    static constexpr int value = V;
    __device__ __forceinline__ constexpr operator int() const { return V; }
};

// Compile-time loop over [B, E) by binary splitting (template depth is log2(E-B)).
template <int B, int E, class F>
__device__ __forceinline__ void sfor(F&& f) {
    if constexpr (E - B == 1) {
        f(IC<B>{});
    } else if constexpr (E - B > 1) {
        constexpr int M = (B + E) / 2;
        sfor<B, M>(f);
        sfor<M, E>(f);
    }
}

__device__ __forceinline__ unsigned smem_u32(const void* p) {
    return static_cast<unsigned>(__cvta_generic_to_shared(p));
}

// Error codes written to the status word by a kernel that gave up on a wait.
constexpr int ERR_WAIT_FULL = 1;
constexpr int ERR_WAIT_EMPTY = 2;
constexpr int ERR_WAIT_STORE = 3;

// Upper bound on polls of one mbarrier phase (each poll is a try_wait with a
// hardware-side suspend window, so this is on the order of a second).
constexpr unsigned WAIT_LIMIT = 1u << 20;

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(
                     smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: returns false (and records why) instead of spinning for ever.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, int* status, int code) {
    for (unsigned spin = 0; spin < WAIT_LIMIT; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    if (status) atomicCAS(status, 0, code);
    return false;
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Make generic-proxy writes to shared memory visible to the async (TMA) proxy.
__device__ __forceinline__ void fence_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// global -> shared bulk copy (1-D TMA, no tensor map, one destination CTA); both
// addresses 16-byte aligned, bytes a multiple of 16; completion on `bar`.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, unsigned bytes,
                                         unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// L2 eviction policies for bulk copies: rows that are gathered again soon (node features, output
// gradients) should outlive the per-edge arrays that stream through the cache exactly once.
__device__ __forceinline__ unsigned long long l2_policy_evict_first() {
    unsigned long long pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ unsigned long long l2_policy_evict_last() {
    unsigned long long pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void* dst_smem, const void* src_gmem, unsigned bytes,
                                              unsigned long long* bar, unsigned long long policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// shared -> global bulk copy, tracked by the issuing thread's bulk async-group.
__device__ __forceinline__ void bulk_s2g(void* dst_gmem, const void* src_smem, unsigned bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem),
                 "r"(smem_u32(src_smem)), "r"(bytes)
                 : "memory");
}

// shared -> global bulk reduction (element-wise add performed at L2).
__device__ __forceinline__ void bulk_red_add_f32(float* dst_gmem, const void* src_smem, unsigned bytes) {
    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst_gmem),
                 "r"(smem_u32(src_smem)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_red_add_f64(double* dst_gmem, const void* src_smem, unsigned bytes) {
    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f64 [%0], [%1], %2;" ::"l"(dst_gmem),
                 "r"(smem_u32(src_smem)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// Ampere-style asynchronous element copy for rows that do not meet the
// 16-byte rule of the bulk copy (4- or 8-byte granularity).
template <int BYTES>
__device__ __forceinline__ void cp_async_elem(void* dst_smem, const void* src_gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "n"(BYTES)
                 : "memory");
}
// 16-byte variant (both addresses 16-byte aligned), bypassing L1.
__device__ __forceinline__ void cp_async_16(void* dst_smem, const void* src_gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem) : "memory");
}
// Arrive on `bar` once all prior cp.async of this thread have landed (the
// arrival is one of the barrier's expected arrivals: ".noinc").
__device__ __forceinline__ void cp_async_arrive_noinc(unsigned long long* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Barrier over `count` threads (a multiple of 32) using hardware barrier `id` (1..15).
__device__ __forceinline__ void group_sync(int id, int count) {
    if (count == 32) {
        __syncwarp();
    } else {
        asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
    }
}

template <class T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

template <class T>
__device__ __forceinline__ void red_add(T* addr, T v) {
    atomicAdd(addr, v);
}

}  // namespace oeq
