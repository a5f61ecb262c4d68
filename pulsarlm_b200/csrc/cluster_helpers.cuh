// Barriers in shared memory with bounded waits, and what a thread-block cluster adds:
// a peer's shared memory, stores that count their bytes on a peer's barrier, and the
// cluster's own barrier in two halves.
#pragma once

#include "common.cuh"

namespace {

constexpr uint32_t kWaitLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait: false after kWaitLimit tries or once another role has given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t tries = 0; tries < kWaitLimit; ++tries) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
        if ((tries & 1023u) == 1023u && *abort_flag) {
            return false;
        }
    }
    *abort_flag = 1;
    return false;
}

// ---- thread-block clusters: a peer's shared memory and barriers
// The address, in the cluster's shared window, of `local` in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t cluster_map(const void* local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    return remote;
}
// Stores four floats into a peer's shared memory (16-byte aligned) and counts their
// sixteen bytes on the peer's barrier, whose phase completes once the bytes it
// expects have arrived: the values carry their own completion, no fence or arrival
// follows.
__device__ __forceinline__ void cluster_store4_counted(uint32_t remote, float4 v, uint32_t remote_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
                 ::"r"(remote), "r"(__float_as_uint(v.x)), "r"(__float_as_uint(v.y)), "r"(__float_as_uint(v.z)),
                 "r"(__float_as_uint(v.w)), "r"(remote_bar)
                 : "memory");
}
// The same for two floats (8-byte aligned).
__device__ __forceinline__ void cluster_store2_counted(uint32_t remote, float2 v, uint32_t remote_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.b32 [%0], {%1, %2}, [%3];" ::"r"(remote),
                 "r"(__float_as_uint(v.x)), "r"(__float_as_uint(v.y)), "r"(remote_bar)
                 : "memory");
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t tries = 0; tries < kWaitLimit; ++tries) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (done) {
            return true;
        }
        if ((tries & 1023u) == 1023u && *abort_flag) {
            return false;
        }
    }
    *abort_flag = 1;
    return false;
}
// The cluster's barrier in two halves: every thread of every CTA arrives (without
// blocking); a thread that waits returns once all have arrived, and sees what they
// wrote before arriving.
__device__ __forceinline__ void cluster_arrive_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_all() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

}  // namespace
