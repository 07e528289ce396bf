// bulk_copy.cuh — cp.async.bulk (global -> shared) with mbarrier completion, and the
// cluster barrier, as inline PTX.  Every wait is bounded.
#pragma once
#include <stdint.h>

__device__ __forceinline__ uint32_t bc_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void bc_mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bc_mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void bc_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// The suspend-time hint parks the thread until the phase completes or ~10 us pass.
__device__ __forceinline__ bool bc_mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(10000u) : "memory");
    return ok != 0;
}
// bounded wait: gives up (returns false) after ~1 s instead of waiting for ever
__device__ __forceinline__ bool bc_mbar_wait(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < (1 << 17); i++)
        if (bc_mbar_try_wait(bar, parity)) return true;
    return false;
}
// dst, src 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bc_copy(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bc_fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// hardware cluster barrier, split into arrive and wait; every thread of every CTA of
// the cluster executes both, the same number of times
__device__ __forceinline__ void bc_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void bc_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }
__device__ __forceinline__ uint32_t bc_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// address of this CTA's shared variable `p` inside CTA `rank` of the cluster
__device__ __forceinline__ uint32_t bc_map_rank(const void *p, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(a) : "r"(bc_smem_u32(p)), "r"(rank));
    return a;
}
