// Device primitives shared by the kernels that stream weight rows through a shared-memory ring
// (decode_persistent.cu, gemv_ring.cu): bulk copies global -> shared with mbarrier completion, the mma.sync
// GEMV fragments, cp.async for activation pieces, cache-hinted loads.
#pragma once
#include "md_internal.cuh"

namespace ring {

constexpr int RING_K = 2048;                     // halves per weight row piece in a ring stage
constexpr int ROW_PITCH = RING_K * 2 + 64;       // bytes; +64 keeps the 8 rows of a fragment read on distinct banks
constexpr int STAGE_BYTES = 8 * ROW_PITCH;       // 8 rows x 2048 halves = 33280 bytes
constexpr int XS_PITCH = RING_K + 32;            // halves per activation row in shared memory, same bank argument

// The weight stream is marked evict-first in L2: 2.6 GB per step pass through, and they must not push out the
// small operands (parameters, cache rows) that were prefetched for the phases ahead.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_load_row(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar), "l"(pol)
        : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 ldcg128(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ldnc128(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ float ldcg_f16(const __half* p) {
    unsigned short u;
    asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(u) : "l"(p) : "memory");
    __half_raw r;
    r.x = u;
    return __half2float(__half(r));
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = __half22float2(h[i]);
        f[2 * i] = x.x;
        f[2 * i + 1] = x.y;
    }
}

// rows [r0, r1) of `total` owned by CTA `cta` of `n`
__device__ __forceinline__ void row_range(int total, int cta, int n, int& r0, int& r1) {
    r0 = (int)(((long long)total * cta) / n);
    r1 = (int)(((long long)total * (cta + 1)) / n);
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ float ldnc_f16(const __half* p) {
    unsigned short u;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(u) : "l"(p));
    __half_raw r;
    r.x = u;
    return __half2float(__half(r));
}

}  // namespace ring
