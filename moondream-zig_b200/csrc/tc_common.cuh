// PTX wrappers shared by the tcgen05 kernels (GEMM and attention): mbarriers with bounded waits,
// TMA tile loads / stores, tcgen05 MMA / commit / TMEM loads, shared-memory matrix descriptors.
#pragma once

#include "md_internal.cuh"

namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

constexpr unsigned long long WAIT_BUDGET_NS = 1000000000ull;  // 1 s

// Bounded wait.  Returns false (and records the failure) instead of spinning forever.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                            md_devflags* flags, unsigned site,
                                            unsigned long long budget_ns = WAIT_BUDGET_NS) {
    const unsigned long long t0 = global_ns();
    for (unsigned spin = 0;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if ((spin & 63u) == 63u && global_ns() - t0 > budget_ns) {
            *abort_flag = 1;
            md_flag_timeout(flags, site);
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          md_devflags* flags, unsigned site) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, flags, site);
}

// Bounded wait of the push warps until EVERY epilogue warp has finished `target` tiles (one shared-memory word per
// epilogue warp).  A single count over all warps is not enough: the accumulators are double-buffered, so some warps
// may be a tile ahead of the others, and their extra counts would stand in for warps that have not stored yet.
static __device__ __noinline__ bool wait_stored(volatile unsigned* stored, int n_warps, unsigned target,
                                                volatile int* abort_flag, md_devflags* flags, unsigned site) {
    const unsigned long long t0 = global_ns();
    for (unsigned spin = 0;; ++spin) {
        unsigned least = stored[0];
        for (int e = 1; e < n_warps; ++e) least = min(least, stored[e]);
        if (least >= target) {
            __threadfence_block();
            return true;
        }
        if (*abort_flag) return false;
        if ((spin & 63u) == 63u && global_ns() - t0 > WAIT_BUDGET_NS) {
            *abort_flag = 1;
            md_flag_timeout(flags, site);
            return false;
        }
        __nanosleep(64);
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
// Fetch a tensor map (kernel parameter) into the TMA unit's descriptor cache ahead of its first use.
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src),
                 "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// tcgen05.mma (kind::f16, one CTA) with the shared-memory descriptors given as 32-bit halves (layout below).
// The issuing thread is a single lane, so
// every instruction it spends between two MMAs is tensor-pipe idle time when the MMAs are small: the high words
// (stride offset, version, swizzle) are loop constants and the low words (address | leading offset) advance by
// plain 32-bit adds.  ACC = true accumulates into D, false overwrites it.
__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
    return ((smem_addr >> 4) & 0x3FFFu) | ((lbo_bytes >> 4) << 16);
}
__device__ __forceinline__ uint32_t desc_hi(uint32_t sbo_bytes, uint32_t layout) {
    return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (layout << 29);
}
template <bool ACC>
__device__ __forceinline__ void tc_mma_f16_parts(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                 uint32_t b_hi, uint32_t idesc) {
    if (ACC)
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "setp.eq.u32 p, 1, 1;\n\t"
            "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
            ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "setp.ne.u32 p, 1, 1;\n\t"
            "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
            ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc)
            : "memory");
}
// The same product with the A operand in tensor memory (M = 128 rows = lanes, K-major, two 16-bit elements per
// 32-bit column: a k-step of 16 elements is 8 columns) and B in shared memory.
template <bool ACC>
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi,
                                              uint32_t idesc) {
    if (ACC)
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
            "setp.eq.u32 p, 1, 1;\n\t"
            "mov.b64 db, {%2, %3};\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
            ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
            "setp.ne.u32 p, 1, 1;\n\t"
            "mov.b64 db, {%2, %3};\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
            ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc)
            : "memory");
}
__device__ __forceinline__ void tc_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 8 consecutive halves (16-byte aligned) widened to f32.
__device__ __forceinline__ void load8(const __half* p, float (&f)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = __half22float2(h[i]);
        f[2 * i] = x.x;
        f[2 * i + 1] = x.y;
    }
}

// The fused glue of a GEMM epilogue on 8 consecutive output columns of one row: f32 accumulators in, four packed
// half2 out.  Every step keeps the reference's rounding point (one rounding to f16 after the product, after the
// bias, after the GELU, after each residual).  Sums of two f16 values are formed with packed f16 adds: an f16 + f16
// sum is exact in f32, so f16(f32(a) + f32(b)) and the correctly rounded f16 add are the same number; only the GELU
// needs f32 arithmetic.  (cq, row) is the position of the first column; N % 8 == 0 and 16-byte aligned operands.
__device__ __forceinline__ void epilogue_glue8(const uint32_t* acc_bits, const md_epilogue& ep, int row, int cq, int N,
                                               bool apply, uint32_t (&pk)[4]) {
    __half2 h[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(__uint_as_float(acc_bits[2 * j]), __uint_as_float(acc_bits[2 * j + 1]));
    if (apply) {
        if (ep.bias) {
            const uint4 u = *reinterpret_cast<const uint4*>(ep.bias + cq);
            const __half2* b = reinterpret_cast<const __half2*>(&u);
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __hadd2(h[j], b[j]);
        }
        if (ep.gelu) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 x = __half22float2(h[j]);
                h[j] = __floats2half2_rn(md_gelu_fast_f32(x.x), md_gelu_fast_f32(x.y));
            }
        }
        if (ep.residual) {
            const int rm = ep.residual_rows > 0 ? row % ep.residual_rows : row;
            const uint4 u = *reinterpret_cast<const uint4*>(ep.residual + (size_t)rm * N + cq);
            const __half2* b = reinterpret_cast<const __half2*>(&u);
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __hadd2(h[j], b[j]);
        }
        if (ep.residual2) {
            const uint4 u = *reinterpret_cast<const uint4*>(ep.residual2 + (size_t)row * N + cq);
            const __half2* b = reinterpret_cast<const __half2*>(&u);
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __hadd2(h[j], b[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) pk[j] = *reinterpret_cast<uint32_t*>(&h[j]);
}

// Shared-memory matrix descriptor (version 1, sm_100) as built by desc_lo / desc_hi:
//   bits 0-13 address >> 4, 16-29 leading byte offset >> 4, 32-45 stride byte offset >> 4, 46 version,
//   61-63 swizzle (2 = 128-byte, 4 = 64-byte, 6 = 32-byte, 0 = none).
//   K-major operand, 128B swizzle (rows of 64 halves = 128 B, 8-row groups 1024 B apart): leading offset
//   unused (16), stride offset 1024 B; 16 k further = +32 B.
//   MN-major operand, 128B swizzle (64-element chunks of the MN dimension contiguous, k rows 128 B apart,
//   8-k-row groups 1024 B apart): leading offset = distance of successive 64-element chunks, stride offset
//   1024 B; 16 k further = +2048 B.
//   32B swizzle: rows of 16 halves = 32 B, 8-row groups 256 B apart (stride offset 256 B).

}  // namespace tc
