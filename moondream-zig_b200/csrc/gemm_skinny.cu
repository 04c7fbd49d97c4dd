// Skinny GEMM for sm_100a: C[M,N] = A[M,K] . B with 8 < M <= 64 (a short prefill: the reference's own hgemm
// benchmark shape is 64 x 2048 . 2048 x 8192, hgemm.zig:446-542).  Such a product is bound by HBM, not by the tensor
// cores: B is read once (N*K*2 bytes) and everything else is small.  Two things keep the general tcgen05 kernel far
// from the HBM rate at these shapes, and this kernel removes both:
//
//   * operand roles are swapped.  The weights are the "M side" of the MMA (128 weight rows per tile) and the
//     activations the "N side" (64 columns), so a k-block of 64 costs 16 KB of weights + 8 KB of activations for
//     128 weight rows, instead of 8 KB + 16 KB (half of it zero fill) for 64 of them.  What bounds an SM here is
//     the bytes it pulls from L2 into shared memory, so this halves the time per weight row.
//   * K is split.  N / 128 tiles alone leave most SMs idle (64 tiles for N = 8192 on 148 SMs); with S splits of K
//     there are ~2 CTAs per SM, each streaming its own part of the weights.  The S CTAs of a tile form a thread-block
//     cluster: every CTA leaves its partial sums (f32, [64][128]) in its own shared memory, and after one cluster
//     barrier CTA r adds rows r, r + S, ... of all S partials through distributed shared memory, in a fixed order,
//     applies the fused glue and writes f16.  No global scratch, no tickets, no second kernel.  (A first version
//     reduced through an L2-resident workspace with a last-arriver ticket: 13 us of fences and dependent L2 round
//     trips for a product whose operands stream in 7.)
//
// Roles inside a CTA (192 threads): warp 0 TMA producer (weights are requested before the dependency wait of a
// programmatic dependent launch, activations after it), warp 1 one lane issuing tcgen05.mma (128 x 64 x 16, f32 in
// TMEM), warps 2..5 epilogue: tcgen05.ld of the transposed tile (TMEM lane = output column) into shared memory as
// [row][128 columns], then 16-byte pieces of rows go to the workspace or, through the glue, to C.
// Every mbarrier wait is bounded as in the general kernel.
#include "md_internal.cuh"
#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int TILE_N = 128;          // weight rows (output columns) per CTA
constexpr int XN = 64;               // activation rows covered by the MMA's N side (M <= 64)
constexpr int BLOCK_K = 64, UMMA_K = 16;
constexpr int W_STAGE_BYTES = TILE_N * BLOCK_K * 2;   // 16 KiB
constexpr int X_STAGE_BYTES = XN * BLOCK_K * 2;       // 8 KiB
constexpr int STAGE_BYTES = W_STAGE_BYTES + X_STAGE_BYTES;
constexpr int STAGES = 4;
constexpr int THREADS = 192;
constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 256;
constexpr uint32_t TMEM_COLS = 64;
constexpr int MAX_SPLITS = 8;          // portable cluster size

template <bool W_MN_MAJOR>
__global__ void __launch_bounds__(THREADS, 2)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, __half* C, int M,
                   int N, int K, int kb_per_split, int splits, md_epilogue ep, md_devflags* flags) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t smem_w = base, smem_x = base + STAGES * W_STAGE_BYTES;
    uint8_t* bars_ptr = base_ptr + STAGES * STAGE_BYTES;
    const uint32_t bars = base + STAGES * STAGE_BYTES;
    const uint32_t bar_full = bars, bar_empty = bars + 8 * STAGES, bar_done = bars + 16 * STAGES;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars_ptr + 16 * STAGES + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_ptr + 16 * STAGES + 12);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int n0 = tile * TILE_N;
    const int num_kb = (K + BLOCK_K - 1) / BLOCK_K;
    const int kb0 = split * kb_per_split;
    const int kbs = max(0, min(kb_per_split, num_kb - kb0));   // 0 for a split past the end of K: it contributes zeros

    md_pdl_launch_dependents();
    if (threadIdx.x == 0) {
        tma_prefetch_map(&tm_w);
        tma_prefetch_map(&tm_x);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_done, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(const_cast<uint32_t*>(tmem_slot))),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            auto load_w = [&](int stage, int kb) {
                const uint32_t full = bar_full + 8 * stage;
                mbar_expect_tx(full, STAGE_BYTES);
                if (W_MN_MAJOR) {
#pragma unroll
                    for (int j = 0; j < TILE_N / 64; ++j)
                        tma_load_2d(smem_w + stage * W_STAGE_BYTES + j * (64 * BLOCK_K * 2), &tm_w, full, n0 + j * 64,
                                    kb * BLOCK_K);
                } else {
                    tma_load_2d(smem_w + stage * W_STAGE_BYTES, &tm_w, full, kb * BLOCK_K, n0);
                }
            };
            auto load_x = [&](int stage, int kb) {
                tma_load_2d(smem_x + stage * X_STAGE_BYTES, &tm_x, bar_full + 8 * stage, kb * BLOCK_K, 0);
            };
            // the first ring of weight tiles does not depend on the predecessor kernel (registered weights are
            // never written on the stream): request it before waiting for the activations' producer
            const int first = min(kbs, STAGES);
            for (int i = 0; i < first; ++i) load_w(i, kb0 + i);
            md_pdl_wait();
            for (int i = 0; i < first; ++i) load_x(i, kb0 + i);
            int stage = first == STAGES ? 0 : first;
            uint32_t phase = first == STAGES ? 1u : 0u;
            for (int i = first; i < kbs; ++i) {
                mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, flags, 11);
                load_w(stage, kb0 + i);
                load_x(stage, kb0 + i);
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (*abort_flag) {
                const unsigned long long t0 = global_ns();
                while (global_ns() - t0 < 500000ull) {}
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        md_pdl_wait();
        if (lane == 0) {
            // D[128 weight rows, 64 activation rows] (f32), A = weights (K-major, or MN-major for the [K,N] layout),
            // B = activations (K-major)
            const uint32_t idesc = (1u << 4) | ((W_MN_MAJOR ? 1u : 0u) << 15) | ((uint32_t)(XN >> 3) << 17) |
                                   ((uint32_t)(TILE_N >> 4) << 24);
            constexpr uint32_t W_KSTEP = (W_MN_MAJOR ? UMMA_K * 128 : UMMA_K * 2) >> 4, X_KSTEP = (UMMA_K * 2) >> 4;
            const uint32_t hi = desc_hi(1024, 2);
            const uint32_t w_lo0 = desc_lo(smem_w, W_MN_MAJOR ? 64 * BLOCK_K * 2 : 16), x_lo0 = desc_lo(smem_x, 16);
            int stage = 0;
            uint32_t phase = 0;
            for (int i = 0; i < kbs; ++i) {
                mbar_wait(bar_full + 8 * stage, phase, abort_flag, flags, 12);
                tc_fence_after();
                const uint32_t w_lo = w_lo0 + (uint32_t)stage * (W_STAGE_BYTES >> 4);
                const uint32_t x_lo = x_lo0 + (uint32_t)stage * (X_STAGE_BYTES >> 4);
                if (i == 0) tc_mma_f16_parts<false>(tmem_base, w_lo, hi, x_lo, hi, idesc);
                else tc_mma_f16_parts<true>(tmem_base, w_lo, hi, x_lo, hi, idesc);
#pragma unroll
                for (int k = 1; k < BLOCK_K / UMMA_K; ++k)
                    tc_mma_f16_parts<true>(tmem_base, w_lo + k * W_KSTEP, hi, x_lo + k * X_KSTEP, hi, idesc);
                tc_commit(bar_empty + 8 * stage);
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (kbs > 0) tc_commit(bar_done);
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        md_pdl_wait();
        const int quad = warp & 3;                     // TMEM lane quadrant this warp may read
        const int nl = quad * 32 + lane;               // this thread's column of the tile
        // The accumulator goes to shared memory (the ring is idle: every MMA has retired), transposed to
        // [m][128 columns], where the CTAs of the cluster can read it.
        float* tile_f32 = reinterpret_cast<float*>(base_ptr);
        if (kbs > 0) {
            mbar_wait(bar_done, 0, abort_flag, flags, 13);
            tc_fence_after();
#pragma unroll
            for (int h = 0; h < XN / 32; ++h) {
                uint32_t r[32];
                tc_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(h * 32), r);
                tc_wait_ld();
#pragma unroll
                for (int j = 0; j < 32; ++j) tile_f32[(h * 32 + j) * TILE_N + nl] = __uint_as_float(r[j]);
            }
        } else {
#pragma unroll 8
            for (int m = 0; m < XN; ++m) tile_f32[m * TILE_N + nl] = 0.f;
        }
        tc_fence_before();
    }

    // every CTA's partial tile is complete and visible to the cluster
    __syncthreads();
    if (splits > 1) {
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    if (warp >= 2) {
        // CTA `split` (its rank in the cluster) finishes rows split, split + S, ...: four rows per turn, a thread
        // owns one 16-byte piece of a row; the S partials are read from the S CTAs' shared memory (its own included)
        // and added in the order 0 .. S-1, so the result does not depend on timing.
        const int et = threadIdx.x - 64;
        const int c4 = (et & 31) * 4, n = n0 + c4;
        const uint32_t tile_addr = base;   // shared-memory address of tile_f32 (same offset in every CTA of the cluster)
        auto finish = [&](int m, const float4& acc) {
            if (n >= N || m >= M) return;   // N % 8 == 0: a piece of four columns is inside or outside C
            const __half2 lo = __floats2half2_rn(md_epilogue_value(ep, acc.x, m, n, N), md_epilogue_value(ep, acc.y, m, n + 1, N));
            const __half2 hi = __floats2half2_rn(md_epilogue_value(ep, acc.z, m, n + 2, N), md_epilogue_value(ep, acc.w, m, n + 3, N));
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&lo);
            pk.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(C + (size_t)m * N + n) = pk;
        };
        // two turns at a time: all loads of both turns are issued before the first sum
        for (int ma = split + splits * (et >> 5); ma < M; ma += splits * 8) {
            const int mb = ma + splits * 4;   // may be >= M (rows past M hold zeros or stale sums: never stored)
            float4 pa[8], pb[8];
            const uint32_t la = tile_addr + (uint32_t)((ma * TILE_N + c4) * 4);
            const uint32_t lb = tile_addr + (uint32_t)(((mb < XN ? mb : ma) * TILE_N + c4) * 4);
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                if (s < splits) {
                    uint32_t ra, rb;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(la), "r"(s));
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rb) : "r"(lb), "r"(s));
                    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
                                 : "=f"(pa[s].x), "=f"(pa[s].y), "=f"(pa[s].z), "=f"(pa[s].w) : "r"(ra));
                    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
                                 : "=f"(pb[s].x), "=f"(pb[s].y), "=f"(pb[s].z), "=f"(pb[s].w) : "r"(rb));
                }
            }
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                if (s < splits) {
                    a.x += pa[s].x; a.y += pa[s].y; a.z += pa[s].z; a.w += pa[s].w;
                    b.x += pb[s].x; b.y += pb[s].y; b.z += pb[s].z; b.w += pb[s].w;
                }
            }
            finish(ma, a);
            finish(mb, b);
        }
    }
    if (splits > 1) {
        // nobody leaves while a peer may still read its shared memory
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

int md_make_map_2d(md_ctx* ctx, CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint32_t box_inner,
                   uint32_t box_outer, uint64_t ld);

bool md_gemm_skinny_supported(const void* a, const void* b, const void* c, size_t M, size_t N, size_t K) {
    if (M <= 8 || M > (size_t)XN || N == 0 || K == 0) return false;
    if ((K % 8) != 0 || (N % 8) != 0) return false;  // row strides must be multiples of 16 bytes for TMA
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) return false;
    if (reinterpret_cast<uintptr_t>(c) & 7) return false;  // 8-byte stores of four outputs
    return N <= (1u << 30) && K <= (1u << 30);
}

int md_launch_gemm_skinny(md_ctx* ctx, const __half* a, const __half* b, __half* c, size_t M, size_t N, size_t K,
                          int b_layout, const md_epilogue& ep) {
    if (!md_gemm_skinny_supported(a, b, c, M, N, K))
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "skinny GEMM needs 8 < M <= 64, K %% 8 == 0, N %% 8 == 0 and 16-byte aligned operands");
    const bool mn = (b_layout == 0);
    CUtensorMap tm_w, tm_x;
    if (mn) MD_TRY(md_make_map_2d(ctx, &tm_w, b, N, K, 64, BLOCK_K, 0));
    else MD_TRY(md_make_map_2d(ctx, &tm_w, b, K, N, BLOCK_K, TILE_N, 0));
    MD_TRY(md_make_map_2d(ctx, &tm_x, a, K, M, BLOCK_K, XN, 0));
    const int tiles = (int)((N + TILE_N - 1) / TILE_N);
    const int num_kb = (int)((K + BLOCK_K - 1) / BLOCK_K);
    // splits of K = CTAs per cluster: about two CTAs per SM in one wave, a power of two up to the portable cluster
    // size of 8, at least two k-blocks per split
    int want = ctx->skinny_splits > 0 ? ctx->skinny_splits : (2 * ctx->sm_count) / tiles;
    if (want > num_kb / 2) want = num_kb / 2;
    int splits = 1;
    while (splits * 2 <= want && splits * 2 <= MAX_SPLITS) splits *= 2;
    const int kb_per_split = (num_kb + splits - 1) / splits;
    const uint32_t cfg_bit = 1u << (mn ? 14 : 13);
    if (!(ctx->tc_configured & cfg_bit)) {
        if (mn) MD_CUDA(ctx, cudaFuncSetAttribute(gemm_skinny_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        else MD_CUDA(ctx, cudaFuncSetAttribute(gemm_skinny_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        ctx->tc_configured |= cfg_bit;
    }
    ctx->last_tc_tile = 1000 + splits;   // md_get_option("last_tc_tile"): 1000 + S = the skinny kernel with S splits
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)tiles, (unsigned)splits);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (splits > 1) {   // the splits of a tile are one cluster along y
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = (unsigned)splits;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (ctx->pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    const int Mi = (int)M, Ni = (int)N, Ki = (int)K;
    const cudaError_t e = mn ? cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<true>, tm_w, tm_x, c, Mi, Ni, Ki, kb_per_split, splits, ep, ctx->flags)
                             : cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<false>, tm_w, tm_x, c, Mi, Ni, Ki, kb_per_split, splits, ep, ctx->flags);
    if (e != cudaSuccess) return md_fail(ctx, MD_ERR_CUDA, "launch of gemm_skinny_kernel failed: %s", cudaGetErrorString(e));
    ctx->launches++;
    return MD_OK;
}
