// Tensor-core GEMM on CTA pairs (tcgen05 cta_group::2) for sm_100a: C[M,N] = A[M,K] . B with many rows.
//
// The single-CTA kernel (gemm_tc.cu) is bound by the bytes an SM pulls from L2 into shared memory: a 128 x 256 tile
// costs 16 KB of A + 32 KB of B per k-block of 64 for 512 tensor cycles, and the path delivers about 50 B per cycle.
// Here two CTAs on neighbouring SMs (a cluster of 2) compute one 256 x 256 tile together: each CTA loads its own 128
// rows of A and its own HALF of the B tile (128 of the 256 columns) with ordinary TMA loads, 32 KB per k-block, and
// one thread of the pair's first CTA issues tcgen05.mma.cta_group::2 (M = 256), which reads both halves of B from the
// two CTAs' shared memories and accumulates each CTA's 128 rows in that CTA's own tensor memory.  Every SM still
// covers 128 x 256 per tile, its accumulators stay double-buffered (2 x 256 TMEM columns), and it pulls a third less
// from L2.  No load is multicast; nothing is read from another GPU.
//
// Protocol (barriers live at the same shared-memory offsets in both CTAs; "leader" = cluster rank 0):
//   full[s]    leader's only: one arrival (the leader's producer announces the 64 KB of both CTAs) + the bytes of both
//              CTAs' TMA loads, which name the leader's barrier (cp.async.bulk.tensor ... .cta_group::2)
//   empty[s]   per CTA: the leader's issuing thread commits its MMAs to its own and to the second CTA's barrier
//   tfull[b]   per CTA: committed the same way when a tile's accumulators are complete
//   tempty[b]  leader's only: 16 arrivals, the 8 epilogue warps of each CTA (the second CTA's remotely)
// Every wait is bounded as in the single-CTA kernel; the two cluster barriers (set-up, tear-down) are unconditional.
#include <cstring>

#include "md_internal.cuh"
#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int BLOCK_M = 128, BLOCK_N = 256, HALF_N = 128, BLOCK_K = 64, UMMA_K = 16;
constexpr int A_STAGE_BYTES = BLOCK_M * BLOCK_K * 2;   // 16 KiB
constexpr int B_STAGE_BYTES = HALF_N * BLOCK_K * 2;    // 16 KiB: this CTA's half of the B tile
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int STAGES = 6;
constexpr int EPI_WARPS = 8, EPI_BUF_BYTES = 32 * 128, EPI_BYTES = EPI_WARPS * EPI_BUF_BYTES;
constexpr int NUM_THREADS = (2 + EPI_WARPS) * 32;
constexpr int PUSH_WARPS = 8;                            // extra warps of the column-split form
constexpr int NUM_THREADS_PUSH = NUM_THREADS + PUSH_WARPS * 32;
constexpr int BAR_BYTES = 1024;
constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES;   // 231,424 of the 232,448 available
constexpr uint32_t TMEM_COLS = 512;
constexpr int RASTER_GROUP_M = 4;   // pair-tile rows (256 matrix rows each) per rasterisation group

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
// TMA tile load whose completion bytes go to a barrier of this CTA or of the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <bool ACC>
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                            uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.eq.u32 p, %6, 1;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(ACC ? 1u : 0u)
        : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Linear pair-tile index -> (tile row, tile column), groups of RASTER_GROUP_M tile rows, row fastest inside a group.
__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int per_group = RASTER_GROUP_M * tiles_n;
    const int g = tile / per_group, r = tile - g * per_group;
    const int m_first = g * RASTER_GROUP_M;
    const int rows = min(RASTER_GROUP_M, tiles_m - m_first);
    tm = m_first + r % rows;
    tn = r / rows;
}

// PUSH = the column-split form: eight more warps per CTA copy every finished tile (this CTA's 128 rows of it) from
// this GPU's C into the peers' C, as in the single-CTA kernel (its own instantiation, so that the plain kernel keeps
// the register budget of 320 threads).
template <bool B_MN_MAJOR, bool PUSH>
__global__ void __launch_bounds__(PUSH ? NUM_THREADS_PUSH : NUM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_c, int M, int N, int K, int tiles_m, int num_tiles,
                 md_epilogue ep, md_push push, md_devflags* flags, const __grid_constant__ md_peer_maps pm) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t smem_a = base;
    const uint32_t smem_b = base + STAGES * A_STAGE_BYTES;
    const uint32_t smem_epi = base + STAGES * STAGE_BYTES;
    uint8_t* epi_ptr = base_ptr + STAGES * STAGE_BYTES;
    const uint32_t bars = smem_epi + EPI_BYTES;
    uint8_t* bars_ptr = epi_ptr + EPI_BYTES;
    const uint32_t bar_full = bars, bar_empty = bars + 8 * STAGES;
    const uint32_t bar_tfull = bars + 16 * STAGES, bar_tempty = bar_tfull + 16;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars_ptr + 16 * STAGES + 32);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_ptr + 16 * STAGES + 36);
    // per epilogue warp: the number of this CTA's tiles it has finished (all of its TMA stores complete)
    volatile unsigned* stored = reinterpret_cast<volatile unsigned*>(bars_ptr + 16 * STAGES + 40);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();   // 0 = leader (issues the MMAs), 1 = second CTA of the pair
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int num_kb = (K + BLOCK_K - 1) / BLOCK_K;
    const int tiles_n = num_tiles / tiles_m;

    md_pdl_launch_dependents();
    if (threadIdx.x == 0) {
        tma_prefetch_map(&tm_a);
        tma_prefetch_map(&tm_b);
        tma_prefetch_map(&tm_c);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);    // the leader's producer announces both CTAs' bytes (used in the leader only)
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_tfull + 8 * b, 1);
            mbar_init(bar_tempty + 8 * b, 2 * EPI_WARPS);   // both CTAs' epilogue warps (used in the leader only)
        }
        *abort_flag = 0;
        for (int e = 0; e < EPI_WARPS; ++e) stored[e] = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // one warp of each CTA of the pair takes part in the allocation; both CTAs get the same columns
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(const_cast<uint32_t*>(tmem_slot))),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // both CTAs' barriers are initialised before anyone signals them remotely
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    md_pdl_wait();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            const uint32_t leader_full = map_to(bar_full, 0);
            for (int tile = pair; tile < num_tiles; tile += num_pairs) {
                int tm, tn;
                pair_tile_coords(tile, tiles_m, tiles_n, tm, tn);
                const int m0 = tm * (2 * BLOCK_M) + (int)rank * BLOCK_M;   // this CTA's 128 rows of A
                const int n0 = tn * BLOCK_N + (int)rank * HALF_N;          // this CTA's 128 columns of B
                for (int kb = 0; kb < num_kb; ++kb) {
                    mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, flags, 21);
                    // the leader announces the bytes of both CTAs on its own barrier (a plain local arrive: a remote
                    // arrive per k-block from the second CTA cost 0.7 us each); the second CTA's loads only name it
                    uint32_t full = bar_full + 8 * stage;
                    if (rank == 0) mbar_expect_tx(full, 2 * STAGE_BYTES);
                    else full = leader_full + 8 * stage;
                    tma_load_2d_pair(smem_a + stage * A_STAGE_BYTES, &tm_a, full, kb * BLOCK_K, m0);
                    if (B_MN_MAJOR) {
#pragma unroll
                        for (int j = 0; j < HALF_N / 64; ++j)
                            tma_load_2d_pair(smem_b + stage * B_STAGE_BYTES + j * (64 * BLOCK_K * 2), &tm_b, full,
                                             n0 + j * 64, kb * BLOCK_K);
                    } else {
                        tma_load_2d_pair(smem_b + stage * B_STAGE_BYTES, &tm_b, full, kb * BLOCK_K, n0);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (*abort_flag) {
                const unsigned long long t0 = global_ns();
                while (global_ns() - t0 < 500000ull) {}
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader only)
        if (lane == 0 && rank == 0) {
            // M = 256 over the pair (128 rows per CTA), N = 256, f32 accumulators
            const uint32_t idesc = (1u << 4) | ((B_MN_MAJOR ? 1u : 0u) << 16) | ((uint32_t)(BLOCK_N >> 3) << 17) |
                                   ((uint32_t)((2 * BLOCK_M) >> 4) << 24);
            constexpr uint32_t A_KSTEP = (UMMA_K * 2) >> 4, B_KSTEP = (B_MN_MAJOR ? UMMA_K * 128 : UMMA_K * 2) >> 4;
            const uint32_t a_hi = desc_hi(1024, 2), b_hi = desc_hi(1024, 2);
            const uint32_t a_lo0 = desc_lo(smem_a, 16), b_lo0 = desc_lo(smem_b, B_MN_MAJOR ? 64 * BLOCK_K * 2 : 16);
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            const uint32_t peer_empty = map_to(bar_empty, 1), peer_tfull = map_to(bar_tfull, 1);
            for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local) {
                const int buf = local & 1;
                const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
                mbar_wait(bar_tempty + 8 * buf, acc_phase ^ 1u, abort_flag, flags, 22);
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BLOCK_N);
                for (int kb = 0; kb < num_kb; ++kb) {
                    mbar_wait(bar_full + 8 * stage, phase, abort_flag, flags, 23);
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + (uint32_t)stage * (A_STAGE_BYTES >> 4);
                    const uint32_t b_lo = b_lo0 + (uint32_t)stage * (B_STAGE_BYTES >> 4);
                    if (kb == 0) tc_mma_pair<false>(tmem_d, a_lo, a_hi, b_lo, b_hi, idesc);
                    else tc_mma_pair<true>(tmem_d, a_lo, a_hi, b_lo, b_hi, idesc);
#pragma unroll
                    for (int k = 1; k < BLOCK_K / UMMA_K; ++k)
                        tc_mma_pair<true>(tmem_d, a_lo + k * A_KSTEP, a_hi, b_lo + k * B_KSTEP, b_hi, idesc);
                    // both CTAs' stages are free once these MMAs retire
                    tc_commit_pair(bar_empty + 8 * stage);
                    tc_commit_pair(peer_empty + 8 * stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                tc_commit_pair(bar_tfull + 8 * buf);   // accumulators complete, in both CTAs' tensor memory
                tc_commit_pair(peer_tfull + 8 * buf);
            }
        }
    } else if (warp < 2 + EPI_WARPS) {
        // ------------------------------------------------------------ epilogue (warps 2..9, both CTAs)
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;
        const uint32_t my_epi = smem_epi + (uint32_t)(warp - 2) * EPI_BUF_BYTES;
        uint8_t* my_epi_ptr = epi_ptr + (warp - 2) * EPI_BUF_BYTES;
        const bool any_glue = ep.bias || ep.residual || ep.residual2 || ep.gelu;
        const uint32_t leader_tempty = map_to(bar_tempty, 0);
        constexpr int CHUNKS = BLOCK_N / 64;
        int local = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local) {
            int tm, tn;
            pair_tile_coords(tile, tiles_m, tiles_n, tm, tn);
            const int m0 = tm * (2 * BLOCK_M) + (int)rank * BLOCK_M, n0 = tn * BLOCK_N;
            const int buf = local & 1;
            const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
            mbar_wait(bar_tfull + 8 * buf, acc_phase, abort_flag, flags, 24);
            tc_fence_after();
#pragma unroll 1
            for (int c = half; c < CHUNKS; c += 2) {
                const int mrow0 = m0 + quad * 32, row = mrow0 + lane;
                const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BLOCK_N);
                if (lane == 0) tma_store_wait_read<0>();
                __syncwarp();
                uint8_t* out_row = my_epi_ptr + lane * 128;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t r[32];
                    tc_ld_32x32(t_row + (uint32_t)(c * 64 + h * 32), r);
                    tc_wait_ld();
                    const int col0 = n0 + c * 64 + h * 32;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int cq = col0 + 8 * q;
                        uint32_t pk[4];
                        epilogue_glue8(r + 8 * q, ep, row, cq, N, any_glue && row < M && cq < N, pk);
                        const int chunk = (h * 4 + q) ^ (lane & 7);  // 128-byte swizzle, matches the store map
                        *reinterpret_cast<uint4*>(out_row + chunk * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
                if (c + 2 >= CHUNKS) {
                    // all of this warp's TMEM reads of the tile are done: hand the buffer back to the leader
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(leader_tempty + 8 * buf);
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(&tm_c, my_epi, n0 + c * 64, mrow0);
                    if (PUSH && push.tma) {
                        // the same staged chunk into every peer's C, starting with a different peer in every CTA
                        for (int pi = 0; pi < push.n; ++pi) {
                            int peer = pi + (int)blockIdx.x;
                            peer -= (peer / push.n) * push.n;
                            tma_store_2d(&pm.m[peer], my_epi, n0 + c * 64, mrow0);
                        }
                    }
                    tma_store_commit();
                }
            }
            if (PUSH && !push.tma && lane == 0) {
                // this warp's part of the tile is in this GPU's C once its TMA stores have completed: tell the
                // push warps (every epilogue warp counts its own tiles)
                tma_store_wait_all();
                __threadfence_block();
                stored[warp - 2] = (unsigned)(local + 1);
            }
        }
        if (lane == 0) tma_store_wait_all();
    } else if (PUSH) {
        // ------------------------------------------------------------ push (warps 10..17, column-split GEMM)
        // This CTA's 128 x 256 part of every tile of the pair, read back from this GPU's C and stored into every
        // peer's C: a warp instruction covers one whole tile row (512 contiguous bytes), eight row groups are
        // requested before their peer stores are issued.
        constexpr int UNR = 8, ROW_STEP = PUSH_WARPS;
        const int pw = warp - (2 + EPI_WARPS);
        const int cl = lane * 8, ld = (int)push.ld;
        int local = 0;
        for (int tile = pair; tile < num_tiles && !push.tma; tile += num_pairs, ++local) {
            int tm, tn;
            pair_tile_coords(tile, tiles_m, tiles_n, tm, tn);
            const int m0 = tm * (2 * BLOCK_M) + (int)rank * BLOCK_M, n0 = tn * BLOCK_N;
            if (!wait_stored(stored, EPI_WARPS, (unsigned)(local + 1), abort_flag, flags, 25)) break;
            const int gc = n0 + cl;
            if (gc >= N) continue;  // columns past this rank's block belong to a neighbour
            const long long tile_off = (long long)m0 * push.ld + gc;
            for (int r = pw; r < BLOCK_M; r += ROW_STEP * UNR) {
                uint4 val[UNR];
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    const int rr = r + u * ROW_STEP;
                    if (rr < BLOCK_M && m0 + rr < M) val[u] = __ldcg(reinterpret_cast<const uint4*>(push.self + tile_off + rr * ld));
                }
                for (int pi = 0; pi < push.n; ++pi) {
                    // start with a different peer in every CTA so that the stores spread over the links
                    int peer = pi + (int)blockIdx.x;
                    peer -= (peer / push.n) * push.n;
                    __half* dst = push.base[peer] + tile_off;
#pragma unroll
                    for (int u = 0; u < UNR; ++u) {
                        const int rr = r + u * ROW_STEP;
                        if (rr < BLOCK_M && m0 + rr < M) *reinterpret_cast<uint4*>(dst + rr * ld) = val[u];
                    }
                }
            }
        }
        __threadfence_system();  // peer stores performed before the kernel ends
    }

    // nobody frees tensor memory or leaves while the pair's MMAs may still read its shared memory
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

int md_make_map_2d(md_ctx* ctx, CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint32_t box_inner,
                   uint32_t box_outer, uint64_t ld);

// C[M,N] = A . B (+ fused glue) on CTA pairs.  Same operand rules as the single-CTA kernel (K % 8 == 0, N % 8 == 0,
// 16-byte aligned pointers, C with row stride ldc); the caller decides when the shape is large enough to pay for the
// pairing.  push.n > 0: the column-split form (every tile also stored into the peers' C).
int md_launch_gemm_pair(md_ctx* ctx, const __half* a, const __half* b, __half* c, size_t M, size_t N, size_t K, int b_layout,
                        const md_epilogue& ep, size_t ldc, const md_push& push) {
    const bool mn = (b_layout == 0), with_push = push.n > 0;
    CUtensorMap tm_a, tm_b, tm_c;
    MD_TRY(md_make_map_2d(ctx, &tm_a, a, K, M, BLOCK_K, BLOCK_M, 0));
    if (mn) MD_TRY(md_make_map_2d(ctx, &tm_b, b, N, K, 64, BLOCK_K, 0));
    else MD_TRY(md_make_map_2d(ctx, &tm_b, b, K, N, BLOCK_K, HALF_N, 0));
    MD_TRY(md_make_map_2d(ctx, &tm_c, c, N, M, 64, 32, ldc));
    const int tiles_m = (int)((M + 2 * BLOCK_M - 1) / (2 * BLOCK_M)), tiles_n = (int)((N + BLOCK_N - 1) / BLOCK_N);
    const int num_tiles = tiles_m * tiles_n;
    const int max_pairs = ctx->sm_count / 2;
    const int pairs = num_tiles < max_pairs ? num_tiles : max_pairs;
    md_peer_maps pm;
    memset(&pm, 0, sizeof(pm));
    if (with_push && push.tma)
        for (int i = 0; i < push.n; ++i) MD_TRY(md_make_map_2d(ctx, &pm.m[i], push.base[i], N, M, 64, 32, ldc));
    void (*kern)(CUtensorMap, CUtensorMap, CUtensorMap, int, int, int, int, int, md_epilogue, md_push, md_devflags*,
                 md_peer_maps) =
        with_push ? (mn ? gemm_pair_kernel<true, true> : gemm_pair_kernel<false, true>)
                  : (mn ? gemm_pair_kernel<true, false> : gemm_pair_kernel<false, false>);
    const uint32_t cfg_bit = 1u << ((mn ? 1 : 0) + (with_push ? 2 : 0));
    if (!(ctx->pair_configured & cfg_bit)) {
        MD_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        ctx->pair_configured |= cfg_bit;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(with_push ? NUM_THREADS_PUSH : NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 2 : 1;
    ctx->last_tc_tile = 2256;   // md_get_option("last_tc_tile"): 2256 = a 256 x 256 tile on a CTA pair
    const int Mi = (int)M, Ni = (int)N, Ki = (int)K;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tm_a, tm_b, tm_c, Mi, Ni, Ki, tiles_m, num_tiles, ep, push, ctx->flags, pm);
    if (e != cudaSuccess) return md_fail(ctx, MD_ERR_CUDA, "launch of gemm_pair_kernel failed: %s", cudaGetErrorString(e));
    ctx->launches++;
    return MD_OK;
}
