// Tensor-core GEMM for sm_100a: C[M,N] = A[M,K] . B, f16 operands, f32 accumulation in
// tensor memory, one rounding to f16, optional fused glue.  B is [N,K] ("NT",
// hgemm_trans.zig:400-488) or [K,N] ("NN", hgemm.zig:362-426).
//
// Structure (one persistent CTA per SM, 320 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor loads of the A tile (128 x 64) and the
//               B tile (BLOCK_N x 64) into a ring of shared-memory stages, 128-byte swizzle.
//   warp 1      MMA issuer: one lane issues tcgen05.mma (128 x BLOCK_N x 16, kind::f16) with
//               shared-memory descriptors; accumulators live in TMEM, two buffers of
//               BLOCK_N columns so the epilogue of tile i overlaps the main loop of tile i+1.
//               tcgen05.commit releases smem stages and publishes finished accumulators.
//               Large problems use a 256 x 256 tile: two 128-row sub-tiles of A against one B
//               tile per k-block (two MMAs per k-step, accumulators in TMEM columns 0-255 and
//               256-511), because the kernel is bound by the bytes an SM pulls from L2 per flop:
//               64 KB per 1024 tensor cycles instead of 48 KB per 512.
//   warps 2..9  epilogue: tcgen05.ld (32 lanes x 32 columns) -> fused glue -> f16 ->
//               swizzled smem -> TMA store (clips the M and N tails).
//               Column-split GEMM (push.tma): every staged chunk also leaves as one TMA store per peer into
//               the other GPUs' copies of C; the warp goes on when the stores have read the chunk.
//   warps 10..17 (column-split GEMM with push.tma = 0) push: once a tile's TMA stores have completed they read
//               the tile back from this GPU's C (L2 hits) and store it into the other GPUs' copies of C with
//               plain 16-byte peer stores.  The epilogue warps never wait for NVLink: they hand the accumulator
//               back to the MMA issuer as before, and the push of tile i runs beside the main loop of the
//               following tiles.
// Tiles are walked in groups of 8 tile rows (all tile columns of a group before the next group), so that the
// CTAs of one wave share a few A row blocks and a band of B in L2 instead of streaming all of A per wave.
// Tails: TMA zero-fills out-of-bounds loads and clips out-of-bounds stores, so any M, N, K
// with 16-byte-aligned row strides is accepted.
//
// Every mbarrier wait is bounded (about a second); a wait that gives up records an error
// in the context's device flag word, raises a CTA-wide abort flag that makes all later
// waits return at once, and the kernel still runs to its end, frees its TMEM and exits.
#include <cstring>

#include "md_internal.cuh"
#include "tc_common.cuh"

namespace {

constexpr int BLOCK_M = 128, BLOCK_K = 64, UMMA_K = 16;
constexpr int A_STAGE_BYTES = BLOCK_M * BLOCK_K * 2;     // 16 KiB
constexpr int EPI_WARPS = 8, EPI_BUF_BYTES = 32 * 128;   // 32 rows x 64 f16 per epilogue warp
constexpr int EPI_BYTES = EPI_WARPS * EPI_BUF_BYTES;     // 32 KiB
constexpr int NUM_THREADS = (2 + EPI_WARPS) * 32;
constexpr int PUSH_WARPS = 8;                            // extra warps of the column-split form
constexpr int NUM_THREADS_PUSH = NUM_THREADS + PUSH_WARPS * 32;
constexpr int RASTER_GROUP_M = 8;                        // tile rows per rasterisation group
constexpr int SMEM_LIMIT = 232448;                       // 227 KiB opt-in maximum
constexpr int BAR_BYTES = 1024;

// mt = number of 128-row sub-tiles of A per CTA tile (1 or 2): with 2 the tile is 256 x 256, both sub-tiles
// share one B tile, and a k-block costs 64 KB for 1024 cycles of tensor time instead of 48 KB for 512.
__host__ __device__ constexpr int stage_bytes(int block_n, int mt) { return mt * A_STAGE_BYTES + block_n * BLOCK_K * 2; }
__host__ __device__ constexpr int num_stages(int block_n, int mt) {
    int s = (SMEM_LIMIT - 1024 /*alignment slack*/ - EPI_BYTES - BAR_BYTES) / stage_bytes(block_n, mt);
    return s > 10 ? 10 : s;
}
__host__ __device__ constexpr int smem_bytes(int block_n, int mt) {
    return 1024 + num_stages(block_n, mt) * stage_bytes(block_n, mt) + EPI_BYTES + BAR_BYTES;
}

using namespace tc;

// Linear tile index -> (tile row, tile column): groups of RASTER_GROUP_M tile rows, row index fastest inside a group.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int per_group = RASTER_GROUP_M * tiles_n;
    const int g = tile / per_group, r = tile - g * per_group;
    const int m_first = g * RASTER_GROUP_M;
    const int rows = min(RASTER_GROUP_M, tiles_m - m_first);
    tm = m_first + r % rows;
    tn = r / rows;
}

// Barrier of the eight epilogue warps (id 1; 0 is __syncthreads).
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory"); }

// PUSH = the column-split form with its eight extra warps (its own instantiation, so that the plain kernel keeps the
// register budget of 320 threads)
// SPLITK = the form that may split K over several CTAs per tile (its own instantiation: the others compile with one
// range per tile and carry none of its code).
template <int BLOCK_N, bool B_MN_MAJOR, int MT, bool PUSH, bool SPLITK>
__global__ void __launch_bounds__(PUSH ? NUM_THREADS_PUSH : NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
               const __grid_constant__ CUtensorMap tm_c, int M, int N, int K, int tiles_m, int num_tiles,
               md_epilogue ep, md_push push, md_devflags* flags, int splits_arg, float* part, unsigned* tickets,
               const __grid_constant__ md_peer_maps pm) {
    const int splits = SPLITK ? splits_arg : 1;
    // splits > 1 (MT == 1, no peers): a work unit is one of `splits` ranges of k-blocks of a tile.  Every unit leaves
    // its f32 accumulators in `part` ([unit][column][row]); the unit that arrives last at the tile's ticket adds the
    // ranges up in their order and runs the epilogue.  For products with fewer tiles than SMs and a long K.
    constexpr int STAGES = num_stages(BLOCK_N, MT);
    constexpr int A_TILE_BYTES = MT * A_STAGE_BYTES;   // MT sub-tiles of 128 rows, one after the other
    constexpr int B_STAGE_BYTES = BLOCK_N * BLOCK_K * 2;
    constexpr int STAGE_BYTES = A_TILE_BYTES + B_STAGE_BYTES;
    // accumulators: MT == 1: two buffers of BLOCK_N columns (the epilogue of tile i overlaps the main loop of
    // tile i+1); MT == 2: the two sub-tiles fill all 512 columns, one buffer
    constexpr int NBUF = MT == 1 ? 2 : 1;
    constexpr uint32_t TMEM_COLS = 2 * BLOCK_N;  // 128, 256 or 512: a power of two >= 32
    constexpr int TILE_M = MT * BLOCK_M, CHUNKS_N = BLOCK_N / 64, CHUNKS = MT * CHUNKS_N;
    static_assert(BLOCK_N == 64 || BLOCK_N == 128 || BLOCK_N == 256, "BLOCK_N");
    static_assert(MT == 1 || (MT == 2 && BLOCK_N == 256), "two sub-tiles only with 256-wide tiles");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t smem_a = base;
    const uint32_t smem_b = base + STAGES * A_TILE_BYTES;
    const uint32_t smem_epi = base + STAGES * STAGE_BYTES;
    uint8_t* epi_ptr = base_ptr + STAGES * STAGE_BYTES;
    const uint32_t bars = smem_epi + EPI_BYTES;
    uint8_t* bars_ptr = epi_ptr + EPI_BYTES;
    // barrier block: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], then tmem address, abort flag
    const uint32_t bar_full = bars, bar_empty = bars + 8 * STAGES;
    const uint32_t bar_tfull = bars + 16 * STAGES, bar_tempty = bar_tfull + 16;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars_ptr + 16 * STAGES + 32);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_ptr + 16 * STAGES + 36);
    // per epilogue warp: the number of this CTA's tiles it has finished (all of its TMA stores complete)
    volatile unsigned* stored = reinterpret_cast<volatile unsigned*>(bars_ptr + 16 * STAGES + 40);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (K + BLOCK_K - 1) / BLOCK_K;
    const int tiles_n = num_tiles / tiles_m;
    const int num_units = num_tiles * splits, kb_per = (num_kb + splits - 1) / splits;
    volatile int* last_flag = reinterpret_cast<volatile int*>(bars_ptr + 16 * STAGES + 40 + 4 * EPI_WARPS);

    // programmatic dependent launch: the successor may start its own set-up now; this kernel sets up its
    // barriers and tensor memory, then waits for its predecessor before any global access
    md_pdl_launch_dependents();
    if (threadIdx.x == 0) {
        // the descriptors are kernel parameters: fetching them does not depend on the predecessor kernel
        tma_prefetch_map(&tm_a);
        tma_prefetch_map(&tm_b);
        tma_prefetch_map(&tm_c);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_tfull + 8 * b, 1);
            mbar_init(bar_tempty + 8 * b, EPI_WARPS);
        }
        *abort_flag = 0;
        for (int e = 0; e < EPI_WARPS; ++e) stored[e] = 0u;
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
    md_pdl_wait();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int unit = blockIdx.x; unit < num_units; unit += gridDim.x) {
                const int tile = unit / splits, kb0 = (unit - tile * splits) * kb_per, kb1 = min(num_kb, kb0 + kb_per);
                int tm, tn;
                tile_coords(tile, tiles_m, tiles_n, tm, tn);
                const int m0 = tm * TILE_M, n0 = tn * BLOCK_N;
                for (int kb = kb0; kb < kb1; ++kb) {
                    mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, flags, 1);
                    const uint32_t full = bar_full + 8 * stage;
                    mbar_expect_tx(full, STAGE_BYTES);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
                        tma_load_2d(smem_a + stage * A_TILE_BYTES + mt * A_STAGE_BYTES, &tm_a, full, kb * BLOCK_K,
                                    m0 + mt * BLOCK_M);
                    if (B_MN_MAJOR) {
#pragma unroll
                        for (int j = 0; j < BLOCK_N / 64; ++j)
                            tma_load_2d(smem_b + stage * B_STAGE_BYTES + j * (64 * BLOCK_K * 2), &tm_b, full,
                                        n0 + j * 64, kb * BLOCK_K);
                    } else {
                        tma_load_2d(smem_b + stage * B_STAGE_BYTES, &tm_b, full, kb * BLOCK_K, n0);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            // After an abort loads may still be in flight towards this CTA's shared memory:
            // give them time to land before the CTA exits (they complete within microseconds).
            if (*abort_flag) {
                const unsigned long long t0 = global_ns();
                while (global_ns() - t0 < 500000ull) {}
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | ((B_MN_MAJOR ? 1u : 0u) << 16) | ((uint32_t)(BLOCK_N >> 3) << 17) |
                                   ((uint32_t)(BLOCK_M >> 4) << 24);
            // descriptors as 32-bit halves: constant high words, low words advanced by adds (tc_common.cuh)
            // K-major operand: 16 k = 32 B further along the swizzled row; MN-major B: 16 k-rows = 2048 B
            constexpr uint32_t A_KSTEP = (UMMA_K * 2) >> 4, B_KSTEP = (B_MN_MAJOR ? UMMA_K * 128 : UMMA_K * 2) >> 4;
            const uint32_t a_hi = desc_hi(1024, 2), b_hi = desc_hi(1024, 2);
            const uint32_t a_lo0 = desc_lo(smem_a, 16), b_lo0 = desc_lo(smem_b, B_MN_MAJOR ? 64 * BLOCK_K * 2 : 16);
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            for (int unit = blockIdx.x; unit < num_units; unit += gridDim.x, ++local) {
                const int kb0 = (unit % splits) * kb_per, kb1 = min(num_kb, kb0 + kb_per);
                const int buf = local % NBUF;
                const uint32_t acc_phase = (uint32_t)(local / NBUF) & 1u;
                mbar_wait(bar_tempty + 8 * buf, acc_phase ^ 1u, abort_flag, flags, 2);
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BLOCK_N);
                for (int kb = kb0; kb < kb1; ++kb) {
                    mbar_wait(bar_full + 8 * stage, phase, abort_flag, flags, 3);
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + (uint32_t)stage * (A_TILE_BYTES >> 4);
                    const uint32_t b_lo = b_lo0 + (uint32_t)stage * (B_STAGE_BYTES >> 4);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        // sub-tile mt: rows mt*128.. of the A tile, accumulator columns mt*256..
                        const uint32_t d = tmem_d + (uint32_t)(mt * 256), am = a_lo + (uint32_t)(mt * (A_STAGE_BYTES >> 4));
                        if (kb == kb0) tc_mma_f16_parts<false>(d, am, a_hi, b_lo, b_hi, idesc);
                        else tc_mma_f16_parts<true>(d, am, a_hi, b_lo, b_hi, idesc);
                    }
#pragma unroll
                    for (int k = 1; k < BLOCK_K / UMMA_K; ++k) {
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt)
                            tc_mma_f16_parts<true>(tmem_d + (uint32_t)(mt * 256),
                                                   a_lo + (uint32_t)(mt * (A_STAGE_BYTES >> 4)) + k * A_KSTEP, a_hi,
                                                   b_lo + k * B_KSTEP, b_hi, idesc);
                    }
                    tc_commit(bar_empty + 8 * stage);  // frees the smem stage once these MMAs retire
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                tc_commit(bar_tfull + 8 * buf);  // accumulator complete
            }
        }
    } else if (warp < 2 + EPI_WARPS) {
        // ------------------------------------------------------------ epilogue (warps 2..9)
        // Two warps per TMEM lane quadrant; they take alternate 64-column chunks of the tile.
        const int quad = warp & 3;  // TMEM lane quadrant this warp may read
        const int half = (warp - 2) >> 2;
        const uint32_t my_epi = smem_epi + (uint32_t)(warp - 2) * EPI_BUF_BYTES;
        uint8_t* my_epi_ptr = epi_ptr + (warp - 2) * EPI_BUF_BYTES;
        const bool any_glue = ep.bias || ep.residual || ep.residual2 || ep.gelu;
        int local = 0;
        for (int unit = blockIdx.x; unit < num_units; unit += gridDim.x, ++local) {
            const int tile = unit / splits;
            int tm, tn;
            tile_coords(tile, tiles_m, tiles_n, tm, tn);
            const int m0 = tm * TILE_M, n0 = tn * BLOCK_N;
            const int buf = local % NBUF;
            const uint32_t acc_phase = (uint32_t)(local / NBUF) & 1u;
            mbar_wait(bar_tfull + 8 * buf, acc_phase, abort_flag, flags, 4);
            tc_fence_after();
            const bool from_part = SPLITK && splits > 1;
            if (from_part) {
                // this unit's accumulators to global memory, [column][row] so that a warp's 32 rows are neighbours
                float* mine = part + (size_t)unit * (BLOCK_M * BLOCK_N) + quad * 32 + lane;
                const uint32_t t_acc = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BLOCK_N);
#pragma unroll 1
                for (int c = half; c < CHUNKS_N; c += 2) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint32_t r[32];
                        tc_ld_32x32(t_acc + (uint32_t)(c * 64 + h * 32), r);
                        tc_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; ++e) mine[(size_t)(c * 64 + h * 32 + e) * BLOCK_M] = __uint_as_float(r[e]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
                __threadfence();
                epi_sync();
                if (threadIdx.x == 64) {
                    const unsigned t = atomicAdd(tickets + tile, 1u);
                    const int last = t == (unsigned)(splits - 1);
                    if (last) tickets[tile] = 0u;   // zero again for the next launch
                    *last_flag = last;
                }
                epi_sync();
                if (!*last_flag) continue;   // another unit of this tile finishes it
                __threadfence();
            }
            const float* parts = part + (size_t)tile * splits * (BLOCK_M * BLOCK_N) + quad * 32 + lane;
#pragma unroll 1
            for (int cc = half; cc < CHUNKS; cc += 2) {
                // chunk cc = 64 columns c of sub-tile mt
                const int mt = cc / CHUNKS_N, c = cc % CHUNKS_N;
                const int mrow0 = m0 + mt * BLOCK_M + quad * 32, row = mrow0 + lane;
                const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BLOCK_N + mt * 256);
                // the staging buffer must have been read by this warp's previous TMA store
                if (lane == 0) tma_store_wait_read<0>();
                __syncwarp();
                uint8_t* out_row = my_epi_ptr + lane * 128;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t r[32];
                    if (from_part) {
                        // the k ranges added up in their order, whichever unit got here last; a range's 32 loads are
                        // independent of one another and all in flight before the first add
                        const float* src = parts + (size_t)(c * 64 + h * 32) * BLOCK_M;
                        float acc[32];
#pragma unroll
                        for (int e = 0; e < 32; ++e) acc[e] = __ldcg(src + e * BLOCK_M);
                        for (int sp = 1; sp < splits; ++sp) {
                            src += BLOCK_M * BLOCK_N;
                            float nxt[32];
#pragma unroll
                            for (int e = 0; e < 32; ++e) nxt[e] = __ldcg(src + e * BLOCK_M);
#pragma unroll
                            for (int e = 0; e < 32; ++e) acc[e] += nxt[e];
                        }
#pragma unroll
                        for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(acc[e]);
                    } else {
                        tc_ld_32x32(t_row + (uint32_t)(c * 64 + h * 32), r);
                        tc_wait_ld();
                    }
                    const int col0 = n0 + c * 64 + h * 32;
                    // Glue per group of 8 columns (N % 8 == 0, so a group is entirely inside or outside
                    // the matrix): bias, residual and residual2 arrive as single 16-byte loads.
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int cq = col0 + 8 * q;
                        uint32_t pk[4];
                        epilogue_glue8(r + 8 * q, ep, row, cq, N, any_glue && row < M && cq < N, pk);
                        const int chunk = (h * 4 + q) ^ (lane & 7);  // 128-byte swizzle, matches the store map
                        *reinterpret_cast<uint4*>(out_row + chunk * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
                if (cc + 2 >= CHUNKS && !from_part) {
                    // all of this warp's TMEM reads of the tile are done: hand the buffer back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(&tm_c, my_epi, n0 + c * 64, mrow0);
                    if (PUSH && push.tma) {
                        // the same staged chunk into every peer's C, starting with a different peer in every CTA;
                        // the staging buffer is reused once all of these stores have read it
                        for (int pi = 0; pi < push.n; ++pi) {
                            int peer = pi + (int)blockIdx.x;
                            peer -= (peer / push.n) * push.n;
                            tma_store_2d(&pm.m[peer], my_epi, n0 + c * 64, mrow0);
                        }
                    }
                    tma_store_commit();
                }
            }
            if (half >= CHUNKS && !from_part) {
                // a warp without a chunk (tile narrower than its share) still releases the accumulator
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
            }
            if (PUSH && !push.tma && lane == 0) {
                // Column-split GEMM: this warp's part of the tile is in this GPU's C once its TMA stores have
                // completed; tell the push warps (every epilogue warp counts its own tiles).  The wait costs
                // nothing: the warp would next wait for the following tile's accumulator anyway.
                tma_store_wait_all();
                __threadfence_block();
                stored[warp - 2] = (unsigned)(local + 1);
            }
        }
        if (lane == 0) tma_store_wait_all();
    } else if (PUSH) {
        // ------------------------------------------------------------ push (warps 10..17, column-split GEMM)
        // A warp instruction covers 32 / (BLOCK_N / 8) whole tile rows (BLOCK_N * 2 contiguous bytes each); four
        // row groups are loaded before their peer stores are issued, peers interleaved.
        // While the main loop runs, the SM's return path from L2 is full of operand tiles and a load round trip of a
        // push warp takes several microseconds: eight warps request 8 row groups each at once, so that a 128-row
        // tile is two rounds (with four warps and four groups in flight the pushes fell behind the math: 317 us at
        // four GPUs against 200 us for the product alone).
        constexpr int LANES_PER_ROW = BLOCK_N / 8, ROWS_PER_INSTR = 32 / LANES_PER_ROW, UNR = 8;
        constexpr int ROW_STEP = PUSH_WARPS * ROWS_PER_INSTR;
        const int pw = warp - (2 + EPI_WARPS);
        const int sub = lane / LANES_PER_ROW, cl = (lane % LANES_PER_ROW) * 8;
        const int ld = (int)push.ld;
        int local = 0;
        for (int tile = blockIdx.x; tile < num_tiles && !push.tma; tile += gridDim.x, ++local) {
            int tm, tn;
            tile_coords(tile, tiles_m, tiles_n, tm, tn);
            const int m0 = tm * TILE_M, n0 = tn * BLOCK_N;
            if (!wait_stored(stored, EPI_WARPS, (unsigned)(local + 1), abort_flag, flags, 5)) break;
            const int gc = n0 + cl;
            if (gc >= N) continue;  // columns past this rank's block belong to a neighbour
            const long long tile_off = (long long)m0 * push.ld + gc;
            for (int r = pw * ROWS_PER_INSTR + sub; r < TILE_M; r += ROW_STEP * UNR) {
                uint4 val[UNR];
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    const int rr = r + u * ROW_STEP;
                    if (rr < TILE_M && m0 + rr < M) val[u] = __ldcg(reinterpret_cast<const uint4*>(push.self + tile_off + rr * ld));
                }
                for (int pi = 0; pi < push.n; ++pi) {
                    // start with a different peer in every CTA so that the stores spread over the links
                    int peer = pi + (int)blockIdx.x;
                    peer -= (peer / push.n) * push.n;
                    __half* dst = push.base[peer] + tile_off;
#pragma unroll
                    for (int u = 0; u < UNR; ++u) {
                        const int rr = r + u * ROW_STEP;
                        if (rr < TILE_M && m0 + rr < M) *reinterpret_cast<uint4*>(dst + rr * ld) = val[u];
                    }
                }
            }
        }
        __threadfence_system();  // peer stores performed before the kernel ends
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                     : "memory");
    }
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int resolve_encode_tiled(md_ctx* ctx) {
    if (!ctx->encode_tiled) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn)
            return md_fail(ctx, MD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        ctx->encode_tiled = fn;
    }
    return MD_OK;
}

int make_map_2d(md_ctx* ctx, CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint32_t box_inner,
                uint32_t box_outer, uint64_t ld = 0) {
    MD_TRY(resolve_encode_tiled(ctx));
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {(ld ? ld : inner) * 2};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = reinterpret_cast<encode_tiled_fn>(ctx->encode_tiled)(
        map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return md_fail(ctx, MD_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return MD_OK;
}

template <int BLOCK_N, bool B_MN_MAJOR, int MT, bool PUSH>
int launch_as(md_ctx* ctx, const __half* a, const __half* b, __half* c, size_t M, size_t N, size_t K,
           const md_epilogue& ep, size_t ldc, const md_push& push, int splits = 1) {
    CUtensorMap tm_a, tm_b, tm_c;
    MD_TRY(make_map_2d(ctx, &tm_a, a, K, M, BLOCK_K, BLOCK_M));
    if (B_MN_MAJOR) MD_TRY(make_map_2d(ctx, &tm_b, b, N, K, 64, BLOCK_K));
    else MD_TRY(make_map_2d(ctx, &tm_b, b, K, N, BLOCK_K, BLOCK_N));
    MD_TRY(make_map_2d(ctx, &tm_c, c, N, M, 64, 32, ldc));
    const int tiles_m = (int)((M + MT * BLOCK_M - 1) / (MT * BLOCK_M)), tiles_n = (int)((N + BLOCK_N - 1) / BLOCK_N);
    const int num_tiles = tiles_m * tiles_n;
    float* part = nullptr;
    unsigned* tickets = nullptr;
    if constexpr (MT != 1 || PUSH || BLOCK_N != 256) {
        if (splits > 1)
            return md_fail(ctx, MD_ERR_UNSUPPORTED,
                           "tcgen05 GEMM: K is split only for single 128 x 256 tiles without peers");
    } else if (splits > 1) {
        if (num_tiles > (int)MD_SPLITK_TICKETS)
            return md_fail(ctx, MD_ERR_UNSUPPORTED, "tcgen05 GEMM: too many tiles for a split K");
        MD_TRY(md_splitk_workspace(ctx, (size_t)num_tiles * splits * BLOCK_M * BLOCK_N * sizeof(float), &part, &tickets));
    }
    md_peer_maps pm;
    memset(&pm, 0, sizeof(pm));
    if (PUSH && push.tma)
        for (int i = 0; i < push.n; ++i) MD_TRY(make_map_2d(ctx, &pm.m[i], push.base[i], N, M, 64, 32, ldc));
    const int units = num_tiles * splits;
    const int grid = units < ctx->sm_count ? units : ctx->sm_count;
    // the split-K instantiation exists for single 128-row tiles of 256 columns without peers only
    constexpr bool CAN_SPLIT = MT == 1 && !PUSH && BLOCK_N == 256;
    auto kern = (CAN_SPLIT && splits > 1) ? gemm_tc_kernel<BLOCK_N, B_MN_MAJOR, MT, PUSH, CAN_SPLIT>
                                          : gemm_tc_kernel<BLOCK_N, B_MN_MAJOR, MT, PUSH, false>;
    constexpr int smem = smem_bytes(BLOCK_N, MT);
    const uint32_t cfg_bit = (CAN_SPLIT && splits > 1)
                                 ? 1u << (B_MN_MAJOR ? 7 : 6)
                                 : (MT == 2 ? (1u << (B_MN_MAJOR ? 12 : 11))
                                            : 1u << ((BLOCK_N == 256 ? 0 : BLOCK_N == 128 ? 1 : 2) + (B_MN_MAJOR ? 3 : 0)))
                                       << (PUSH ? 16 : 0);
    if (!(ctx->tc_configured & cfg_bit)) {
        MD_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        ctx->tc_configured |= cfg_bit;
    }
    ctx->last_tc_tile = (MT == 2 ? 512 : BLOCK_N) + (splits > 1 ? 10000 * splits : 0);   // 30256 = 128 x 256 tiles, K in 3
    return md_launch_ex(ctx, kern, dim3((unsigned)grid), dim3(PUSH ? NUM_THREADS_PUSH : NUM_THREADS), smem,
                        "gemm_tc_kernel", tm_a, tm_b, tm_c, (int)M, (int)N, (int)K, tiles_m, num_tiles, ep, push, ctx->flags,
                        splits, part, tickets, pm);
}

template <int BLOCK_N, bool B_MN_MAJOR, int MT = 1>
int launch(md_ctx* ctx, const __half* a, const __half* b, __half* c, size_t M, size_t N, size_t K,
           const md_epilogue& ep, size_t ldc, const md_push& push, int splits = 1) {
    if (push.n > 0) return launch_as<BLOCK_N, B_MN_MAJOR, MT, true>(ctx, a, b, c, M, N, K, ep, ldc, push);
    return launch_as<BLOCK_N, B_MN_MAJOR, MT, false>(ctx, a, b, c, M, N, K, ep, ldc, push, splits);
}

}  // namespace

bool md_gemm_tc_supported(const void* a, const void* b, const void* c, size_t M, size_t N, size_t K, int b_layout) {
    (void)b_layout;
    if (M == 0 || N == 0 || K == 0) return false;
    if ((K % 8) != 0 || (N % 8) != 0) return false;  // row strides must be multiples of 16 bytes
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15)
        return false;
    if (M > (1u << 30) || N > (1u << 30) || K > (1u << 30)) return false;
    return true;
}

int md_launch_gemm_tc(md_ctx* ctx, const __half* a, const __half* b, __half* c, size_t M, size_t N, size_t K,
                      int b_layout, const md_epilogue& ep) {
    md_push none;
    return md_launch_gemm_tc_ex(ctx, a, b, c, M, N, K, b_layout, ep, N, none);
}

int md_launch_gemm_tc_ex(md_ctx* ctx, const __half* a, const __half* b, __half* c, size_t M, size_t N, size_t K,
                         int b_layout, const md_epilogue& ep, size_t ldc, const md_push& push) {
    if ((ldc % 8) != 0 || ldc < N)
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "tcgen05 GEMM: the output row stride must be a multiple of 8 and >= N");
    if (ldc != N && (ep.residual || ep.residual2))
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "tcgen05 GEMM: residuals are not supported with a strided output");
    if (!md_gemm_tc_supported(a, b, c, M, N, K, b_layout))
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "tcgen05 GEMM needs K %% 8 == 0, N %% 8 == 0 and 16-byte aligned operands");
    // Tile shape.  The kernel is bound by the bytes an SM pulls from L2 per k-block, (rows + columns) x 128,
    // so a tile's time is proportional to its rows + columns: 128 x 64, 128 x 128, 128 x 256, or 256 x 256 (two
    // 128-row sub-tiles sharing one B tile).  Cost = (waves over the SMs) x (rows + columns).  Skinny problems
    // (M <= 64) are HBM-bound and take the narrowest tile to get many CTAs streaming B.
    int bn = 64, mt = 1;
    if (M > 64) {
        const int cand_n[4] = {256, 256, 128, 64}, cand_mt[4] = {2, 1, 1, 1};
        double best = -1.0;
        for (int i = 0; i < 4; ++i) {
            const size_t rows = (size_t)cand_mt[i] * BLOCK_M;
            const size_t t = ((M + rows - 1) / rows) * ((N + cand_n[i] - 1) / cand_n[i]);
            const size_t waves = (t + ctx->sm_count - 1) / ctx->sm_count;
            // per tile: (rows + columns) per k-block; measured, the 256 x 256 tile moves ~42 B per cycle against
            // ~55 for the 128-row tiles (three ring stages), hence the factor 1.3, and its epilogue is not hidden
            // behind the next tile's main loop (one accumulator buffer): a fixed cost per tile, larger with glue
            const double kblocks = (double)((K + BLOCK_K - 1) / BLOCK_K);
            const bool glue = ep.bias || ep.gelu || ep.residual || ep.residual2;
            const double tile = (double)(rows + cand_n[i]) * kblocks * (cand_mt[i] == 2 ? 1.3 : 1.0) +
                                (cand_mt[i] == 2 ? (glue ? 7000.0 : 2500.0) : 0.0);
            double cost = (double)waves * tile;
            if (push.n > 0) {
                // Column-split GEMM: the block also has to cross NVLink to every peer (~770 GB/s per direction: in
                // the units of `tile`, 128 bytes pulled from L2 = ~2.5 cycles, about 1000 bytes of link time).  The
                // pushes can start when the first tile is done, and the last wave's tiles are pushed after the math.
                const double per_byte = 1.0 / 1000.0;
                const double total_push = (double)M * (double)N * 2.0 * push.n * per_byte;
                const size_t last_wave = t - (waves - 1) * (size_t)ctx->sm_count;
                const double tail_push = (double)last_wave * (double)(rows * cand_n[i]) * 2.0 * push.n * per_byte;
                const double through = tile + total_push;
                cost = cost + tail_push > through ? cost + tail_push : through;
            }
            if (best < 0.0 || cost < best) { best = cost; bn = cand_n[i]; mt = cand_mt[i]; }
        }
    }
    // Column-split products with rows for both CTAs of a pair and at least one 256-wide tile take the pair kernel
    // whatever the search above found: measured at 8 GPUs (8192 x 1024 x 8192 per rank, seven peers) 265 us on pairs
    // against 289-292 us on 128 x 128, 128 x 256 or 256 x 256 single-CTA tiles; at 2 and 4 GPUs the search picks the
    // 128 x 256 tile, and with it the pairs, by itself.
    if (push.n > 0 && M > 256 && N >= 256 && !ctx->tc_block_n && ctx->tc_pair < 0) { bn = 256; mt = 1; }
    // Split K (md_set_option("tc_splitk"), off by default: inside the forked prefill layer the other chain's kernels
    // already use the SMs such a product leaves idle, and the whole prefill measured 3.13 ms without against 3.27 ms
    // with it).  With fewer 128 x 256 tiles than SMs and a long K (the 2048-wide outputs of a 761-row prefill, the
    // 1152-wide ones of a one-crop ViT layer) most of the machine would idle through a long main loop.  S CTAs per
    // tile take a range of k-blocks each; the f32 partial tiles meet in global memory, which measured about 10 us
    // per launch whatever the shape (7600 units of the cost above: the partials out, fence and ticket, S partial tiles
    // back in through the one SM that finishes the tile).  So it pays for the 2048 x 8192 product of a 761-row
    // prefill (42.6 -> 33.4 us in three ranges) and not for its 2048 x 2048 one (15.3 -> 20.6 us) or the one-crop
    // ViT shapes.  At least 8 k-blocks per range.
    int splits = 1;
    if (M > 64 && push.n == 0 && !ctx->tc_block_n && ctx->tc_splitk != 0) {
        const size_t t256 = ((M + BLOCK_M - 1) / BLOCK_M) * ((N + 255) / 256);
        const int kblocks = (int)((K + BLOCK_K - 1) / BLOCK_K);
        int s_max = t256 ? (int)((size_t)ctx->sm_count / t256) : 1;
        if (s_max > 4) s_max = 4;
        if (ctx->tc_splitk >= 2) s_max = ctx->tc_splitk;
        while (s_max > 1 && (kblocks / s_max < 8 || (s_max - 1) * ((kblocks + s_max - 1) / s_max) >= kblocks)) --s_max;
        if (s_max >= 2 && t256 <= MD_SPLITK_TICKETS) {
            const double rows = BLOCK_M, per = (double)((kblocks + s_max - 1) / s_max);
            const size_t waves = (t256 * s_max + ctx->sm_count - 1) / ctx->sm_count;
            const double cost = (double)waves * ((rows + 256.0) * per + 7600.0);
            // the unsplit choice above, recomputed (best is local to the loop): rows + columns per k-block and wave
            const size_t rows_b = (size_t)mt * BLOCK_M;
            const size_t t_b = ((M + rows_b - 1) / rows_b) * ((N + bn - 1) / bn);
            const size_t waves_b = (t_b + ctx->sm_count - 1) / ctx->sm_count;
            const double cost_b = (double)waves_b * (double)(rows_b + bn) * kblocks * (mt == 2 ? 1.3 : 1.0);
            if (ctx->tc_splitk >= 2 || cost < cost_b) { splits = s_max; bn = 256; mt = 1; }
        }
    }
    if (splits > 1) {
        if (b_layout == 0) return launch<256, true>(ctx, a, b, c, M, N, K, ep, ldc, push, splits);
        return launch<256, false>(ctx, a, b, c, M, N, K, ep, ldc, push, splits);
    }
    // CTA pairs (gemm_pair.cu): where the single-CTA choice is the 128 x 256 tile and there are rows for both CTAs of
    // a pair, the pair's 256 x 256 tile does the same work per SM with a third less traffic from L2 and measured
    // 1 to 12 % faster (761 x 8192 x 2048: 34.8 -> 31.2 us; 9477 x 1152 x 4304: 91.1 -> 84.7 us); with the other
    // choices it lost.  md_set_option("tc_pair"): 1 = always, 0 = never.
    if (!ctx->tc_block_n &&
        (ctx->tc_pair == 1 || (ctx->tc_pair < 0 && bn == 256 && mt == 1 && M > 256)))
        return md_launch_gemm_pair(ctx, a, b, c, M, N, K, b_layout, ep, ldc, push);
    if (ctx->tc_block_n) {  // forced: 512 = the 256 x 256 tile
        bn = ctx->tc_block_n == 512 ? 256 : ctx->tc_block_n;
        mt = ctx->tc_block_n == 512 ? 2 : 1;
    }
    const bool mn = (b_layout == 0);
    if (mn) {
        if (mt == 2) return launch<256, true, 2>(ctx, a, b, c, M, N, K, ep, ldc, push);
        if (bn == 256) return launch<256, true>(ctx, a, b, c, M, N, K, ep, ldc, push);
        if (bn == 128) return launch<128, true>(ctx, a, b, c, M, N, K, ep, ldc, push);
        return launch<64, true>(ctx, a, b, c, M, N, K, ep, ldc, push);
    }
    if (mt == 2) return launch<256, false, 2>(ctx, a, b, c, M, N, K, ep, ldc, push);
    if (bn == 256) return launch<256, false>(ctx, a, b, c, M, N, K, ep, ldc, push);
    if (bn == 128) return launch<128, false>(ctx, a, b, c, M, N, K, ep, ldc, push);
    return launch<64, false>(ctx, a, b, c, M, N, K, ep, ldc, push);
}

// 2-D f16 tensor map with 128-byte swizzle for other translation units (the attention kernel).
int md_make_map_2d(md_ctx* ctx, CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint32_t box_inner,
                   uint32_t box_outer, uint64_t ld) {
    return make_map_2d(ctx, map, ptr, inner, outer, box_inner, box_outer, ld);
}

// 4-D f16 tensor map (dim 0 contiguous), 128- or 32-byte swizzle, zero fill outside the extents; the box is
// box0 x box_d[0..2] elements.  strides_bytes[i] is the stride of dim i+1.
int md_make_map_4d(md_ctx* ctx, CUtensorMap* map, const void* ptr, const uint64_t dims[4], const uint64_t strides_bytes[3],
                   uint32_t box0, const uint32_t box_d[3], int swizzle_bytes) {
    MD_TRY(resolve_encode_tiled(ctx));
    const cuuint64_t gd[4] = {dims[0], dims[1], dims[2], dims[3]};
    const cuuint64_t gs[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
    const cuuint32_t box[4] = {box0, box_d[0], box_d[1], box_d[2]};
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    CUresult r = reinterpret_cast<encode_tiled_fn>(ctx->encode_tiled)(
        map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(ptr), gd, gs, box, elem,
        CU_TENSOR_MAP_INTERLEAVE_NONE,
        swizzle_bytes == 0 ? CU_TENSOR_MAP_SWIZZLE_NONE : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_128B,
        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return md_fail(ctx, MD_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled (4-D) failed with CUresult %d", (int)r);
    return MD_OK;
}

// ---------------------------------------------------------------------------- failure-path self-test
namespace {
// One thread waits on an mbarrier that expects an arrival nobody makes, through the same bounded wait as the
// kernels above, with a short budget; it gives up, records site 99 and the kernel ends normally.
__global__ void selftest_wait_kernel(md_devflags* flags, unsigned long long budget_ns) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    const uint32_t b = smem_u32(&bar);
    abort_flag = 0;
    mbar_init(b, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_wait_slow(b, 0, &abort_flag, flags, 99, budget_ns);
}
}  // namespace

int md_launch_selftest_wait(md_ctx* ctx, unsigned limit_ms) {
    selftest_wait_kernel<<<1, 1, 0, ctx->stream>>>(ctx->flags, (unsigned long long)limit_ms * 1000000ull);
    MD_LAUNCH_CHECK(ctx, "selftest_wait_kernel");
    return MD_OK;
}
