// Weight-streaming GEMV for the decode path: C[M,N] = A[M,K] . Bt[N,K]^T with M <= 8.
//
// Replaces the M == 1 vector path of hgemm_trans.zig:55-134,430-455 and, for
// M in 2..8, the scalar remainder-row loop the reference falls into
// (hgemm_trans.zig:348-356).  HBM-bound: every weight byte is read exactly once
// (N*K*2 bytes); the M activation rows (M*K*2 bytes) stay in L1/L2.
//
// Mapping.  A CTA owns 16 consecutive weight rows; its WARPS warps split K.
// Each lane streams 16-byte pieces (8 halves) of two weight rows with
// ld.global.nc, so the 4 lanes of a quad cover 64 contiguous bytes of a row and
// a warp instruction covers 16 rows x 64 B.  The multiply-accumulate runs on the
// tensor cores as mma.sync.m16n8k16 with the 16 weight rows as the "M" side and
// the (up to) 8 activation rows as the "N" side: the order of the k index inside
// a dot product is free, so the 8 halves a lane loaded feed two MMAs directly
// (halves 0..3 -> k slots {2t,2t+1,2t+8,2t+9} of the first, 4..7 of the second)
// as long as the activation fragment is loaded with the same permutation, which
// it is by reading the same 16-byte piece of row g of A.  This removes the
// f16->f32 convert and FMA issue pressure of a SIMT GEMV for every M up to 8,
// accumulates in f32, and needs no shuffle reduction: the warps' partial 16x8
// tiles are summed through shared memory.
//
// Split K.  A matrix with few rows (N = 2048: 128 CTAs) cannot keep enough bytes in
// flight to reach the HBM rate, however many loads a lane issues.  Such a launch
// splits K over the S CTAs of a thread-block cluster (grid.y = S): every CTA streams
// K / S of its 16 rows, leaves its 16 x 8 partial sums in shared memory, and after one
// cluster barrier the first CTA of the cluster adds the S partials through distributed
// shared memory (fixed order), applies the glue and stores.  No global scratch.
#include "md_internal.cuh"

namespace {

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Activations may be written by the predecessor kernel while this kernel already runs (programmatic
// dependent launch), so they must not go through the non-coherent path: an L2-cached load that the
// compiler may not move above the dependency wait.
__device__ __forceinline__ uint4 ld_act(const __half* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int ROWS_PER_CTA = 16;

// UNROLL = number of 32-wide k chunks whose loads are issued before any is consumed.
template <int WARPS, int UNROLL>
__global__ void __launch_bounds__(WARPS * 32)
gemv_nt_mma_kernel(const __half* A, const __half* __restrict__ Bt, __half* C, int M, int N,
                   int K, int ldb, md_epilogue ep) {
    __shared__ float partial[WARPS][ROWS_PER_CTA][8];
    __shared__ float cta_sum[ROWS_PER_CTA * 8];   // this CTA's 16 x 8 sums, read by the cluster's first CTA
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * ROWS_PER_CTA;
    // Rows past N are clamped for the loads and dropped at the store.
    const int r_lo = min(row0 + g, N - 1), r_hi = min(row0 + g + 8, N - 1);
    const __half* w_lo = Bt + (size_t)r_lo * ldb + t * 8;   // ldb >= K: the rows may be K-slices of a wider matrix
    const __half* w_hi = Bt + (size_t)r_hi * ldb + t * 8;
    const bool has_x = g < M;
    const __half* x = A + (size_t)(has_x ? g : 0) * K + t * 8;

    // K is split into 32-wide chunks dealt round-robin to the warps, so that at any
    // moment the CTA reads one contiguous span of each of its 16 rows.
    const int all_chunks = K / 32;
    const int splits = gridDim.y, split = blockIdx.y;
    const int per_split = (all_chunks + splits - 1) / splits;
    const int chunks = min(all_chunks, (split + 1) * per_split);   // this CTA's chunks: [split * per_split, chunks)
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int ch = split * per_split + warp;
    // Programmatic dependent launch: let the next kernel of the stream start its own prologue now, and
    // stream this kernel's first weights (which no earlier kernel writes) before waiting for the kernel
    // that produces the activations.  Without the launch attribute both instructions are no-ops.
    asm volatile("griddepcontrol.launch_dependents;");
    bool waited = false;
    for (; ch + (UNROLL - 1) * WARPS < chunks; ch += UNROLL * WARPS) {
        uint4 lo[UNROLL], hi[UNROLL], xv[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = (ch + u * WARPS) * 32;
            lo[u] = ldg_stream(w_lo + k);
            hi[u] = ldg_stream(w_hi + k);
        }
        if (!waited) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            waited = true;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = (ch + u * WARPS) * 32;
            xv[u] = has_x ? ld_act(x + k) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            mma_16816(acc, lo[u].x, hi[u].x, lo[u].y, hi[u].y, xv[u].x, xv[u].y);
            mma_16816(acc, lo[u].z, hi[u].z, lo[u].w, hi[u].w, xv[u].z, xv[u].w);
        }
    }
    if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (; ch < chunks; ch += WARPS) {
        const int k = ch * 32;
        const uint4 lo = ldg_stream(w_lo + k), hi = ldg_stream(w_hi + k);
        const uint4 xv = has_x ? ld_act(x + k) : make_uint4(0, 0, 0, 0);
        mma_16816(acc, lo.x, hi.x, lo.y, hi.y, xv.x, xv.y);
        mma_16816(acc, lo.z, hi.z, lo.w, hi.w, xv.z, xv.w);
    }
    // K tail (K % 32 != 0, still a multiple of 8): 8-half pieces handled by warp 0 with
    // the lanes whose piece exists; missing pieces contribute zeros.
    const int tail0 = all_chunks * 32;
    if (warp == 0 && split == 0 && tail0 < K) {
        const int k = tail0 + t * 8;
        uint4 lo = make_uint4(0, 0, 0, 0), hi = lo, xv = lo;
        if (k < K) {
            lo = ldg_stream(Bt + (size_t)r_lo * ldb + k);
            hi = ldg_stream(Bt + (size_t)r_hi * ldb + k);
            if (has_x) xv = ld_act(A + (size_t)g * K + k);
        }
        mma_16816(acc, lo.x, hi.x, lo.y, hi.y, xv.x, xv.y);
        mma_16816(acc, lo.z, hi.z, lo.w, hi.w, xv.z, xv.w);
    }

    // c0,c1 = (weight row g, activation rows 2t,2t+1); c2,c3 = (weight row g+8, same).
    partial[warp][g][2 * t] = acc[0];
    partial[warp][g][2 * t + 1] = acc[1];
    partial[warp][g + 8][2 * t] = acc[2];
    partial[warp][g + 8][2 * t + 1] = acc[3];
    __syncthreads();
    if (splits == 1) {
        // 16 rows x 8 activation rows = 128 outputs; a CTA of two warps takes two turns
        for (int o = threadIdx.x; o < ROWS_PER_CTA * 8; o += WARPS * 32) {
            const int m = o >> 4, r = o & 15;  // consecutive threads -> consecutive n
            const int n = row0 + r;
            if (m < M && n < N) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) s += partial[w][r][m];
                if (ep.out_f32) ep.out_f32[(size_t)m * N + n] = s;
                else C[(size_t)m * N + n] = __float2half_rn(md_epilogue_value(ep, s, m, n, N));
            }
        }
        return;
    }
    // split K: this CTA's sums go to cta_sum; the cluster's first CTA adds the S of them in the order 0 .. S-1
    for (int o = threadIdx.x; o < ROWS_PER_CTA * 8; o += WARPS * 32) {
        const int m = o >> 4, r = o & 15;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) s += partial[w][r][m];
        cta_sum[o] = s;
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (split == 0) {
        for (int o = threadIdx.x; o < ROWS_PER_CTA * 8; o += WARPS * 32) {
            const int m = o >> 4, r = o & 15;
            const int n = row0 + r;
            if (m < M && n < N) {
                const uint32_t local = (uint32_t)__cvta_generic_to_shared(&cta_sum[o]);
                float s = 0.f;
                for (int c = 0; c < splits; ++c) {
                    uint32_t remote;
                    float v;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(c));
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote));
                    s += v;
                }
                if (ep.out_f32) ep.out_f32[(size_t)m * N + n] = s;
                else C[(size_t)m * N + n] = __float2half_rn(md_epilogue_value(ep, s, m, n, N));
            }
        }
    }
    // nobody leaves while the first CTA may still read its shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

}  // namespace

int md_launch_gemv_nt(md_ctx* ctx, const __half* a, const __half* bt, __half* c, size_t M, size_t N, size_t K,
                      const md_epilogue& ep, size_t ldb) {
    if (ldb == 0) ldb = K;
    if (ldb < K || (ldb % 8) != 0) return md_fail(ctx, MD_ERR_UNSUPPORTED, "gemv_nt: the weight row stride must be >= K and a multiple of 8");
    if (M == 0 || M > 8 || (K % 8) != 0 || K == 0 || N == 0)
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "gemv_nt needs 1 <= M <= 8 and K %% 8 == 0 (M=%zu K=%zu)", M, K);
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(bt)) & 15)
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "gemv_nt needs 16-byte aligned operands");
    const unsigned grid = (unsigned)((N + ROWS_PER_CTA - 1) / ROWS_PER_CTA);
    // (warps, unroll) variants; 0 = automatic choice by K.
    int variant = ctx->gemv_variant;
    if (variant == 0) {
        // Measured on B200 with weights streamed from HBM: many CTAs (vocabulary-sized N) want
        // small CTAs; few CTAs (N <= 2048) or long rows (K >= 4096) want many warps per CTA so
        // that the whole matrix is in flight at once.
        if (N >= 16384) variant = 4;
        else if (K >= 4096 || N <= 2048) variant = 6;
        else variant = 2;
    }
    // With ctx->pdl the launch carries the programmatic-stream-serialization attribute: the kernel may
    // start while its predecessor drains and orders itself with griddepcontrol.wait.  Only valid when
    // the weights are not produced by an earlier kernel of the stream (true for registered weights).
    // K splits (a cluster along y).  Clusters start more slowly than plain CTAs, so a split pays only where a
    // matrix has at most one CTA per SM and rows of K >= 8192 (the 8192 -> 2048 projection: 10.3 -> 8.4 us with two splits;
    // four were slower again, and every shape with more rows lost).  md_set_option("gemv_ksplit") fixes the count.
    int ksplit = ctx->gemv_ksplit;
    if (ksplit <= 0) ksplit = (grid <= (unsigned)ctx->sm_count && K >= 8192) ? 2 : 1;
    while (ksplit > 1 && (size_t)(K / 32) < (size_t)ksplit) ksplit /= 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, (unsigned)ksplit);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (ksplit > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = (unsigned)ksplit;
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
    const int Mi = (int)M, Ni = (int)N, Ki = (int)K, ldbi = (int)ldb;
    cudaError_t le = cudaSuccess;
#define MD_GEMV_CASE(id, W, U)                                                          \
    case id:                                                                            \
        cfg.blockDim = dim3(W * 32);                                                    \
        le = cudaLaunchKernelEx(&cfg, gemv_nt_mma_kernel<W, U>, a, bt, c, Mi, Ni, Ki, ldbi, ep); \
        break;
    switch (variant) {
        MD_GEMV_CASE(1, 4, 8)
        MD_GEMV_CASE(2, 8, 4)
        MD_GEMV_CASE(3, 8, 8)
        MD_GEMV_CASE(4, 4, 4)
        MD_GEMV_CASE(5, 2, 8)
        MD_GEMV_CASE(6, 16, 2)
        default:
            return md_fail(ctx, MD_ERR_INVALID_ARG, "unknown gemv variant %d", variant);
    }
#undef MD_GEMV_CASE
    if (le != cudaSuccess) return md_fail(ctx, MD_ERR_CUDA, "launch of gemv_nt_mma_kernel failed: %s", cudaGetErrorString(le));
    MD_LAUNCH_CHECK(ctx, "gemv_nt_mma_kernel");
    return MD_OK;
}
