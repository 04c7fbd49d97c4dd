// General-shape f16 GEMM on CUDA cores: C[M,N] = A[M,K] . B, B given as [K,N]
// (hgemm.zig:362-426) or [N,K] (hgemm_trans.zig:400-488).
//
// This kernel exists for the shapes the TMA-fed tensor-core kernel cannot take:
// row strides that are not multiples of 16 bytes (K or N not a multiple of 8, as
// in the reference's small test shapes and the 588-wide patch vectors) or
// unaligned base pointers.  Same arithmetic contract as the reference: f16
// operands widened to f32, f32 accumulation, one rounding to f16, then the
// optional fused glue.
#include "md_internal.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <bool B_IS_NK>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const __half* __restrict__ A, const __half* __restrict__ B, __half* __restrict__ C, int M, int N,
                 int K, md_epilogue ep) {
    __shared__ float As[BK][BM + 1];
    __shared__ float Bs[BK][BN + 1];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // A tile: 64 rows x 16 k, thread -> (row = tid/16 + 16*i, k = tid%16)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = tid / 16 + 16 * i, kk = tid % 16;
            const int gm = m0 + r, gk = k0 + kk;
            As[kk][r] = (gm < M && gk < K) ? __half2float(A[(size_t)gm * K + gk]) : 0.f;
        }
        if (B_IS_NK) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int c = tid / 16 + 16 * i, kk = tid % 16;
                const int gn = n0 + c, gk = k0 + kk;
                Bs[kk][c] = (gn < N && gk < K) ? __half2float(B[(size_t)gn * K + gk]) : 0.f;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int kk = tid / 64 + 4 * i, c = tid % 64;
                const int gn = n0 + c, gk = k0 + kk;
                Bs[kk][c] = (gn < N && gk < K) ? __half2float(B[(size_t)gk * N + gn]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx + 16 * j;
            if (gn >= N) continue;
            C[(size_t)gm * N + gn] = __float2half_rn(md_epilogue_value(ep, acc[i][j], gm, gn, N));
        }
    }
}

}  // namespace

int md_launch_gemm_simt(md_ctx* ctx, const __half* a, const __half* b, __half* c, size_t M, size_t N, size_t K,
                        int b_layout, const md_epilogue& ep) {
    if (M == 0 || N == 0) return MD_OK;
    dim3 grid((unsigned)((N + BN - 1) / BN), (unsigned)((M + BM - 1) / BM));
    if (grid.y > 65535) return md_fail(ctx, MD_ERR_UNSUPPORTED, "gemm_simt: M too large (%zu)", M);
    if (b_layout)
        gemm_simt_kernel<true><<<grid, 256, 0, ctx->stream>>>(a, b, c, (int)M, (int)N, (int)K, ep);
    else
        gemm_simt_kernel<false><<<grid, 256, 0, ctx->stream>>>(a, b, c, (int)M, (int)N, (int)K, ep);
    MD_LAUNCH_CHECK(ctx, "gemm_simt_kernel");
    return MD_OK;
}
