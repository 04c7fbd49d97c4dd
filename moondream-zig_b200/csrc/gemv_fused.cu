// Fused GEMV kernels of the decode step (M <= 8 activation rows).
//
// The reference runs one decoder layer for one token as LayerNorm, four GEMVs with their bias /
// GELU passes and two residual adds (text_model.zig:150-172, 182-323): ten tensor-wide passes, each
// of which is a separate kernel launch on a GPU.  At one token per step every one of them is far
// shorter than a launch-to-launch dependency, so the layer is restated as two weight-streaming
// kernels around the attention kernel, with every rounding point of the reference kept:
//
//   gemv_ln_dual_kernel   y = LayerNorm(hidden) (ops.zig:1152-1419, f16-rounded), then
//                         qkv = f16(f16(y Wqkv^T) + bqkv)                 (text_model.zig:193-196)
//                         fc1 = gelu(f16(f16(y Wfc1^T) + bfc1))           (text_model.zig:310-312)
//                         Both matrices consume the same y (the Phi block is parallel), so one grid
//                         streams both; every CTA recomputes the LayerNorm of the M rows (8 KB of L2
//                         reads) instead of waiting for a separate kernel.
//   gemv_dual_k_kernel    a   = f16(f16(attn Wout^T) + bout)              (text_model.zig:296-299)
//                         m   = f16(f16(fc1 Wfc2^T) + bfc2)               (text_model.zig:317-318)
//                         hidden = f16(hidden + f16(a + m))               (text_model.zig:170-171)
//                         One CTA owns 8 output rows and both dot products of those rows.
//
// Both use the tensor-core mapping of gemv.cu (weight rows on the M side of mma.sync.m16n8k16, the
// <= 8 activation rows on the N side).  gemv_dual_k_kernel needs more CTAs than 2048 / 16 to cover the
// SMs, so its A fragment holds the SAME 8 weight rows twice, rows 0-7 from one 32-wide k slab and rows
// 8-15 from the next; two MMAs with the two matching activation slabs then produce the valid halves
// (rows 0-7 of the first, rows 8-15 of the second).  Tensor work doubles, which is free here.
//
// All kernels are written for programmatic dependent launch: weights (never written on the stream)
// are requested before griddepcontrol.wait, activations only after it and never through the
// non-coherent path.
#include "md_internal.cuh"

namespace {

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_act(const __half* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ float ld_act1(const __half* p) {
    unsigned short u;
    asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(u) : "l"(p) : "memory");
    __half_raw r;
    r.x = u;
    return __half2float(__half(r));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---------------------------------------------------------------------------- LN + dual-N GEMV
constexpr int LN_K = 2048;                 // model dim this kernel is specialised for
constexpr int LN_WARPS = 8;                // 256 threads: one 16-byte piece of a row per thread
constexpr int LN_PITCH = LN_K + 32;        // halves; +64 bytes keeps the fragment reads conflict-free
constexpr int LN_CHUNKS = LN_K / 32;       // 64 chunks of 32 k, 8 per warp

struct LnDualParams {
    const __half* hidden;            // [M][2048]
    const __half *ln_w, *ln_b;       // [2048]
    float eps;
    const __half *w1, *b1;           // [n1][2048], [n1]
    __half* out1;                    // [M][n1]
    const __half *w2, *b2;           // [n2][2048], [n2]; GELU applied
    __half* out2;                    // [M][n2]
    int n1, n2, M;
    unsigned long long* amax;        // optional [M]: running argmax keys of out1 (greedy sampling), see below
    int gelu1;                       // GELU on segment 1 as well (fc1 alone as segment 1)
};

// MM = compile-time bound on the number of activation rows (1, 2, 4 or 8): keeps the register
// footprint of the single-stream case small enough for two CTAs per SM.
template <int MM>
__global__ void __launch_bounds__(LN_WARPS * 32)
gemv_ln_dual_kernel(LnDualParams p) {
    __shared__ __align__(16) __half xs[8][LN_PITCH];
    __shared__ float partial[LN_WARPS][16][8];
    __shared__ float red[LN_WARPS][8];
    __shared__ float stat[2][8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * 16;
    const bool seg2 = row0 >= p.n1;
    const int n_seg = seg2 ? p.n2 : p.n1, r0 = seg2 ? row0 - p.n1 : row0;
    const __half* W = seg2 ? p.w2 : p.w1;
    const int r_lo = min(r0 + g, n_seg - 1), r_hi = min(r0 + g + 8, n_seg - 1);
    const __half* w_lo = W + (size_t)r_lo * LN_K + t * 8;
    const __half* w_hi = W + (size_t)r_hi * LN_K + t * 8;

    pdl_launch_dependents();
    // every weight of this CTA is requested before anything else: 16 x 16 bytes per lane
    uint4 lo[LN_CHUNKS / LN_WARPS], hi[LN_CHUNKS / LN_WARPS];
#pragma unroll
    for (int u = 0; u < LN_CHUNKS / LN_WARPS; ++u) {
        const int k = (warp + u * LN_WARPS) * 32;
        lo[u] = ldg_stream(w_lo + k);
        hi[u] = ldg_stream(w_hi + k);
    }
    // LayerNorm parameters are weights too
    const uint4 gw = ldg_stream(p.ln_w + tid * 8), gb = ldg_stream(p.ln_b + tid * 8);
    pdl_wait();

    // ---- LayerNorm of the M rows into shared memory (two-pass f32, one f16 rounding)
    float v[MM][8];
    float s[MM];
#pragma unroll
    for (int m = 0; m < MM; ++m) {
        s[m] = 0.f;
        if (m < p.M) {
            const uint4 u = ld_act(p.hidden + (size_t)m * LN_K + tid * 8);
            const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h[i]);
                v[m][2 * i] = f.x;
                v[m][2 * i + 1] = f.y;
                s[m] += f.x + f.y;
            }
        }
    }
    auto block_sum8 = [&](float (&x)[MM], int slot) {
#pragma unroll
        for (int m = 0; m < MM; ++m) {
#pragma unroll
            for (int o = 16; o; o >>= 1) x[m] += __shfl_xor_sync(0xffffffffu, x[m], o);
        }
        if (lane == 0) {
#pragma unroll
            for (int m = 0; m < MM; ++m) red[warp][m] = x[m];
        }
        __syncthreads();
        if (tid < MM) {
            float a = 0.f;
#pragma unroll
            for (int w = 0; w < LN_WARPS; ++w) a += red[w][tid];
            stat[slot][tid] = a;
        }
        __syncthreads();
    };
    block_sum8(s, 0);
    float q[MM];
#pragma unroll
    for (int m = 0; m < MM; ++m) {
        q[m] = 0.f;
        if (m < p.M) {
            const float mean = stat[0][m] * (1.0f / LN_K);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float d = v[m][i] - mean;
                q[m] += d * d;
            }
        }
    }
    block_sum8(q, 1);
    {
        const __half2* wh = reinterpret_cast<const __half2*>(&gw);
        const __half2* bh = reinterpret_cast<const __half2*>(&gb);
        float wv[8], bv[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 a = __half22float2(wh[i]), b = __half22float2(bh[i]);
            wv[2 * i] = a.x; wv[2 * i + 1] = a.y;
            bv[2 * i] = b.x; bv[2 * i + 1] = b.y;
        }
#pragma unroll
        for (int m = MM; m < 8; ++m) *reinterpret_cast<uint4*>(&xs[m][tid * 8]) = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int m = 0; m < MM; ++m) {
            uint4 o = make_uint4(0, 0, 0, 0);
            if (m < p.M) {
                const float mean = stat[0][m] * (1.0f / LN_K);
                const float rstd = 1.0f / sqrtf(stat[1][m] * (1.0f / LN_K) + p.eps);
                const float mean_rstd = mean * rstd;
                __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float y0 = (v[m][2 * i] * rstd - mean_rstd) * wv[2 * i] + bv[2 * i];
                    const float y1 = (v[m][2 * i + 1] * rstd - mean_rstd) * wv[2 * i + 1] + bv[2 * i + 1];
                    oh[i] = __floats2half2_rn(y0, y1);
                }
            }
            *reinterpret_cast<uint4*>(&xs[m][tid * 8]) = o;
        }
    }
    __syncthreads();

    // ---- the dot products
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int u = 0; u < LN_CHUNKS / LN_WARPS; ++u) {
        const int k = (warp + u * LN_WARPS) * 32;
        const uint4 xv = *reinterpret_cast<const uint4*>(&xs[g][k + t * 8]);  // rows >= M are zeros
        mma_16816(acc, lo[u].x, hi[u].x, lo[u].y, hi[u].y, xv.x, xv.y);
        mma_16816(acc, lo[u].z, hi[u].z, lo[u].w, hi[u].w, xv.z, xv.w);
    }
    partial[warp][g][2 * t] = acc[0];
    partial[warp][g][2 * t + 1] = acc[1];
    partial[warp][g + 8][2 * t] = acc[2];
    partial[warp][g + 8][2 * t + 1] = acc[3];
    __syncthreads();
    if (tid < 128) {
        const int m = tid >> 4, r = tid & 15, n = r0 + r;
        unsigned long long key = 0ull;
        if (m < p.M && n < n_seg) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < LN_WARPS; ++w) sum += partial[w][r][m];
            float val = md_round_f16(sum);
            val = md_round_f16(val + __half2float((seg2 ? p.b2 : p.b1)[n]));
            if (seg2 || p.gelu1) val = md_round_f16(md_gelu_f32(val));
            (seg2 ? p.out2 : p.out1)[(size_t)m * n_seg + n] = __float2half_rn(val);
            // Greedy sampling folded into the lm_head (sampling.zig:257-273: first strict maximum of the f16
            // logits): a 64-bit key orders by value, then by LOWER index; one atomicMax per CTA and row.
            const unsigned bits = __float_as_uint(val);
            const unsigned ordered = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
            key = ((unsigned long long)ordered << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)n);
        }
        if (p.amax && !seg2) {
#pragma unroll
            for (int o = 8; o; o >>= 1) {
                const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
                key = other > key ? other : key;
            }
            if (r == 0 && m < p.M) atomicMax(p.amax + m, key);
        }
    }
}

// ---------------------------------------------------------------------------- dual-K GEMV + residuals


struct DualKParams {
    const __half *x1, *w1, *b1;   // [M][k1], [N][k1], [N]
    const __half *x2, *w2, *b2;   // [M][k2], [N][k2], [N]
    __half* hidden;               // [M][N], updated in place
    int N, k1, k2, M;
};

template <int DK_WARPS, int UNROLL>
__global__ void __launch_bounds__(DK_WARPS * 32)
gemv_dual_k_kernel(DualKParams p) {
    __shared__ float partial[DK_WARPS][2][8][8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * 8;
    const int r = min(row0 + g, p.N - 1);
    const int units1 = p.k1 / 64, units = units1 + p.k2 / 64;  // a unit = two consecutive 32-wide k slabs
    const bool has_x = g < p.M;

    float a1e[4] = {0.f, 0.f, 0.f, 0.f}, a1o[4] = {0.f, 0.f, 0.f, 0.f};
    float a2e[4] = {0.f, 0.f, 0.f, 0.f}, a2o[4] = {0.f, 0.f, 0.f, 0.f};

    pdl_launch_dependents();
    bool waited = false;
    for (int u0 = warp; u0 < units; u0 += UNROLL * DK_WARPS) {
        uint4 lo[UNROLL], hi[UNROLL];
#pragma unroll
        for (int j = 0; j < UNROLL; ++j) {
            const int u = u0 + j * DK_WARPS;
            if (u < units) {
                const bool s2 = u >= units1;
                const __half* wrow = s2 ? p.w2 + (size_t)r * p.k2 + (size_t)(u - units1) * 64
                                        : p.w1 + (size_t)r * p.k1 + (size_t)u * 64;
                lo[j] = ldg_stream(wrow + t * 8);        // slab A: k .. k+31
                hi[j] = ldg_stream(wrow + 32 + t * 8);   // slab B: k+32 .. k+63
            } else {
                lo[j] = hi[j] = make_uint4(0, 0, 0, 0);
            }
        }
        if (!waited) { pdl_wait(); waited = true; }
#pragma unroll
        for (int j = 0; j < UNROLL; ++j) {
            const int u = u0 + j * DK_WARPS;
            if (u >= units) continue;
            const bool s2 = u >= units1;
            const __half* xrow = s2 ? p.x2 + (size_t)(has_x ? g : 0) * p.k2 + (size_t)(u - units1) * 64
                                    : p.x1 + (size_t)(has_x ? g : 0) * p.k1 + (size_t)u * 64;
            const uint4 xa = has_x ? ld_act(xrow + t * 8) : make_uint4(0, 0, 0, 0);
            const uint4 xb = has_x ? ld_act(xrow + 32 + t * 8) : make_uint4(0, 0, 0, 0);
            if (s2) {
                mma_16816(a2e, lo[j].x, hi[j].x, lo[j].y, hi[j].y, xa.x, xa.y);
                mma_16816(a2e, lo[j].z, hi[j].z, lo[j].w, hi[j].w, xa.z, xa.w);
                mma_16816(a2o, lo[j].x, hi[j].x, lo[j].y, hi[j].y, xb.x, xb.y);
                mma_16816(a2o, lo[j].z, hi[j].z, lo[j].w, hi[j].w, xb.z, xb.w);
            } else {
                mma_16816(a1e, lo[j].x, hi[j].x, lo[j].y, hi[j].y, xa.x, xa.y);
                mma_16816(a1e, lo[j].z, hi[j].z, lo[j].w, hi[j].w, xa.z, xa.w);
                mma_16816(a1o, lo[j].x, hi[j].x, lo[j].y, hi[j].y, xb.x, xb.y);
                mma_16816(a1o, lo[j].z, hi[j].z, lo[j].w, hi[j].w, xb.z, xb.w);
            }
        }
    }
    if (!waited) pdl_wait();
    // valid halves: rows 0-7 of the "even" accumulators (c0, c1), rows 8-15 of the "odd" ones (c2, c3)
    partial[warp][0][g][2 * t] = a1e[0] + a1o[2];
    partial[warp][0][g][2 * t + 1] = a1e[1] + a1o[3];
    partial[warp][1][g][2 * t] = a2e[0] + a2o[2];
    partial[warp][1][g][2 * t + 1] = a2e[1] + a2o[3];
    __syncthreads();
    if (tid < 64) {
        const int m = tid >> 3, rr = tid & 7, n = row0 + rr;
        if (m < p.M && n < p.N) {
            float s1 = 0.f, s2 = 0.f;
#pragma unroll
            for (int w = 0; w < DK_WARPS; ++w) {
                s1 += partial[w][0][rr][m];
                s2 += partial[w][1][rr][m];
            }
            const float a = md_round_f16(md_round_f16(s1) + __half2float(p.b1[n]));
            const float mlp = md_round_f16(md_round_f16(s2) + __half2float(p.b2[n]));
            const float sum = md_round_f16(a + mlp);
            __half* h = p.hidden + (size_t)m * p.N + n;
            *h = __float2half_rn(ld_act1(h) + sum);
        }
    }
}

template <class Kern, class Params>
int launch_pdl(md_ctx* ctx, Kern kern, unsigned grid, unsigned block, const Params& p, const char* name) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    if (e != cudaSuccess) return md_fail(ctx, MD_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e));
    ctx->launches++;
    return MD_OK;
}

}  // namespace

bool md_gemv_ln_dual_supported(size_t M, size_t K, size_t n1, size_t n2) {
    return M >= 1 && M <= 8 && K == LN_K && n1 % 16 == 0 && n2 % 16 == 0 && n1 > 0;
}

int md_launch_gemv_ln_dual(md_ctx* ctx, const __half* hidden, const __half* ln_w, const __half* ln_b, float eps,
                           const __half* w1, const __half* b1, __half* out1, size_t n1, const __half* w2,
                           const __half* b2, __half* out2, size_t n2, size_t M, size_t K, unsigned long long* amax,
                           bool gelu1) {
    if (!md_gemv_ln_dual_supported(M, K, n1, n2))
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "gemv_ln_dual: unsupported shape M=%zu K=%zu n1=%zu n2=%zu", M, K, n1, n2);
    LnDualParams p;
    p.hidden = hidden; p.ln_w = ln_w; p.ln_b = ln_b; p.eps = eps;
    p.w1 = w1; p.b1 = b1; p.out1 = out1; p.w2 = w2; p.b2 = b2; p.out2 = out2;
    p.n1 = (int)n1; p.n2 = (int)n2; p.M = (int)M;
    p.amax = amax;
    p.gelu1 = gelu1 ? 1 : 0;
    const unsigned grid = (unsigned)((n1 + n2) / 16);
    if (M == 1) return launch_pdl(ctx, gemv_ln_dual_kernel<1>, grid, LN_WARPS * 32, p, "gemv_ln_dual_kernel");
    if (M == 2) return launch_pdl(ctx, gemv_ln_dual_kernel<2>, grid, LN_WARPS * 32, p, "gemv_ln_dual_kernel");
    if (M <= 4) return launch_pdl(ctx, gemv_ln_dual_kernel<4>, grid, LN_WARPS * 32, p, "gemv_ln_dual_kernel");
    return launch_pdl(ctx, gemv_ln_dual_kernel<8>, grid, LN_WARPS * 32, p, "gemv_ln_dual_kernel");
}

bool md_gemv_dual_k_supported(size_t M, size_t N, size_t k1, size_t k2) {
    return M >= 1 && M <= 8 && N > 0 && k1 % 64 == 0 && k2 % 64 == 0 && k1 > 0 && k2 > 0;
}

int md_launch_gemv_dual_k(md_ctx* ctx, const __half* x1, const __half* w1, const __half* b1, size_t k1,
                          const __half* x2, const __half* w2, const __half* b2, size_t k2, __half* hidden, size_t N,
                          size_t M) {
    if (!md_gemv_dual_k_supported(M, N, k1, k2))
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "gemv_dual_k: unsupported shape M=%zu N=%zu k1=%zu k2=%zu", M, N, k1, k2);
    DualKParams p;
    p.x1 = x1; p.w1 = w1; p.b1 = b1; p.x2 = x2; p.w2 = w2; p.b2 = b2; p.hidden = hidden;
    p.N = (int)N; p.k1 = (int)k1; p.k2 = (int)k2; p.M = (int)M;
    const unsigned grid = (unsigned)((N + 7) / 8);
    switch (ctx->dualk_variant) {
        case 1: return launch_pdl(ctx, gemv_dual_k_kernel<16, 5>, grid, 16 * 32, p, "gemv_dual_k_kernel");
        case 2: return launch_pdl(ctx, gemv_dual_k_kernel<8, 10>, grid, 8 * 32, p, "gemv_dual_k_kernel");
        case 3: return launch_pdl(ctx, gemv_dual_k_kernel<4, 10>, grid, 4 * 32, p, "gemv_dual_k_kernel");
        case 4: return launch_pdl(ctx, gemv_dual_k_kernel<16, 10>, grid, 16 * 32, p, "gemv_dual_k_kernel");
        default: return launch_pdl(ctx, gemv_dual_k_kernel<8, 5>, grid, 8 * 32, p, "gemv_dual_k_kernel");
    }
}
