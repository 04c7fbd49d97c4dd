// Small bandwidth-bound kernels for the glue the reference runs between its GEMMs
// (src/core/ops.zig), plus rope, the attention mask builder, the KV-cache copies,
// argmax and the vision preprocessing.  All keep the reference's rounding points:
// f32 arithmetic on widened f16 inputs, one rounding to f16 per op.
#include "md_internal.cuh"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ops.zig:1152-1419 — one CTA per row; mean and biased variance in f32 (two passes over
// the row held in registers), y = (x*rstd - mean*rstd)*w + b, rounded once to f16.
template <int THREADS, int PER_THREAD>
__global__ void __launch_bounds__(THREADS)
layernorm_kernel(const __half* __restrict__ x, const __half* __restrict__ w, const __half* __restrict__ b,
                 __half* __restrict__ y, int cols, float eps) {
    __shared__ float red[THREADS / 32];
    __shared__ float bcast;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    md_pdl_launch_dependents();
    md_pdl_wait();
    const __half* xr = x + (size_t)blockIdx.x * cols;
    float v[PER_THREAD];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
        const int c = tid + i * THREADS;
        v[i] = c < cols ? __half2float(xr[c]) : 0.f;
        sum += v[i];
    }
    sum = warp_sum(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (tid == 0) {
        float s = 0.f;
        for (int i = 0; i < THREADS / 32; ++i) s += red[i];
        bcast = s / (float)cols;
    }
    __syncthreads();
    const float mean = bcast;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
        const int c = tid + i * THREADS;
        const float dlt = c < cols ? v[i] - mean : 0.f;
        sq += dlt * dlt;
    }
    sq = warp_sum(sq);
    __syncthreads();
    if (lane == 0) red[warp] = sq;
    __syncthreads();
    if (tid == 0) {
        float s = 0.f;
        for (int i = 0; i < THREADS / 32; ++i) s += red[i];
        bcast = 1.0f / sqrtf(s / (float)cols + eps);
    }
    __syncthreads();
    const float rstd = bcast, mean_rstd = mean * rstd;
    __half* yr = y + (size_t)blockIdx.x * cols;
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
        const int c = tid + i * THREADS;
        if (c < cols) {
            const float n = v[i] * rstd - mean_rstd;
            yr[c] = __float2half_rn(n * __half2float(w[c]) + __half2float(b[c]));
        }
    }
}

// The same LayerNorm for rows of up to 2048 columns with cols % 8 == 0 and 16-byte aligned rows: one warp per
// row (no shared memory, no block barrier), every access a 16-byte vector, the row held in registers.
constexpr int LN_ROWS_PER_CTA = 4;
__global__ void __launch_bounds__(LN_ROWS_PER_CTA * 32)
layernorm_vec_kernel(const __half* __restrict__ x, const __half* __restrict__ w, const __half* __restrict__ b,
                     __half* __restrict__ y, int rows, int cols, float eps) {
    constexpr int MAXCH = 8;  // 8 chunks x 32 lanes x 8 halves = 2048 columns
    const int lane = threadIdx.x & 31, row = blockIdx.x * LN_ROWS_PER_CTA + (threadIdx.x >> 5);
    md_pdl_launch_dependents();
    md_pdl_wait();
    if (row >= rows) return;
    const int chunks = cols >> 3;
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * cols);
    float v[MAXCH][8];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
        const int c = lane + 32 * i;
        if (c < chunks) {
            const uint4 u = xr[c];
            const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]);
                v[i][2 * j] = f.x;
                v[i][2 * j + 1] = f.y;
                sum += f.x + f.y;
            }
        }
    }
    const float mean = warp_sum(sum) / (float)cols;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
        if (lane + 32 * i < chunks) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float d = v[i][j] - mean;
                sq += d * d;
            }
        }
    }
    const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)cols + eps), mean_rstd = mean * rstd;
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * cols);
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
        const int c = lane + 32 * i;
        if (c < chunks) {
            const uint4 uw = reinterpret_cast<const uint4*>(w)[c], ub = reinterpret_cast<const uint4*>(b)[c];
            const __half2 *hw = reinterpret_cast<const __half2*>(&uw), *hb = reinterpret_cast<const __half2*>(&ub);
            uint4 o;
            __half2* ho = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 fw = __half22float2(hw[j]), fb = __half22float2(hb[j]);
                ho[j] = __floats2half2_rn((v[i][2 * j] * rstd - mean_rstd) * fw.x + fb.x,
                                          (v[i][2 * j + 1] * rstd - mean_rstd) * fw.y + fb.y);
            }
            yr[c] = o;
        }
    }
}

// The same for many rows (more than the kernel above keeps resident at once): the row stays in registers as the 16-byte
// vectors it was loaded as (4 registers per 8 columns, not 8 floats), so that eight CTAs fit an SM and enough loads
// are in flight to reach the memory rate (9477 x 1152: 14.7 -> 11.9 us); the three passes (sum, squared deviations,
// output) convert on the fly, in the same order, so the results are the same bits.  With few rows the conversions
// only lengthen each row's chain, and the kernel above is the faster one.
__global__ void __launch_bounds__(LN_ROWS_PER_CTA * 32, 8)
layernorm_vec_packed_kernel(const __half* __restrict__ x, const __half* __restrict__ w, const __half* __restrict__ b,
                     __half* __restrict__ y, int rows, int cols, float eps) {
    constexpr int MAXCH = 8;  // 8 chunks x 32 lanes x 8 halves = 2048 columns
    const int lane = threadIdx.x & 31, row = blockIdx.x * LN_ROWS_PER_CTA + (threadIdx.x >> 5);
    md_pdl_launch_dependents();
    md_pdl_wait();
    if (row >= rows) return;
    const int chunks = cols >> 3;
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * cols);
    uint4 raw[MAXCH];
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
        const int c = lane + 32 * i;
        if (c < chunks) raw[i] = xr[c];
    }
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
        if (lane + 32 * i < chunks) {
            const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]);
                sum += f.x + f.y;
            }
        }
    }
    const float mean = warp_sum(sum) / (float)cols;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
        if (lane + 32 * i < chunks) {
            const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]);
                const float d0 = f.x - mean, d1 = f.y - mean;
                sq += d0 * d0;
                sq += d1 * d1;
            }
        }
    }
    const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)cols + eps), mean_rstd = mean * rstd;
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * cols);
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
        const int c = lane + 32 * i;
        if (c < chunks) {
            const uint4 uw = reinterpret_cast<const uint4*>(w)[c], ub = reinterpret_cast<const uint4*>(b)[c];
            const __half2 *hw = reinterpret_cast<const __half2*>(&uw), *hb = reinterpret_cast<const __half2*>(&ub);
            const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
            uint4 o;
            __half2* ho = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]), fw = __half22float2(hw[j]), fb = __half22float2(hb[j]);
                ho[j] = __floats2half2_rn((f.x * rstd - mean_rstd) * fw.x + fb.x, (f.y * rstd - mean_rstd) * fw.y + fb.y);
            }
            yr[c] = o;
        }
    }
}

__global__ void gelu_kernel(__half* __restrict__ x, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        x[i] = __float2half_rn(md_gelu_f32(__half2float(x[i])));
}

__global__ void bias_add_kernel(__half* __restrict__ a, const __half* __restrict__ b, size_t rows, size_t cols) {
    const size_t n = rows * cols, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        a[i] = __float2half_rn(__half2float(a[i]) + __half2float(b[i % cols]));
}

__global__ void add_kernel(__half* __restrict__ a, const __half* __restrict__ b, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        a[i] = __float2half_rn(__half2float(a[i]) + __half2float(b[i]));
}

// sampling.zig:257-273 — first index of the strict maximum.  Single CTA: n is the
// vocabulary (51200 f16 = 100 KB), far below what one SM streams in a few microseconds.
__global__ void __launch_bounds__(1024)
argmax_kernel(const __half* __restrict__ x, size_t n, unsigned long long* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ unsigned long long si[32];
    float best = -INFINITY;
    unsigned long long bi = ~0ull;
    for (size_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = __half2float(x[i]);
        if (bi == ~0ull || v > best) { best = v; bi = i; }  // ascending i: strict > keeps the first
    }
    auto better = [](float v, unsigned long long i, float bv, unsigned long long bidx) {
        if (i == ~0ull) return false;
        if (bidx == ~0ull) return true;
        return v > bv || (v == bv && i < bidx);
    };
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const unsigned long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : ~0ull;
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const unsigned long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) *out = (bi == ~0ull) ? 0ull : bi;
    }
}

// The same for `gridDim.x` rows at once (row r at x + r * stride, n % 8 == 0, 16-byte aligned rows), one CTA per
// row: 16-byte loads, all of a thread's loads requested before the first compare.  A thread walks its elements in
// ascending order and a later element replaces the best only when strictly greater, as above.
constexpr int ARGMAX_VEC_MAX = 8;   // vectors per thread: rows of up to 1024 x 8 x 8 = 65536 elements
__global__ void __launch_bounds__(1024)
argmax_rows_kernel(const __half* __restrict__ x, size_t n, size_t stride, unsigned long long* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ unsigned long long si[32];
    md_pdl_launch_dependents();
    md_pdl_wait();
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)blockIdx.x * stride);
    const size_t nvec = n >> 3;
    uint4 v[ARGMAX_VEC_MAX];
#pragma unroll
    for (int k = 0; k < ARGMAX_VEC_MAX; ++k) {
        const size_t c = threadIdx.x + (size_t)k * blockDim.x;
        if (c < nvec) v[k] = __ldcg(xr + c);
    }
    float best = -INFINITY;
    unsigned long long bi = ~0ull;
#pragma unroll
    for (int k = 0; k < ARGMAX_VEC_MAX; ++k) {
        const size_t c = threadIdx.x + (size_t)k * blockDim.x;
        if (c < nvec) {
            const __half* h = reinterpret_cast<const __half*>(&v[k]);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float f = __half2float(h[e]);
                if (bi == ~0ull || f > best) { best = f; bi = c * 8 + e; }
            }
        }
    }
    auto better = [](float a, unsigned long long i, float bv, unsigned long long bidx) {
        if (i == ~0ull) return false;
        if (bidx == ~0ull) return true;
        return a > bv || (a == bv && i < bidx);
    };
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const unsigned long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : ~0ull;
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const unsigned long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) out[blockIdx.x] = (bi == ~0ull) ? 0ull : bi;
    }
}

// vision_model.zig:137-183 + reshape_handler.zig:5-129.  One thread per output element.
__global__ void patchify_kernel(const uint8_t* __restrict__ img, __half* __restrict__ out, int crops, int height,
                                int width, int patch, int out_stride) {
    const int wp = width / patch, hp = height / patch, pd = 3 * patch * patch;
    const size_t total = (size_t)crops * hp * wp * out_stride;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int e = (int)(i % out_stride);
        const size_t tok = i / out_stride;
        if (e >= pd) { out[i] = __float2half_rn(0.f); continue; }
        const int pidx = (int)(tok % (hp * wp)), b = (int)(tok / (hp * wp));
        const int c = e / (patch * patch), ph = (e / patch) % patch, pw = e % patch;
        const int yy = (pidx / wp) * patch + ph, xx = (pidx % wp) * patch + pw;
        const uint8_t u = img[(((size_t)b * height + yy) * width + xx) * 3 + c];
        // every step rounds to f16, as the reference's f16 tensor arithmetic does
        float v = md_round_f16((float)u);
        v = md_round_f16(v / 255.0f);
        v = md_round_f16(v - 0.5f);
        v = md_round_f16(v / 0.5f);
        out[i] = __float2half_rn(v);
    }
}

// rope.zig:32-128
__global__ void rope_table_kernel(float* __restrict__ table, int dim, int end, float theta) {
    const int half = dim / 2;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= end * half) return;
    const int p = i / half, j = i % half;
    const float freq = 1.0f / powf(theta, (float)(2 * j) / (float)dim);
    const float ang = (float)p * freq;
    table[2 * i] = cosf(ang);
    table[2 * i + 1] = sinf(ang);
}

// rope.zig:130-272
__global__ void rope_apply_kernel(const __half* __restrict__ x, __half* __restrict__ out, int n_heads, int seq_len,
                                  int d, const float* __restrict__ freqs, const unsigned long long* __restrict__ pos,
                                  int rot_dim) {
    const size_t total = (size_t)n_heads * seq_len * d;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const int half = rot_dim / 2;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int dd = (int)(i % d);
        const int s = (int)((i / d) % seq_len);
        if (dd >= rot_dim) { out[i] = x[i]; continue; }
        const int j = dd < half ? dd : dd - half;
        const size_t base = i - dd;
        const float* f = freqs + ((size_t)pos[s] * half + j) * 2;
        const float c = f[0], sn = f[1];
        const float xr = __half2float(x[base + j]), xi = __half2float(x[base + j + half]);
        out[i] = __float2half_rn(dd < half ? xr * c - xi * sn : xr * sn + xi * c);
    }
}

// attention.zig:256-281
__global__ void mask_kernel(uint8_t* __restrict__ mask, size_t pos, size_t seq_len) {
    const size_t w = pos + seq_len, total = seq_len * w;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t r = i / w, c = i % w;
        mask[i] = (c < pos || c - pos <= r) ? 1 : 0;
    }
}

// text_model.zig:476-515 (append) and :436-474 (copy the active prefix out)
__global__ void kv_update_kernel(__half* __restrict__ kc, __half* __restrict__ vc, const __half* __restrict__ k,
                                 const __half* __restrict__ v, int n_heads, int max_seq, int d, int cur, int s_len) {
    const size_t total = (size_t)n_heads * s_len * d, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int dd = (int)(i % d), s = (int)((i / d) % s_len), h = (int)(i / ((size_t)d * s_len));
        const size_t dst = ((size_t)h * max_seq + cur + s) * d + dd;
        kc[dst] = k[i];
        vc[dst] = v[i];
    }
}
__global__ void kv_active_kernel(const __half* __restrict__ kc, const __half* __restrict__ vc, __half* __restrict__ k,
                                 __half* __restrict__ v, int n_heads, int max_seq, int d, int cur) {
    const size_t total = (size_t)n_heads * cur * d, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int dd = (int)(i % d), s = (int)((i / d) % cur), h = (int)(i / ((size_t)d * cur));
        const size_t src = ((size_t)h * max_seq + s) * d + dd;
        k[i] = kc[src];
        v[i] = vc[src];
    }
}

unsigned grid_for(size_t n, int block, int sm_count) {
    size_t g = (n + block - 1) / block;
    const size_t cap = (size_t)sm_count * 16;
    if (g > cap) g = cap;
    return (unsigned)(g ? g : 1);
}

}  // namespace

int md_launch_layernorm(md_ctx* ctx, const __half* x, const __half* w, const __half* b, __half* y, size_t rows,
                        size_t cols, float eps) {
    if (rows == 0) return MD_OK;
    const bool vec = cols <= 2048 && (cols % 8) == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(w) |
                       reinterpret_cast<uintptr_t>(b)) & 15) == 0;
    if (vec) {
        const dim3 grid((unsigned)((rows + LN_ROWS_PER_CTA - 1) / LN_ROWS_PER_CTA)), block(LN_ROWS_PER_CTA * 32);
        // rows beyond what five CTAs per SM hold at once: the form with the smaller register footprint
        if (rows > (size_t)5 * LN_ROWS_PER_CTA * ctx->sm_count)
            return md_launch_ex(ctx, layernorm_vec_packed_kernel, grid, block, 0, "layernorm_vec_packed_kernel", x, w, b, y,
                                (int)rows, (int)cols, eps);
        return md_launch_ex(ctx, layernorm_vec_kernel, grid, block, 0, "layernorm_vec_kernel", x, w, b, y, (int)rows,
                            (int)cols, eps);
    }
    if (cols <= 256 * 8)
        return md_launch_ex(ctx, layernorm_kernel<256, 8>, dim3((unsigned)rows), dim3(256), 0, "layernorm_kernel", x, w, b,
                            y, (int)cols, eps);
    if (cols <= 1024 * 16)
        return md_launch_ex(ctx, layernorm_kernel<1024, 16>, dim3((unsigned)rows), dim3(1024), 0, "layernorm_kernel", x, w,
                            b, y, (int)cols, eps);
    return md_fail(ctx, MD_ERR_UNSUPPORTED, "layernorm rows longer than 16384 are not supported (%zu)", cols);
}

int md_launch_gelu(md_ctx* ctx, __half* x, size_t n) {
    if (!n) return MD_OK;
    gelu_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(x, n);
    MD_LAUNCH_CHECK(ctx, "gelu_kernel");
    return MD_OK;
}

int md_launch_bias_add(md_ctx* ctx, __half* a, const __half* b, size_t rows, size_t cols) {
    if (!rows || !cols) return MD_OK;
    bias_add_kernel<<<grid_for(rows * cols, 256, ctx->sm_count), 256, 0, ctx->stream>>>(a, b, rows, cols);
    MD_LAUNCH_CHECK(ctx, "bias_add_kernel");
    return MD_OK;
}

int md_launch_add(md_ctx* ctx, __half* a, const __half* b, size_t n) {
    if (!n) return MD_OK;
    add_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(a, b, n);
    MD_LAUNCH_CHECK(ctx, "add_kernel");
    return MD_OK;
}

int md_launch_argmax(md_ctx* ctx, const __half* x, size_t n, unsigned long long* idx_dev) {
    return md_launch_argmax_rows(ctx, x, n, n, 1, idx_dev);
}

// The greedy sample of `rows` rows (row r at x + r * stride) into idx_dev[0 .. rows): one launch.
int md_launch_argmax_rows(md_ctx* ctx, const __half* x, size_t n, size_t stride, size_t rows,
                          unsigned long long* idx_dev) {
    if (!rows) return MD_OK;
    const bool vec = n > 0 && (n % 8) == 0 && (stride % 8) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                     n <= (size_t)1024 * 8 * ARGMAX_VEC_MAX && rows <= 65535;
    if (vec)
        return md_launch_ex(ctx, argmax_rows_kernel, dim3((unsigned)rows), dim3(1024), 0, "argmax_rows_kernel", x, n,
                            stride, idx_dev);
    for (size_t r = 0; r < rows; ++r) {
        argmax_kernel<<<1, 1024, 0, ctx->stream>>>(x + r * stride, n, idx_dev + r);
        MD_LAUNCH_CHECK(ctx, "argmax_kernel");
    }
    return MD_OK;
}

int md_launch_patchify(md_ctx* ctx, const uint8_t* img, __half* out, size_t crops, size_t h, size_t w, size_t patch,
                       size_t out_stride) {
    const size_t total = crops * (h / patch) * (w / patch) * out_stride;
    if (!total) return MD_OK;
    patchify_kernel<<<grid_for(total, 256, ctx->sm_count), 256, 0, ctx->stream>>>(img, out, (int)crops, (int)h, (int)w,
                                                                                  (int)patch, (int)out_stride);
    MD_LAUNCH_CHECK(ctx, "patchify_kernel");
    return MD_OK;
}

int md_launch_rope_table(md_ctx* ctx, float* table, size_t dim, size_t end, float theta) {
    const size_t n = end * (dim / 2);
    rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(table, (int)dim, (int)end, theta);
    MD_LAUNCH_CHECK(ctx, "rope_table_kernel");
    return MD_OK;
}

int md_launch_rope_apply(md_ctx* ctx, const __half* x, __half* out, size_t n_heads, size_t seq_len, size_t d,
                         const float* freqs, const unsigned long long* pos, size_t rot_dim) {
    const size_t n = n_heads * seq_len * d;
    if (!n) return MD_OK;
    rope_apply_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(x, out, (int)n_heads, (int)seq_len,
                                                                               (int)d, freqs, pos, (int)rot_dim);
    MD_LAUNCH_CHECK(ctx, "rope_apply_kernel");
    return MD_OK;
}

int md_launch_mask(md_ctx* ctx, uint8_t* mask, size_t pos, size_t seq_len) {
    const size_t n = seq_len * (pos + seq_len);
    if (!n) return MD_OK;
    mask_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(mask, pos, seq_len);
    MD_LAUNCH_CHECK(ctx, "mask_kernel");
    return MD_OK;
}

int md_launch_kv_update(md_ctx* ctx, __half* kc, __half* vc, const __half* k, const __half* v, size_t n_heads,
                        size_t max_seq, size_t d, size_t cur_len, size_t seq_len) {
    const size_t n = n_heads * seq_len * d;
    if (!n) return MD_OK;
    kv_update_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(kc, vc, k, v, (int)n_heads, (int)max_seq,
                                                                              (int)d, (int)cur_len, (int)seq_len);
    MD_LAUNCH_CHECK(ctx, "kv_update_kernel");
    return MD_OK;
}

int md_launch_kv_active(md_ctx* ctx, const __half* kc, const __half* vc, __half* k, __half* v, size_t n_heads,
                        size_t max_seq, size_t d, size_t cur_len) {
    const size_t n = n_heads * cur_len * d;
    if (!n) return MD_OK;
    kv_active_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(kc, vc, k, v, (int)n_heads, (int)max_seq,
                                                                              (int)d, (int)cur_len);
    MD_LAUNCH_CHECK(ctx, "kv_active_kernel");
    return MD_OK;
}
