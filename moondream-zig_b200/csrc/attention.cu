// Fused scaled-dot-product attention kernels.
//
//   sdpa_mma_kernel     multi-query attention (ViT 729 x 729 with d = 72, decoder prefill with
//                       d = 64): replaces attention.multiMasklessSDPA (attention.zig:125-234)
//                       and attention.multiMaskedSDPA (attention.zig:416-541).  The reference
//                       materialises the full f32 score matrix per head and runs two f32 GEMMs
//                       around a row softmax; here scores never leave the SM: 64-query x 64-key
//                       tiles, S = Q K^T and O += P V on tensor cores (mma.sync m16n8k16, f32
//                       accumulate), online softmax in f32 registers.  Strided addressing lets it
//                       read q, k, v straight out of a fused qkv projection or the KV cache.
//   sdpa_generic_kernel any head_dim <= 256, one warp per query row (odd shapes only).
//   sdpa_decode_kernel  one query token against the cache (attention.singleMaskedSDPA,
//                       attention.zig:564-642,759-811): split over the keys, 128-bit loads,
//                       partial (max, sum, out) per split merged by the last CTA of each head.
//                       The fused form also applies the partial rotary embedding to q and the
//                       new k (rope.zig:130-272) and appends k, v to the cache in place
//                       (text_model.zig:476-515), so no copy of the active cache is ever made
//                       (text_model.zig:436-474 copies it on every call).
//
// Numerics: q, k, v are f16, scores / probabilities / accumulators f32, one rounding to f16
// at the output (attention.zig:199-202,505-508,635-640).  The tensor-core kernel rounds the
// probabilities to f16 for the P V product (relative error <= 2^-11 per weight).  A query row
// whose keys are all masked yields zeros (the reference leaves -inf scores in place, which
// cannot happen with the masks createAttentionMask builds).
#include "md_internal.cuh"

#include <cfloat>

namespace {

constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

struct SdpaParams {
    const __half *q, *k, *v;
    __half* out;
    const uint8_t* mask;  // [q_len, kv_len] or null
    int q_len, kv_len;
    long long q_row, q_head, q_batch, kv_row, kv_head, kv_batch, o_row, o_head, o_batch;
    int causal_pos;  // < 0: none; else key j is visible to query i iff j <= causal_pos + i
    float scale_log2;  // (1/sqrt(d)) * log2(e)
};

constexpr int BQ = 64, BKV = 64;

template <int D, int D_PAD>
__global__ void __launch_bounds__(128)
sdpa_mma_kernel(SdpaParams p) {
    md_pdl_launch_dependents();
    md_pdl_wait();
    constexpr int PITCH = D_PAD + 8;  // halves; 144 B or 176 B rows keep ldmatrix conflict-free
    constexpr int CHUNKS = D_PAD / 8, REAL_CHUNKS = D / 8;
    // dynamic shared memory: Q tile, then two K and two V tiles (double buffered)
    extern __shared__ __align__(16) unsigned char sdpa_smem[];
    __half (*Qs)[PITCH] = reinterpret_cast<__half (*)[PITCH]>(sdpa_smem);
    __half (*Ks)[BKV][PITCH] = reinterpret_cast<__half (*)[BKV][PITCH]>(sdpa_smem + BQ * PITCH * 2);
    __half (*Vs)[BKV][PITCH] = reinterpret_cast<__half (*)[BKV][PITCH]>(sdpa_smem + (BQ + 2 * BKV) * PITCH * 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    // causal: the last query blocks see the most keys; give them the lowest block ids so they start first
    const int qblk = p.causal_pos >= 0 ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
    const int q0 = qblk * BQ, head = blockIdx.y, batch = blockIdx.z;
    const __half* qb = p.q + batch * p.q_batch + head * p.q_head;
    const __half* kb = p.k + batch * p.kv_batch + head * p.kv_head;
    const __half* vb = p.v + batch * p.kv_batch + head * p.kv_head;

    for (int idx = tid; idx < BQ * CHUNKS; idx += 128) {
        const int r = idx / CHUNKS, c = idx % CHUNKS;
        if (q0 + r < p.q_len && c < REAL_CHUNKS)
            cp_async16(smem_u32(&Qs[r][c * 8]), qb + (long long)(q0 + r) * p.q_row + c * 8);
        else
            *reinterpret_cast<uint4*>(&Qs[r][c * 8]) = make_uint4(0, 0, 0, 0);
    }
    cp_async_wait_all();
    __syncthreads();

    uint32_t qf[D_PAD / 16][4];
#pragma unroll
    for (int ks = 0; ks < D_PAD / 16; ++ks) {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = ks * 16 + (lane >> 4) * 8;
        ldsm_x4(smem_u32(&Qs[r][c]), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }

    float o[D_PAD / 8][4];
#pragma unroll
    for (int i = 0; i < D_PAD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int qi[2] = {q0 + warp * 16 + g, q0 + warp * 16 + g + 8};

    int kv_end = p.kv_len;
    if (p.causal_pos >= 0) kv_end = min(kv_end, p.causal_pos + min(q0 + BQ, p.q_len));

    // K/V tiles are double buffered: the loads of tile j+1 are in flight while tile j is consumed
    auto load_tile = [&](int k0, int buf) {
        for (int idx = tid; idx < BKV * CHUNKS; idx += 128) {
            const int r = idx / CHUNKS, c = idx % CHUNKS;
            if (k0 + r < p.kv_len && c < REAL_CHUNKS) {
                cp_async16(smem_u32(&Ks[buf][r][c * 8]), kb + (long long)(k0 + r) * p.kv_row + c * 8);
                cp_async16(smem_u32(&Vs[buf][r][c * 8]), vb + (long long)(k0 + r) * p.kv_row + c * 8);
            } else {
                *reinterpret_cast<uint4*>(&Ks[buf][r][c * 8]) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(&Vs[buf][r][c * 8]) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (kv_end > 0) load_tile(0, 0);
    for (int k0 = 0, it = 0; k0 < kv_end; k0 += BKV, ++it) {
        const int buf = it & 1;
        if (k0 + BKV < kv_end) {
            load_tile(k0 + BKV, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();

        float s[BKV / 8][4];
#pragma unroll
        for (int i = 0; i < BKV / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D_PAD / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < BKV / 16; ++np) {
                uint32_t b0, b1, b2, b3;
                const int r = np * 16 + (lane & 7) + (lane >> 4) * 8, c = ks * 16 + ((lane >> 3) & 1) * 8;
                ldsm_x4(smem_u32(&Ks[buf][r][c]), b0, b1, b2, b3);
                mma_16816(s[2 * np], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                mma_16816(s[2 * np + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
            }
        }

        // scale (folded with log2 e), mask, row maxima
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < BKV / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int rr = e >> 1;
                const int key = k0 + nt * 8 + 2 * t + (e & 1);
                bool vis = key < p.kv_len && qi[rr] < p.q_len;
                if (p.causal_pos >= 0) vis = vis && key <= p.causal_pos + qi[rr];
                if (vis && p.mask) vis = p.mask[(long long)qi[rr] * p.kv_len + key] != 0;
                const float v = vis ? s[nt][e] * p.scale_log2 : -INFINITY;
                s[nt][e] = v;
                mx[rr] = fmaxf(mx[rr], v);
            }
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
            const float m_new = fmaxf(m_run[rr], mx[rr]);
            m_use[rr] = (m_new == -INFINITY) ? 0.f : m_new;
            corr[rr] = (m_run[rr] == -INFINITY) ? 0.f : exp2f(m_run[rr] - m_use[rr]);
            m_run[rr] = m_new;
        }
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < BKV / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = exp2f(s[nt][e] - m_use[e >> 1]);
                s[nt][e] = pv;
                rs[e >> 1] += pv;
            }
        }
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            rs[rr] += __shfl_xor_sync(0xffffffffu, rs[rr], 1);
            rs[rr] += __shfl_xor_sync(0xffffffffu, rs[rr], 2);
            l_run[rr] = l_run[rr] * corr[rr] + rs[rr];
        }
#pragma unroll
        for (int i = 0; i < D_PAD / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
            const uint32_t a0 = pack_h2(s[2 * kk][0], s[2 * kk][1]), a1 = pack_h2(s[2 * kk][2], s[2 * kk][3]);
            const uint32_t a2 = pack_h2(s[2 * kk + 1][0], s[2 * kk + 1][1]),
                           a3 = pack_h2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < D_PAD / 16; ++dp) {
                uint32_t b0, b1, b2, b3;
                const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = dp * 16 + (lane >> 4) * 8;
                ldsm_x4_t(smem_u32(&Vs[buf][r][c]), b0, b1, b2, b3);
                mma_16816(o[2 * dp], a0, a1, a2, a3, b0, b1);
                mma_16816(o[2 * dp + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        __syncthreads();
    }

    __half* ob = p.out + batch * p.o_batch + head * p.o_head;
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        if (qi[rr] >= p.q_len) continue;
        const float inv = l_run[rr] > 0.f ? 1.0f / l_run[rr] : 0.f;
        __half* orow = ob + (long long)qi[rr] * p.o_row;
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt) {
            const __half2 h = __floats2half2_rn(o[nt][2 * rr] * inv, o[nt][2 * rr + 1] * inv);
            *reinterpret_cast<__half2*>(orow + nt * 8 + 2 * t) = h;
        }
    }
}

// One warp per (query row, head): any head_dim <= 256.  Slow path for odd shapes.
__global__ void __launch_bounds__(128)
sdpa_generic_kernel(SdpaParams p, int d, int n_heads, float scale) {
    const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int total = p.q_len * n_heads;
    const int batch = blockIdx.y;
    if (warp_global >= total) return;
    const int head = warp_global / p.q_len, qi = warp_global % p.q_len;
    const __half* q = p.q + batch * p.q_batch + head * p.q_head + (long long)qi * p.q_row;
    const __half* kb = p.k + batch * p.kv_batch + head * p.kv_head;
    const __half* vb = p.v + batch * p.kv_batch + head * p.kv_head;
    float qv[8], acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = lane + 32 * i;
        qv[i] = c < d ? __half2float(q[c]) : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (int j = 0; j < p.kv_len; ++j) {
        bool vis = true;
        if (p.causal_pos >= 0) vis = j <= p.causal_pos + qi;
        if (vis && p.mask) vis = p.mask[(long long)qi * p.kv_len + j] != 0;
        if (!vis) continue;
        const __half* kr = kb + (long long)j * p.kv_row;
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = lane + 32 * i;
            if (c < d) dot += qv[i] * __half2float(kr[c]);
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        const float sc = dot * scale;
        const float m_new = fmaxf(m, sc);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float pw = expf(sc - m_new);
        l = l * corr + pw;
        const __half* vr = vb + (long long)j * p.kv_row;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = lane + 32 * i;
            if (c < d) acc[i] = acc[i] * corr + pw * __half2float(vr[c]);
        }
        m = m_new;
    }
    __half* o = p.out + batch * p.o_batch + head * p.o_head + (long long)qi * p.o_row;
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = lane + 32 * i;
        if (c < d) o[c] = __float2half_rn(acc[i] * inv);
    }
}

// ------------------------------------------------------------------------------ decode
constexpr int DEC_D = 64;          // head_dim (attention.zig:248-249)
constexpr int DEC_KEYS = 128;      // keys per CTA (split)
constexpr int DEC_WARPS = 4;

struct DecodeParams {
    const __half* q;        // plain: [n_heads][64]; fused: qkv row [3*n_heads*64]
    const __half* k;        // [n_heads][k_head_stride / 64][64]
    const __half* v;
    __half* k_w;            // fused: cache to append to (same memory as k), else null
    __half* v_w;
    const uint8_t* mask;    // [kv_len] or null
    __half* out;            // [n_heads][64]
    float* partial;         // [n_heads][splits][66]: max, sum, out[64]
    unsigned int* counters; // [n_heads], zero before launch, left zero after
    long long k_head_stride;
    int n_heads, kv_cache_len;  // keys to read from memory
    int fused, pos, rot_dim;
    float theta;
    int splits;
    const float* rope_tab;  // fused: (cos, sin) table [positions][rot_dim/2][2] (rope.zig:32-128)
    const int* pos_ptr;     // fused + graph replay: position read from device memory, else null
    // batch > 0: blockIdx.z selects one of up to 8 requests, each with its own cache and position; q and out
    // advance by a row per request, partial and counters by one request's worth
    int batch;
    long long q_batch_stride, out_batch_stride;
    __half* bk[8];
    __half* bv[8];
    const int* bpos[8];
};

__device__ __forceinline__ uint4 ldg_nc16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
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

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// rope.zig:50-65,223-230 for one head vector held in shared memory (f32 in, f16-rounded by the caller), with the
// (cos, sin) pair of dim dd already in registers.
__device__ __forceinline__ float rope_rotate(const float* x, int dd, int rot_dim, float2 cs) {
    if (dd >= rot_dim) return x[dd];
    const int half = rot_dim / 2, j = dd < half ? dd : dd - half;
    const float xr = x[j], xi = x[j + half];
    return dd < half ? xr * cs.x - xi * cs.y : xr * cs.y + xi * cs.x;
}

// CLUSTER: the splits of one head form a thread-block cluster (16 CTAs along x); the partial results are
// merged through distributed shared memory of the cluster's first CTA instead of global scratch, fences
// and an atomic ticket.
template <bool CLUSTER>
__global__ void __launch_bounds__(DEC_WARPS * 32)
sdpa_decode_kernel(const __grid_constant__ DecodeParams gp) {
    // the per-request tables are indexed in the constant bank; the working copy below is only accessed by field
    DecodeParams p = gp;
    __shared__ float cpart[CLUSTER ? 16 : 1][DEC_D + 2];
    __shared__ float q_s[DEC_D], knew_s[DEC_D], vnew_s[DEC_D], raw_s[DEC_D], rawk_s[DEC_D];
    __shared__ float red_m[DEC_WARPS], red_l[DEC_WARPS], red_o[DEC_WARPS][DEC_D];
    __shared__ int is_last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head = blockIdx.y, split = blockIdx.x;
    if (p.batch > 0) {
        const int b = blockIdx.z;
        p.q += b * p.q_batch_stride;
        p.out += b * p.out_batch_stride;
        p.k = p.k_w = gp.bk[b];
        p.v = p.v_w = gp.bv[b];
        p.pos_ptr = gp.bpos[b];
        p.counters += b * p.n_heads;
        p.partial += (long long)b * p.n_heads * p.splits * (DEC_D + 2);
    }
    if (p.pos_ptr) {
        // Position held in device memory (graph replay): the grid is sized for the longest
        // context, CTAs beyond the splits this position needs leave at once.
        p.pos = *p.pos_ptr;
        p.kv_cache_len = p.pos;
        p.splits = max(1, (p.pos + DEC_KEYS - 1) / DEC_KEYS);
        if (split >= p.splits) {
            if (CLUSTER) cluster_sync_all();  // the merging CTA waits for every CTA of the cluster
            return;
        }
    }
    const bool last_split = split == p.splits - 1;
    const float scale = 0.125f;  // 1/sqrt(64)

    const int sub = lane & 7, grp = lane >> 3;  // 8 lanes x 16 B cover one 128-byte key row
    // ---- request this CTA's keys and values first: the cached prefix was written by earlier steps, so
    //      under programmatic dependent launch these loads overlap the tail of the kernel that produces q
    asm volatile("griddepcontrol.launch_dependents;");
    const __half* kh = p.k + head * p.k_head_stride;
    const __half* vh = p.v + head * p.k_head_stride;
    const int key_lo = split * DEC_KEYS + warp * (DEC_KEYS / DEC_WARPS);
    constexpr int ITER = DEC_KEYS / DEC_WARPS / 4;  // 8 keys per lane group

    uint4 kreg[ITER], vreg[ITER];
    bool valid[ITER];
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
        const int key = key_lo + it * 4 + grp;
        valid[it] = key < p.kv_cache_len;
        kreg[it] = valid[it] ? ldg_nc16(kh + (long long)key * DEC_D + sub * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
        const int key = key_lo + it * 4 + grp;
        vreg[it] = valid[it] ? ldg_nc16(vh + (long long)key * DEC_D + sub * 8) : make_uint4(0, 0, 0, 0);
    }
    // the rope factors of this thread's dim depend on the position alone: requested before the wait as well
    float2 cs = make_float2(1.f, 0.f);
    if (p.fused && tid < p.rot_dim) {
        const int half = p.rot_dim >> 1, j = tid < half ? tid : tid - half;
        cs = __ldg(reinterpret_cast<const float2*>(p.rope_tab + ((size_t)p.pos * half + j) * 2));  // (cos, sin)
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- stage q (and, fused, the new k and v) in shared memory: one round of loads, then the rotation
    if (p.fused) {
        const int hd = p.n_heads * DEC_D;
        __half vn = __float2half_rn(0.f);
        if (tid < DEC_D) {
            const __half rq = __ldcg(p.q + head * DEC_D + tid);
            if (last_split) {
                const __half rk = __ldcg(p.q + hd + head * DEC_D + tid);
                vn = __ldcg(p.q + 2 * hd + head * DEC_D + tid);
                rawk_s[tid] = __half2float(rk);
            }
            raw_s[tid] = __half2float(rq);
        }
        __syncthreads();
        if (tid < DEC_D) {
            q_s[tid] = md_round_f16(rope_rotate(raw_s, tid, p.rot_dim, cs));
            if (last_split) {
                const __half kr = __float2half_rn(rope_rotate(rawk_s, tid, p.rot_dim, cs));
                knew_s[tid] = __half2float(kr);
                vnew_s[tid] = __half2float(vn);
                p.k_w[head * p.k_head_stride + (long long)p.pos * DEC_D + tid] = kr;
                p.v_w[head * p.k_head_stride + (long long)p.pos * DEC_D + tid] = vn;
            }
        }
    } else {
        if (tid < DEC_D) q_s[tid] = __half2float(__ldcg(p.q + head * DEC_D + tid));
    }
    __syncthreads();

    float qv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) qv[i] = q_s[sub * 8 + i];

    float sc[ITER];
    float m = -INFINITY;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
        float kf[8];
        unpack8(kreg[it], kf);
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) dot = fmaf(qv[i], kf[i], dot);
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        dot += __shfl_xor_sync(0xffffffffu, dot, 4);
        const int key = key_lo + it * 4 + grp;
        bool vis = valid[it];
        if (vis && p.mask) vis = p.mask[key] != 0;
        sc[it] = vis ? dot * scale : -INFINITY;
        m = fmaxf(m, sc[it]);
    }
    // the appended token: handled by lane group 0 of warp 0 of the last split
    float s_new = -INFINITY;
    const bool do_new = p.fused && last_split && warp == 0 && grp == 0;
    if (do_new) {
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) dot = fmaf(qv[i], knew_s[sub * 8 + i], dot);
        dot += __shfl_xor_sync(0x000000ffu, dot, 1);
        dot += __shfl_xor_sync(0x000000ffu, dot, 2);
        dot += __shfl_xor_sync(0x000000ffu, dot, 4);
        s_new = dot * scale;
        m = fmaxf(m, s_new);
    }
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
    const float m_use = (m == -INFINITY) ? 0.f : m;
    float l = 0.f, acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
        const float pw = expf(sc[it] - m_use);  // exp(-inf) = 0 for masked / absent keys
        l += pw;
        float vf[8];
        unpack8(vreg[it], vf);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(pw, vf[i], acc[i]);
    }
    if (do_new) {
        const float pw = expf(s_new - m_use);
        l += pw;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(pw, vnew_s[sub * 8 + i], acc[i]);
    }
    // combine the four lane groups (each lane keeps its 8 dims)
    l += __shfl_xor_sync(0xffffffffu, l, 8);
    l += __shfl_xor_sync(0xffffffffu, l, 16);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 8);
        acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 16);
    }
    if (lane < 8) {
#pragma unroll
        for (int i = 0; i < 8; ++i) red_o[warp][lane * 8 + i] = acc[i];
    }
    if (lane == 0) { red_m[warp] = m; red_l[warp] = l; }
    __syncthreads();

    // combine the warps: thread d < 64 owns output dim d
    float M = -INFINITY, L = 0.f, O = 0.f;
    if (tid < DEC_D) {
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, red_m[w]);
        const float Mu = (M == -INFINITY) ? 0.f : M;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float f = (red_m[w] == -INFINITY) ? 0.f : expf(red_m[w] - Mu);
            L += red_l[w] * f;
            O += red_o[w][tid] * f;
        }
    }
    if (CLUSTER) {
        // every CTA deposits (max, sum, out[64]) in slot `split` of the first CTA's shared memory
        const uint32_t local = smem_u32(&cpart[split][0]);
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(0));
        if (tid < DEC_D) asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + (2 + tid) * 4), "f"(O) : "memory");
        if (tid == 0) {
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(M) : "memory");
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + 4), "f"(L) : "memory");
        }
        cluster_sync_all();
        if (split == 0 && tid < DEC_D) {
            float Mg = -INFINITY;
            for (int s2 = 0; s2 < p.splits; ++s2) Mg = fmaxf(Mg, cpart[s2][0]);
            const float Mu = (Mg == -INFINITY) ? 0.f : Mg;
            float Lg = 0.f, Og = 0.f;
            for (int s2 = 0; s2 < p.splits; ++s2) {
                const float ms = cpart[s2][0];
                const float f = (ms == -INFINITY) ? 0.f : expf(ms - Mu);
                Lg += cpart[s2][1] * f;
                Og += cpart[s2][2 + tid] * f;
            }
            p.out[head * DEC_D + tid] = __float2half_rn(Lg > 0.f ? Og / Lg : 0.f);
        }
        return;
    }
    if (p.splits == 1) {
        if (tid < DEC_D) p.out[head * DEC_D + tid] = __float2half_rn(L > 0.f ? O / L : 0.f);
        return;
    }
    float* mine = p.partial + ((long long)head * p.splits + split) * (DEC_D + 2);
    if (tid < DEC_D) mine[2 + tid] = O;
    if (tid == 0) { mine[0] = M; mine[1] = L; }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int ticket = atomicAdd(&p.counters[head], 1u);
        is_last = (ticket == (unsigned)p.splits - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (tid < DEC_D && p.splits <= 16) {
        // every partial in one round of loads
        const float* base = p.partial + (long long)head * p.splits * (DEC_D + 2);
        float ms[16], ls[16], os[16];
#pragma unroll
        for (int s2 = 0; s2 < 16; ++s2) {
            const bool live = s2 < p.splits;
            ms[s2] = live ? __ldcg(base + s2 * (DEC_D + 2)) : -INFINITY;
            ls[s2] = live ? __ldcg(base + s2 * (DEC_D + 2) + 1) : 0.f;
            os[s2] = live ? __ldcg(base + s2 * (DEC_D + 2) + 2 + tid) : 0.f;
        }
        float Mg = -INFINITY;
#pragma unroll
        for (int s2 = 0; s2 < 16; ++s2) Mg = fmaxf(Mg, ms[s2]);
        const float Mu = (Mg == -INFINITY) ? 0.f : Mg;
        float Lg = 0.f, Og = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < 16; ++s2) {
            const float f = (ms[s2] == -INFINITY) ? 0.f : expf(ms[s2] - Mu);
            Lg += ls[s2] * f;
            Og += os[s2] * f;
        }
        p.out[head * DEC_D + tid] = __float2half_rn(Lg > 0.f ? Og / Lg : 0.f);
    } else if (tid < DEC_D) {
        const float* base = p.partial + (long long)head * p.splits * (DEC_D + 2);
        float Mg = -INFINITY;
        for (int s2 = 0; s2 < p.splits; ++s2) Mg = fmaxf(Mg, __ldcg(base + s2 * (DEC_D + 2)));
        const float Mu = (Mg == -INFINITY) ? 0.f : Mg;
        float Lg = 0.f, Og = 0.f;
        for (int s2 = 0; s2 < p.splits; ++s2) {
            const float ms = __ldcg(base + s2 * (DEC_D + 2));
            const float f = (ms == -INFINITY) ? 0.f : expf(ms - Mu);
            Lg += __ldcg(base + s2 * (DEC_D + 2) + 1) * f;
            Og += __ldcg(base + s2 * (DEC_D + 2) + 2 + tid) * f;
        }
        p.out[head * DEC_D + tid] = __float2half_rn(Lg > 0.f ? Og / Lg : 0.f);
    }
    if (tid == 0) p.counters[head] = 0;  // ready for the next launch
}

// The same decode attention for a batched step with enough (head, request) pairs to fill the machine by themselves
// (8 requests x 32 heads = 256 CTAs): ONE CTA per pair walks all of its keys, so nothing is merged across CTAs: no
// partials in global memory, no fence, no ticket, no last-arriver round.  8 warps; a lane group of 8 lanes x 16 B
// covers a key row, a warp 4 keys per load instruction, the CTA 128 keys per turn; every lane keeps the loads of
// the NEXT turn (4 K + 4 V rows) in flight while it works on the current one (two register buffers, the loop is
// unrolled by two).  Each lane group carries a running (max, sum, 8 output dims) over its keys; the 32 groups of the
// CTA meet once through shared memory at the end.  Fused form only (q / new k / new v from the qkv row, rope in-kernel,
// append to the cache, position from device memory).
constexpr int LOOP_WARPS = 8, LOOP_ITER = 4, LOOP_KEYS = LOOP_WARPS * 4 * LOOP_ITER;   // 128 keys per turn

__global__ void __launch_bounds__(LOOP_WARPS * 32, 2)
sdpa_decode_loop_kernel(const __grid_constant__ DecodeParams gp) {
    __shared__ float q_s[DEC_D], knew_s[DEC_D], vnew_s[DEC_D], raw_s[DEC_D], rawk_s[DEC_D];
    __shared__ float red_m[LOOP_WARPS * 4], red_l[LOOP_WARPS * 4], red_o[LOOP_WARPS * 4][DEC_D];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head = blockIdx.x, b = blockIdx.y;
    const bool batched = gp.batch > 0;    // one request: cache and position in the scalar fields
    const __half* qrow = gp.q + (batched ? b * gp.q_batch_stride : 0);
    __half* out = gp.out + (batched ? b * gp.out_batch_stride : 0);
    __half* kc = batched ? gp.bk[b] : gp.k_w;
    __half* vc = batched ? gp.bv[b] : gp.v_w;
    const int* pos_ptr = batched ? gp.bpos[b] : gp.pos_ptr;
    const int pos = pos_ptr ? *pos_ptr : gp.pos;   // keys 0 .. pos-1 are in the cache, the new token becomes key pos
    const float scale = 0.125f;           // 1/sqrt(64)
    const int sub = lane & 7, grp = lane >> 3;
    asm volatile("griddepcontrol.launch_dependents;");
    const __half* kh = kc + head * gp.k_head_stride + sub * 8;
    const __half* vh = vc + head * gp.k_head_stride + sub * 8;
    const int key_w = warp * (4 * LOOP_ITER) + grp;   // this lane group's first key of a turn (then +4 per load)

    uint4 ka[LOOP_ITER], va[LOOP_ITER], kb[LOOP_ITER], vb[LOOP_ITER];
    auto request = [&](int key0, uint4 (&kr)[LOOP_ITER], uint4 (&vr)[LOOP_ITER]) {
#pragma unroll
        for (int it = 0; it < LOOP_ITER; ++it) {
            const int key = key0 + key_w + it * 4;
            kr[it] = key < pos ? ldg_nc16(kh + (long long)key * DEC_D) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int it = 0; it < LOOP_ITER; ++it) {
            const int key = key0 + key_w + it * 4;
            vr[it] = key < pos ? ldg_nc16(vh + (long long)key * DEC_D) : make_uint4(0, 0, 0, 0);
        }
    };
    // the cached prefix was written by earlier steps: the first two turns are requested before the dependency wait
    request(0, ka, va);
    request(LOOP_KEYS, kb, vb);
    float2 cs = make_float2(1.f, 0.f);
    if (tid < gp.rot_dim) {
        const int half = gp.rot_dim >> 1, j = tid < half ? tid : tid - half;
        cs = __ldg(reinterpret_cast<const float2*>(gp.rope_tab + ((size_t)pos * half + j) * 2));  // (cos, sin)
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // q, new k, new v of this head from the qkv row; rotate q and k, append k and v to the cache
    const int hd = gp.n_heads * DEC_D;
    if (tid < DEC_D) {
        raw_s[tid] = __half2float(__ldcg(qrow + head * DEC_D + tid));
        rawk_s[tid] = __half2float(__ldcg(qrow + hd + head * DEC_D + tid));
        vnew_s[tid] = __half2float(__ldcg(qrow + 2 * hd + head * DEC_D + tid));
    }
    __syncthreads();
    if (tid < DEC_D) {
        q_s[tid] = md_round_f16(rope_rotate(raw_s, tid, gp.rot_dim, cs));
        const __half kr = __float2half_rn(rope_rotate(rawk_s, tid, gp.rot_dim, cs));
        knew_s[tid] = __half2float(kr);
        kc[head * gp.k_head_stride + (long long)pos * DEC_D + tid] = kr;
        vc[head * gp.k_head_stride + (long long)pos * DEC_D + tid] = __float2half_rn(vnew_s[tid]);
    }
    __syncthreads();
    float qv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) qv[i] = q_s[sub * 8 + i];

    // running state of this lane group over its keys: exponent reference m, sum l, 8 output dims per lane
    float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    auto consume = [&](int key0, const uint4 (&kr)[LOOP_ITER], const uint4 (&vr)[LOOP_ITER]) {
        float sc[LOOP_ITER], mt = -INFINITY;
#pragma unroll
        for (int it = 0; it < LOOP_ITER; ++it) {
            float kf[8];
            unpack8(kr[it], kf);
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) dot = fmaf(qv[i], kf[i], dot);
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            dot += __shfl_xor_sync(0xffffffffu, dot, 4);
            sc[it] = (key0 + key_w + it * 4 < pos) ? dot * scale : -INFINITY;
            mt = fmaxf(mt, sc[it]);
        }
        if (mt > m) {   // the reference of this group moves: rescale what it holds (uniform within the 8 lanes)
            const float corr = (m == -INFINITY) ? 0.f : expf(m - mt);
            l *= corr;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] *= corr;
            m = mt;
        }
        const float mu = (m == -INFINITY) ? 0.f : m;
#pragma unroll
        for (int it = 0; it < LOOP_ITER; ++it) {
            const float pw = expf(sc[it] - mu);   // exp(-inf) = 0 for keys past the cache
            l += pw;
            float vf[8];
            unpack8(vr[it], vf);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(pw, vf[i], acc[i]);
        }
    };
    for (int key0 = 0; key0 < pos; key0 += 2 * LOOP_KEYS) {
        consume(key0, ka, va);
        if (key0 + 2 * LOOP_KEYS < pos) request(key0 + 2 * LOOP_KEYS, ka, va);
        if (key0 + LOOP_KEYS < pos) {
            consume(key0 + LOOP_KEYS, kb, vb);
            if (key0 + 3 * LOOP_KEYS < pos) request(key0 + 3 * LOOP_KEYS, kb, vb);
        }
    }
    // the appended token: lane group 0 of warp 0
    if (warp == 0 && grp == 0) {
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) dot = fmaf(qv[i], knew_s[sub * 8 + i], dot);
        dot += __shfl_xor_sync(0x000000ffu, dot, 1);
        dot += __shfl_xor_sync(0x000000ffu, dot, 2);
        dot += __shfl_xor_sync(0x000000ffu, dot, 4);
        const float s_new = dot * scale;
        if (s_new > m) {
            const float corr = (m == -INFINITY) ? 0.f : expf(m - s_new);
            l *= corr;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] *= corr;
            m = s_new;
        }
        const float pw = expf(s_new - m);
        l += pw;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(pw, vnew_s[sub * 8 + i], acc[i]);
    }
    // the 32 lane groups of the CTA meet: group g = warp * 4 + grp
    const int g = warp * 4 + grp;
#pragma unroll
    for (int i = 0; i < 8; ++i) red_o[g][sub * 8 + i] = acc[i];
    if (sub == 0) { red_m[g] = m; red_l[g] = l; }
    __syncthreads();
    if (tid < DEC_D) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < LOOP_WARPS * 4; ++w) M = fmaxf(M, red_m[w]);
        const float Mu = (M == -INFINITY) ? 0.f : M;
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < LOOP_WARPS * 4; ++w) {
            const float f = (red_m[w] == -INFINITY) ? 0.f : expf(red_m[w] - Mu);
            L += red_l[w] * f;
            O += red_o[w][tid] * f;
        }
        out[head * DEC_D + tid] = __float2half_rn(L > 0.f ? O / L : 0.f);
    }
}

// qkv [S, 3*H*d] -> rotated q [S, H*d], rotated k and raw v appended to the cache at pos..pos+S-1,
// 8 dims (16 bytes) per thread: thread -> (row s, head h, 8-dim piece c).  A rotated piece needs its
// partner piece half a rotary width away; both are single 16-byte loads.  Needs d % 8 == 0 and rot_dim % 16 == 0.
__global__ void __launch_bounds__(256)
rope_cache_write_vec_kernel(const __half* __restrict__ qkv, __half* __restrict__ q_rot, __half* __restrict__ kc,
                            __half* __restrict__ vc, int S, int H, int d, int max_seq, int pos, int rot_dim,
                            const float* __restrict__ tab) {
    md_pdl_launch_dependents();
    md_pdl_wait();
    const int pieces = d >> 3, hd = H * d, half = rot_dim >> 1;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)S * H * pieces) return;
    const int c = (int)(idx % pieces), h = (int)((idx / pieces) % H), s = (int)(idx / ((long long)pieces * H));
    const int dd0 = c * 8;
    const __half* row = qkv + (long long)s * 3 * hd + h * d;
    auto ld8 = [](const __half* p, float (&f)[8]) {
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const __half2* hh = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 x = __half22float2(hh[i]);
            f[2 * i] = x.x;
            f[2 * i + 1] = x.y;
        }
    };
    auto st8 = [](__half* p, const float (&f)[8]) {
        uint4 u;
        __half2* hh = reinterpret_cast<__half2*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) hh[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = u;
    };
    const long long cidx = ((long long)h * max_seq + pos + s) * d + dd0;
    *reinterpret_cast<uint4*>(vc + cidx) = *reinterpret_cast<const uint4*>(row + 2 * hd + dd0);
    if (dd0 >= rot_dim) {
        *reinterpret_cast<uint4*>(q_rot + (long long)s * hd + h * d + dd0) = *reinterpret_cast<const uint4*>(row + dd0);
        *reinterpret_cast<uint4*>(kc + cidx) = *reinterpret_cast<const uint4*>(row + hd + dd0);
        return;
    }
    const bool lower = dd0 < half;
    const int j0 = lower ? dd0 : dd0 - half, partner = lower ? dd0 + half : dd0 - half;
    float q[8], qp[8], k[8], kp[8], qo[8], ko[8];
    ld8(row + dd0, q);
    ld8(row + partner, qp);
    ld8(row + hd + dd0, k);
    ld8(row + hd + partner, kp);
    const float2* cs = reinterpret_cast<const float2*>(tab + ((size_t)(pos + s) * half + j0) * 2);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float cc = cs[i].x, sn = cs[i].y;
        // lower half: x[j] * cos - x[j + half] * sin; upper half: x[j] * sin + x[j + half] * cos (rope.zig:130-216)
        qo[i] = lower ? q[i] * cc - qp[i] * sn : qp[i] * sn + q[i] * cc;
        ko[i] = lower ? k[i] * cc - kp[i] * sn : kp[i] * sn + k[i] * cc;
    }
    st8(q_rot + (long long)s * hd + h * d + dd0, qo);
    st8(kc + cidx, ko);
}

// The same step one element per thread iteration, for head dims or rotary widths the vector form cannot take.
__global__ void __launch_bounds__(128)
rope_cache_write_kernel(const __half* __restrict__ qkv, __half* __restrict__ q_rot, __half* __restrict__ kc,
                        __half* __restrict__ vc, int S, int H, int d, int max_seq, int pos, int rot_dim,
                        const float* __restrict__ tab) {
    md_pdl_launch_dependents();
    md_pdl_wait();
    const int s = blockIdx.x, hd = H * d;
    const __half* row = qkv + (long long)s * 3 * hd;
    const int half = rot_dim / 2;
    for (int idx = threadIdx.x; idx < hd; idx += blockDim.x) {
        const int h = idx / d, dd = idx % d;
        float qo, ko;
        if (dd < rot_dim) {
            const int j = dd < half ? dd : dd - half;
            const float2 cs = *reinterpret_cast<const float2*>(tab + ((size_t)(pos + s) * half + j) * 2);
            const float c = cs.x, sn = cs.y;
            const float qr = __half2float(row[h * d + j]), qi = __half2float(row[h * d + j + half]);
            const float kr = __half2float(row[hd + h * d + j]), ki = __half2float(row[hd + h * d + j + half]);
            qo = dd < half ? qr * c - qi * sn : qr * sn + qi * c;
            ko = dd < half ? kr * c - ki * sn : kr * sn + ki * c;
        } else {
            qo = __half2float(row[idx]);
            ko = __half2float(row[hd + idx]);
        }
        q_rot[(long long)s * hd + idx] = __float2half_rn(qo);
        const long long cidx = ((long long)h * max_seq + pos + s) * d + dd;
        kc[cidx] = __float2half_rn(ko);
        vc[cidx] = row[2 * hd + idx];
    }
}

}  // namespace

int md_launch_sdpa(md_ctx* ctx, const __half* q, const __half* k, const __half* v, const uint8_t* mask, __half* out,
                   size_t n_heads, size_t q_len, size_t kv_len, size_t d, size_t q_row, size_t q_head, size_t kv_row,
                   size_t kv_head, size_t o_row, size_t o_head, size_t batch, size_t q_batch, size_t kv_batch,
                   size_t o_batch, int causal_pos) {
    if (d == 0 || d > 256) return md_fail(ctx, MD_ERR_UNSUPPORTED, "head_dim %zu not supported (1..256)", d);
    SdpaParams p;
    p.q = q; p.k = k; p.v = v; p.out = out; p.mask = mask;
    p.q_len = (int)q_len; p.kv_len = (int)kv_len;
    p.q_row = (long long)q_row; p.q_head = (long long)q_head; p.q_batch = (long long)q_batch;
    p.kv_row = (long long)kv_row; p.kv_head = (long long)kv_head; p.kv_batch = (long long)kv_batch;
    p.o_row = (long long)o_row; p.o_head = (long long)o_head; p.o_batch = (long long)o_batch;
    p.causal_pos = causal_pos;
    const float scale = 1.0f / sqrtf((float)d);
    p.scale_log2 = scale * LOG2E;
    auto aligned = [](const void* ptr, size_t a, size_t b, size_t c) {
        return (reinterpret_cast<uintptr_t>(ptr) % 16 == 0) && (a % 8 == 0) && (b % 8 == 0) && (c % 8 == 0);
    };
    const bool vec_ok = aligned(q, q_row, q_head, q_batch) && aligned(k, kv_row, kv_head, kv_batch) &&
                        aligned(v, kv_row, kv_head, kv_batch) && (reinterpret_cast<uintptr_t>(out) % 4 == 0) &&
                        (o_row % 2 == 0) && (o_head % 2 == 0) && (o_batch % 2 == 0);
    // tcgen05 path (attention_tc.cu) for the shapes with enough rows to fill its 128-query tiles
    if (ctx->attn_tc != 0 && q_len > 0 && kv_len > 0 &&
        md_sdpa_tc_supported(q, k, v, out, d, q_row, q_head, q_batch, kv_row, kv_head, kv_batch, o_row, o_head, o_batch,
                             n_heads, batch) &&
        (ctx->attn_tc == 1 || q_len > 64))
        return md_launch_sdpa_tc(ctx, q, k, v, mask, out, n_heads, q_len, kv_len, d, q_row, q_head, kv_row, kv_head, o_row,
                                 o_head, batch, q_batch, kv_batch, o_batch, causal_pos);
    if (ctx->attn_tc == 1) return md_fail(ctx, MD_ERR_UNSUPPORTED, "attn_tc forced but the operands are not addressable");
    if ((d == 64 || d == 72) && vec_ok) {
        dim3 grid((unsigned)((q_len + BQ - 1) / BQ), (unsigned)n_heads, (unsigned)batch);
        // Q + 2 x (K, V) tiles of 64 rows; above the 48 KB default for d = 72, so opt in once
        const int smem64 = (BQ + 4 * BKV) * (64 + 8) * 2, smem72 = (BQ + 4 * BKV) * (80 + 8) * 2;
        // the attribute belongs to the device the context lives on: remembered per context, not per process
        if (!ctx->sdpa_mma_configured) {
            MD_CUDA(ctx, cudaFuncSetAttribute(sdpa_mma_kernel<64, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem64));
            MD_CUDA(ctx, cudaFuncSetAttribute(sdpa_mma_kernel<72, 80>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem72));
            ctx->sdpa_mma_configured = true;
        }
        if (d == 64) return md_launch_ex(ctx, sdpa_mma_kernel<64, 64>, grid, dim3(128), smem64, "sdpa_mma_kernel", p);
        return md_launch_ex(ctx, sdpa_mma_kernel<72, 80>, grid, dim3(128), smem72, "sdpa_mma_kernel", p);
    }
    const size_t warps = q_len * n_heads;
    dim3 grid((unsigned)((warps + 3) / 4), (unsigned)batch);
    sdpa_generic_kernel<<<grid, 128, 0, ctx->stream>>>(p, (int)d, (int)n_heads, scale);
    MD_LAUNCH_CHECK(ctx, "sdpa_generic_kernel");
    return MD_OK;
}

// One CTA per (head, request) walking all keys of its head: taken when there are enough such pairs to fill the
// machine (option decode_loop), fused form only.
static bool decode_loop_wanted(const md_ctx* ctx, const DecodeParams& p, size_t batch) {
    if (ctx->decode_loop == 0 || !p.fused || p.rot_dim > DEC_D) return false;
    if (ctx->decode_loop < 0 && batch < 2) return false;   // a single request keeps the key splits unless asked
    return batch * (size_t)p.n_heads >= (size_t)(ctx->decode_loop > 0 ? ctx->decode_loop : 128);
}

static int decode_loop_launch(md_ctx* ctx, const DecodeParams& p, size_t batch) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.n_heads, (unsigned)batch);
    cfg.blockDim = dim3(LOOP_WARPS * 32);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    const cudaError_t le = cudaLaunchKernelEx(&cfg, sdpa_decode_loop_kernel, p);
    if (le != cudaSuccess)
        return md_fail(ctx, MD_ERR_CUDA, "launch of sdpa_decode_loop_kernel failed: %s", cudaGetErrorString(le));
    MD_LAUNCH_CHECK(ctx, "sdpa_decode_loop_kernel");
    return MD_OK;
}

static int decode_launch(md_ctx* ctx, DecodeParams& p) {
    if (decode_loop_wanted(ctx, p, 1)) return decode_loop_launch(ctx, p, 1);
    p.splits = (p.kv_cache_len + DEC_KEYS - 1) / DEC_KEYS;
    if (p.splits < 1) p.splits = 1;
    const size_t partial_bytes = (size_t)p.n_heads * p.splits * (DEC_D + 2) * sizeof(float);
    void* scratch = nullptr;
    MD_TRY(md_scratch(ctx, partial_bytes, &scratch));
    p.counters = ctx->counters;
    p.partial = reinterpret_cast<float*>(scratch);
    dim3 grid((unsigned)p.splits, (unsigned)p.n_heads);
    sdpa_decode_kernel<false><<<grid, DEC_WARPS * 32, 0, ctx->stream>>>(p);
    MD_LAUNCH_CHECK(ctx, "sdpa_decode_kernel");
    return MD_OK;
}

int md_launch_sdpa_single(md_ctx* ctx, const __half* q, const __half* k, const __half* v, const uint8_t* mask,
                          __half* out, size_t kv_len) {
    DecodeParams p{};
    p.q = q; p.k = k; p.v = v; p.k_w = nullptr; p.v_w = nullptr; p.mask = mask; p.out = out;
    p.k_head_stride = (long long)kv_len * DEC_D;
    p.n_heads = 32; p.kv_cache_len = (int)kv_len; p.fused = 0; p.pos = 0; p.rot_dim = 0; p.theta = 0.f;
    return decode_launch(ctx, p);
}

int md_launch_sdpa_decode_fused(md_ctx* ctx, const __half* qkv_row, __half* kc, __half* vc, __half* out,
                                size_t n_heads, size_t d, size_t max_seq, size_t pos, size_t rot_dim, float theta) {
    if (d != DEC_D || n_heads > 256)
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "decode attention supports head_dim 64 and <= 256 heads");
    DecodeParams p{};
    p.q = qkv_row; p.k = kc; p.v = vc; p.k_w = kc; p.v_w = vc; p.mask = nullptr; p.out = out;
    p.k_head_stride = (long long)max_seq * DEC_D;
    p.n_heads = (int)n_heads; p.kv_cache_len = (int)pos; p.fused = 1; p.pos = (int)pos; p.rot_dim = (int)rot_dim;
    p.theta = theta;
    MD_TRY(md_rope_cached(ctx, rot_dim, theta, max_seq, &p.rope_tab));
    return decode_launch(ctx, p);
}

// The decode attention of `batch` requests (1..8) in one launch: request b reads row b of qkv (row stride
// qkv_stride elements), appends to and reads its own cache kc[b] / vc[b] at the position held in pos_dev[b],
// and writes row b of out (row stride out_stride).
int md_launch_sdpa_decode_fused_devpos_batch(md_ctx* ctx, const __half* qkv, size_t qkv_stride, __half* const* kc,
                                             __half* const* vc, __half* out, size_t out_stride, size_t batch,
                                             size_t n_heads, size_t d, size_t max_seq, const int* const* pos_dev,
                                             size_t rot_dim, float theta) {
    if (d != DEC_D || n_heads > 256)
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "decode attention supports head_dim 64 and <= 256 heads");
    if (batch < 1 || batch > 8) return md_fail(ctx, MD_ERR_INVALID_ARG, "decode attention: batch must be 1..8");
    DecodeParams p{};
    p.q = qkv; p.k = kc[0]; p.v = vc[0]; p.k_w = kc[0]; p.v_w = vc[0]; p.mask = nullptr; p.out = out;
    p.k_head_stride = (long long)max_seq * DEC_D;
    p.n_heads = (int)n_heads; p.fused = 1; p.rot_dim = (int)rot_dim; p.theta = theta;
    MD_TRY(md_rope_cached(ctx, rot_dim, theta, max_seq, &p.rope_tab));
    p.pos_ptr = pos_dev[0];
    if (batch > 1) {
        p.batch = (int)batch;
        p.q_batch_stride = (long long)qkv_stride;
        p.out_batch_stride = (long long)out_stride;
        for (size_t b = 0; b < batch; ++b) { p.bk[b] = kc[b]; p.bv[b] = vc[b]; p.bpos[b] = pos_dev[b]; }
    }
    if (decode_loop_wanted(ctx, p, batch)) return decode_loop_launch(ctx, p, batch);
    const int max_splits = (int)((max_seq + DEC_KEYS - 1) / DEC_KEYS);
    if (ctx->decode_cluster_ok < 0) {
        const cudaError_t ce =
            cudaFuncSetAttribute(sdpa_decode_kernel<true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (ce != cudaSuccess) cudaGetLastError();
        ctx->decode_cluster_ok = ce == cudaSuccess ? 1 : 0;
    }
    if (ctx->decode_cluster_mode >= 0) ctx->decode_cluster_ok = ctx->decode_cluster_ok && ctx->decode_cluster_mode;
    // Two ways to merge the key splits of a head: through global scratch with an arrival ticket (the default), or,
    // with md_set_option("decode_cluster", 1), through the shared memory of a 16-CTA thread-block cluster (one CTA
    // per possible split; needs the non-portable cluster size and at most 16 splits).  The cluster form measured
    // slower inside the two-chain decode layer (864 against 784 us per token at 24 layers): its CTAs past the live
    // splits hold their slots until the cluster barrier, and 16-CTA clusters start at a limited rate.
    const bool use_cluster = ctx->decode_cluster_ok && max_splits <= 16 && ctx->decode_cluster_mode == 1;
    if (!use_cluster && batch * n_heads > MD_COUNTER_WORDS)
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "decode attention: batch * n_heads exceeds the arrival counters");
    void* scratch = nullptr;
    MD_TRY(md_scratch(ctx, batch * p.n_heads * max_splits * (DEC_D + 2) * sizeof(float), &scratch));
    p.counters = ctx->counters;
    p.partial = reinterpret_cast<float*>(scratch);
    p.splits = max_splits;  // stride of the partial array; the kernel recomputes the live count
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)max_splits, (unsigned)p.n_heads, (unsigned)batch);
    cfg.blockDim = dim3(DEC_WARPS * 32);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (use_cluster) {
        cfg.gridDim = dim3(16u, (unsigned)p.n_heads, (unsigned)batch);
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 16;
        attr[na].val.clusterDim.y = 1;
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
    const cudaError_t le = use_cluster ? cudaLaunchKernelEx(&cfg, sdpa_decode_kernel<true>, p)
                                       : cudaLaunchKernelEx(&cfg, sdpa_decode_kernel<false>, p);
    if (le != cudaSuccess) return md_fail(ctx, MD_ERR_CUDA, "launch of sdpa_decode_kernel failed: %s", cudaGetErrorString(le));
    MD_LAUNCH_CHECK(ctx, "sdpa_decode_kernel");
    return MD_OK;
}

int md_launch_sdpa_decode_fused_devpos(md_ctx* ctx, const __half* qkv_row, __half* kc, __half* vc, __half* out,
                                       size_t n_heads, size_t d, size_t max_seq, const int* pos_dev, size_t rot_dim,
                                       float theta) {
    return md_launch_sdpa_decode_fused_devpos_batch(ctx, qkv_row, 0, &kc, &vc, out, 0, 1, n_heads, d, max_seq, &pos_dev,
                                                    rot_dim, theta);
}

int md_launch_rope_cache_write(md_ctx* ctx, const __half* qkv, __half* q_rot, __half* kc, __half* vc, size_t S,
                               size_t n_heads, size_t d, size_t max_seq, size_t pos, size_t rot_dim, float theta) {
    if (S == 0) return MD_OK;
    const float* tab = nullptr;
    MD_TRY(md_rope_cached(ctx, rot_dim, theta, max_seq, &tab));
    const bool vec = (d % 8) == 0 && (rot_dim % 16) == 0 &&
                     ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_rot) | reinterpret_cast<uintptr_t>(kc) |
                       reinterpret_cast<uintptr_t>(vc)) & 15) == 0;
    if (vec) {
        const size_t units = S * n_heads * (d / 8);
        MD_TRY(md_launch_ex(ctx, rope_cache_write_vec_kernel, dim3((unsigned)((units + 255) / 256)), dim3(256), 0,
                            "rope_cache_write_vec_kernel", qkv, q_rot, kc, vc, (int)S, (int)n_heads, (int)d, (int)max_seq,
                            (int)pos, (int)rot_dim, tab));
    } else {
        MD_TRY(md_launch_ex(ctx, rope_cache_write_kernel, dim3((unsigned)S), dim3(128), 0, "rope_cache_write_kernel", qkv,
                            q_rot, kc, vc, (int)S, (int)n_heads, (int)d, (int)max_seq, (int)pos, (int)rot_dim, tab));
    }
    return MD_OK;
}

// ------------------------------------------------------------------------------------------
// md_sdpa_single_noalloc: the decode attention above for callers that must not allocate.
//
// Some hosts cannot call cudaMalloc once they are running: a serving process that handed all of
// HBM to its own arena at start-up (weights + KV caches for as many requests as fit) gets
// cudaErrorMemoryAllocation from any later cudaMalloc, and a latency-critical decode loop cannot
// afford the implicit device-wide synchronisation of cudaMalloc/cudaFree.  The regular entry point
// needs a context (whose creation allocates a stream, flags and scratch).  This one needs nothing:
// the split-KV partials and the per-head arrival counters live in the file-scope device array
// below, which every GPU that loads this library holds from module load until process exit.
//
// Limits and rules:
//   * fixed geometry of the reference's decode attention: 32 heads x 64 dims, kv_len <= 2048,
//     hence at most 16 splits; the array is 256 B of counters + 32*16*66 floats = 135,424 bytes.
//   * device pointers only (a host pointer cannot be staged without allocating).
//   * the tensors must live on the current device (checked; a mismatch is MD_ERR_INVALID_ARG).
//   * the first call on a device resolves the array's device address (cudaGetSymbolAddress with that
//     device current).  That first call is set-up work: make it before any stream capture begins, and
//     make it at start-up, before the host reserves the rest of HBM: when the CUDA runtime loads modules
//     lazily, the first use of this library's kernels on a device is what places its code and this array
//     in device memory.
//   * all calls on a device share the one array, which keeps the previous call's contents.  The
//     counters are cleared on the stream before every launch; the partials need no clearing (every
//     slot that is read was written by the same launch).  Two calls that overlap on the GPU (different
//     streams, no dependency between them) race on the array: serialise them.
namespace {

constexpr size_t NOALLOC_MAX_KV = 2048;
constexpr size_t NOALLOC_COUNTER_BYTES = 256;
constexpr size_t NOALLOC_PARTIAL_BYTES = 32 * (NOALLOC_MAX_KV / DEC_KEYS) * (DEC_D + 2) * sizeof(float);
constexpr size_t NOALLOC_BYTES = NOALLOC_COUNTER_BYTES + NOALLOC_PARTIAL_BYTES;
constexpr int NOALLOC_MAX_DEVICES = 64;

static __device__ __align__(256) unsigned char md_noalloc_scratch[NOALLOC_BYTES];

// In host code the name md_noalloc_scratch is only a handle for the runtime, not an address a
// kernel can use; the usable device address is looked up once per device and kept here.
static void* g_noalloc_addr[NOALLOC_MAX_DEVICES] = {};

static int noalloc_fail(int status, char* err, size_t cap, const char* fmt, ...) {
    if (err && cap) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, cap, fmt, ap);
        va_end(ap);
    }
    return status;
}

}  // namespace

extern "C" int md_sdpa_single_noalloc(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint8_t* mask,
                                      uint16_t* out, size_t kv_len, void* cuda_stream, char* err, size_t err_cap) {
    if (err && err_cap) err[0] = '\0';
    if (!q || !k || !v || !mask || !out)
        return noalloc_fail(MD_ERR_INVALID_ARG, err, err_cap, "md_sdpa_single_noalloc: null tensor pointer");
    if (kv_len == 0)
        return noalloc_fail(MD_ERR_INVALID_ARG, err, err_cap, "md_sdpa_single_noalloc: kv_len is 0");
    if (kv_len > NOALLOC_MAX_KV)
        return noalloc_fail(MD_ERR_SEQUENCE_TOO_LONG, err, err_cap,
                            "md_sdpa_single_noalloc: kv_len %zu exceeds the built-in scratch (max %zu keys)", kv_len,
                            NOALLOC_MAX_KV);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES)
        return noalloc_fail(MD_ERR_CUDA, err, err_cap, "md_sdpa_single_noalloc: cudaGetDevice: %s",
                            e != cudaSuccess ? cudaGetErrorString(e) : "device index out of range");
    const void* ptrs[5] = {q, k, v, mask, out};
    for (const void* p : ptrs) {
        cudaPointerAttributes attr;
        if (cudaPointerGetAttributes(&attr, p) != cudaSuccess ||
            (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged)) {
            cudaGetLastError();
            return noalloc_fail(MD_ERR_INVALID_ARG, err, err_cap,
                                "md_sdpa_single_noalloc: every tensor must be device memory (host buffers would "
                                "need a staging allocation)");
        }
        // The kernel runs on the current device with that device's copy of the scratch array; a tensor that lives
        // on another GPU would be dereferenced there without a peer mapping.  Managed memory migrates, so it passes.
        if (attr.type == cudaMemoryTypeDevice && attr.device != dev)
            return noalloc_fail(MD_ERR_INVALID_ARG, err, err_cap,
                                "md_sdpa_single_noalloc: a tensor lives on device %d but device %d is current; make the "
                                "tensors' device current before the call",
                                attr.device, dev);
    }
    if (!g_noalloc_addr[dev]) {
        void* addr = nullptr;
        e = cudaGetSymbolAddress(&addr, md_noalloc_scratch);  // the current device's instance of the array
        if (e != cudaSuccess || !addr)
            return noalloc_fail(MD_ERR_CUDA, err, err_cap, "md_sdpa_single_noalloc: cudaGetSymbolAddress: %s",
                                cudaGetErrorString(e));
        g_noalloc_addr[dev] = addr;
    }
    unsigned char* base = static_cast<unsigned char*>(g_noalloc_addr[dev]);
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    e = cudaMemsetAsync(base, 0, NOALLOC_COUNTER_BYTES, stream);
    if (e != cudaSuccess)
        return noalloc_fail(MD_ERR_CUDA, err, err_cap, "md_sdpa_single_noalloc: cudaMemsetAsync: %s",
                            cudaGetErrorString(e));
    DecodeParams p{};
    p.q = reinterpret_cast<const __half*>(q);
    p.k = reinterpret_cast<const __half*>(k);
    p.v = reinterpret_cast<const __half*>(v);
    p.k_w = nullptr;
    p.v_w = nullptr;
    p.mask = mask;
    p.out = reinterpret_cast<__half*>(out);
    p.k_head_stride = (long long)kv_len * DEC_D;
    p.n_heads = 32;
    p.kv_cache_len = (int)kv_len;
    p.fused = 0;
    p.splits = (int)((kv_len + DEC_KEYS - 1) / DEC_KEYS);
    p.counters = reinterpret_cast<unsigned int*>(base);
    p.partial = reinterpret_cast<float*>(base + NOALLOC_COUNTER_BYTES);
    sdpa_decode_kernel<false><<<dim3((unsigned)p.splits, 32u), DEC_WARPS * 32, 0, stream>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess)
        return noalloc_fail(MD_ERR_CUDA, err, err_cap, "md_sdpa_single_noalloc: launch failed: %s",
                            cudaGetErrorString(e));
    return MD_OK;
}
