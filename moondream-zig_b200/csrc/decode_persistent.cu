// One decoder step (text_model.zig:117-345: 24 x [LayerNorm -> qkv, fc1 | attention | out-proj, fc2,
// residuals] -> final LayerNorm -> lm_head -> greedy argmax) as ONE persistent kernel.
//
// A decode step streams every weight once (2.6 GB) and does almost no arithmetic, so its time is the time
// HBM is kept busy.  As 74 dependent kernels every boundary drains and refills the memory pipeline; here
// one CTA per SM lives for the whole step and the boundaries become grid-wide barriers that the weight
// stream does not take part in:
//   warp 0       producer: walks a static schedule of weight tiles (8 rows x 2048 halves, one 4 KB bulk
//                copy per row, global -> shared, completion on an mbarrier) through a ring of stages.  The
//                schedule depends on nothing computed in the step, so the producer runs ahead across the
//                barriers and through the attention phase: the ring (166 KB per SM, 24 MB in flight over
//                the GPU) is full of the next phase's weights when the consumers arrive there.
//   warps 1..8   consumers: each takes a 256-wide k slice of every tile; the dot products run as
//                mma.sync.m16n8k16 with the 8 weight rows in both halves of the A fragment (two consecutive
//                32-wide k slabs) and the <= 8 activation rows on the N side; partial sums meet in shared
//                memory; the epilogues reproduce the reference's f16 roundings (f16(acc) -> +bias -> GELU ->
//                residual adds, one rounding each).
// Rows are split evenly over the CTAs at a granularity of one row (a tile may hold fewer than 8 rows: only
// those are fetched), so every SM streams the same number of bytes in every phase.
// Attention (attention.zig:236-414, one query per request): a warp owns one (request, head, 32-key split):
// it rotates q, reads its keys and values straight from the cache, the warp of the last split also rotates
// and appends the new key / value; partial (max, sum, out) go to scratch and the last warp to finish a head
// (atomic ticket) merges them.
// The grid barrier is a monotonic counter in global memory; every spin (barrier, mbarrier) is bounded, sets
// the context's error word when it gives up and lets every CTA run to its end.  The kernel is launched
// cooperatively (all CTAs co-resident), which the barrier requires.
#include "md_internal.cuh"
#include "tc_common.cuh"
#include "decode_persistent.cuh"

namespace {

using namespace tc;

constexpr int PD = 2048, PF = 8192, PH = 32, PHD = 64, PROT = 32;  // Phi-1.5 geometry this kernel is built for
constexpr int QKV_ROWS = 3 * PD, A_ROWS = QKV_ROWS + PF;            // phase A: 14336 weight rows of 2048
constexpr int P_STAGES = 5;
constexpr int ROW_PITCH = 4096 + 64;            // bytes; +64 keeps the 8 rows of a fragment read on distinct banks
constexpr int STAGE_BYTES = 8 * ROW_PITCH;      // 33280
constexpr int XS_PITCH = PD + 32;               // halves, same bank argument
constexpr int CONSUMERS = 256, P_THREADS = CONSUMERS + 32;
constexpr int ATT_KEYS = 32;                    // keys per attention unit (one warp): 8 K and 8 V loads in flight per lane
constexpr unsigned long long GRID_WAIT_NS = 1000000000ull;

struct PSmem {
    static constexpr int RING = 0;
    static constexpr int XS = RING + P_STAGES * STAGE_BYTES;         // [8][XS_PITCH] halves
    static constexpr int PARTIAL = XS + 8 * XS_PITCH * 2;            // [2 buffers][8 warps][2 sums][8][8] f32
    static constexpr int RED = PARTIAL + 2 * 8 * 2 * 64 * 4;         // [8 warps] f32 + stat[2]
    static constexpr int BARS = RED + 64;                            // full[5], empty[5]
    static constexpr int MISC = BARS + 2 * 8 * P_STAGES;             // abort flag
    static constexpr int TOTAL = MISC + 16;
};

__device__ __forceinline__ void bulk_load_row(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
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

struct PCtx {
    uint32_t ring, xs, partial, bars;  // shared-memory addresses
    float* partial_ptr;
    float* red_ptr;
    __half* xs_ptr;
    volatile int* abort_flag;
    md_devflags* flags;
    int cw, lane, tc;                  // consumer warp 0..7, lane, consumer thread 0..255
    uint32_t it;                       // stages consumed (or produced) so far: slot = it % P_STAGES
    int pbuf;                          // partial-sum buffer of the next tile
};

__device__ __forceinline__ uint32_t bar_full(const PCtx& c, uint32_t slot) { return c.bars + 8 * slot; }
__device__ __forceinline__ uint32_t bar_empty(const PCtx& c, uint32_t slot) { return c.bars + 8 * (P_STAGES + slot); }

// Grid-wide barrier of the consumer threads (the producers never wait here).  Returns false once the step is
// being abandoned (a wait somewhere ran out of time).
__device__ bool grid_sync(const PCtx& c, unsigned int* counter, unsigned int target) {
    consumer_sync();
    if (c.tc == 0) {
        if (!*c.abort_flag) {
            __threadfence();
            atomicAdd(counter, 1u);
            const unsigned long long t0 = global_ns();
            unsigned spin = 0;
            while (ld_acquire_u32(counter) < target) {
                if ((++spin & 255u) == 0u) {
                    const bool failed_elsewhere = *reinterpret_cast<volatile unsigned int*>(&c.flags->error) != 0u;
                    if (failed_elsewhere || global_ns() - t0 > GRID_WAIT_NS) {
                        if (atomicOr(&c.flags->error, 1u) == 0u) c.flags->where = 40;
                        *c.abort_flag = 1;
                        break;
                    }
                }
            }
            __threadfence();
        }
        // one thread decides for all 256, so that they leave (or stay) together
        c.red_ptr[15] = *c.abort_flag ? 0.f : 1.f;
    }
    consumer_sync();
    return c.red_ptr[15] != 0.f;
}

// LayerNorm (ops.zig layerNorm: two-pass f32, one rounding to f16) of the M rows of `hidden` into xs;
// rows M..7 of xs are zero.  256 consumer threads, 8 elements each.
__device__ void layernorm_to_smem(const PCtx& c, const __half* hidden, const __half* ln_w, const __half* ln_b, int M,
                                  float eps) {
    const uint4 gw = ldnc128(ln_w + c.tc * 8), gb = ldnc128(ln_b + c.tc * 8);
    float wv[8], bv[8];
    unpack8(gw, wv);
    unpack8(gb, bv);
    float* red = c.red_ptr;  // [8] partials, [8..9] results
    for (int m = 0; m < 8; ++m) {
        uint4 o = make_uint4(0, 0, 0, 0);
        if (m < M) {
            const uint4 u = ldcg128(hidden + (size_t)m * PD + c.tc * 8);
            float v[8];
            unpack8(u, v);
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) s += v[2 * i] + v[2 * i + 1];
            auto block_sum = [&](float x, int slot) {
#pragma unroll
                for (int off = 16; off; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
                if (c.lane == 0) red[c.cw] = x;
                consumer_sync();
                if (c.tc == 0) {
                    float a = 0.f;
#pragma unroll
                    for (int w = 0; w < 8; ++w) a += red[w];
                    red[8 + slot] = a;
                }
                consumer_sync();
                return red[8 + slot];
            };
            const float mean = block_sum(s, 0) * (1.0f / PD);
            float q = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float d = v[i] - mean;
                q += d * d;
            }
            const float var = block_sum(q, 1) * (1.0f / PD);
            const float rstd = 1.0f / sqrtf(var + eps), mean_rstd = mean * rstd;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float y0 = (v[2 * i] * rstd - mean_rstd) * wv[2 * i] + bv[2 * i];
                const float y1 = (v[2 * i + 1] * rstd - mean_rstd) * wv[2 * i + 1] + bv[2 * i + 1];
                oh[i] = __floats2half2_rn(y0, y1);
            }
        }
        *reinterpret_cast<uint4*>(c.xs_ptr + (size_t)m * XS_PITCH + c.tc * 8) = o;
    }
    consumer_sync();
}

// One ring stage (8 weight rows x 2048 k) against the activations: this warp's 256-wide k slice.
// XS: activations from the LayerNorm buffer in shared memory, else from global rows x + g * x_ld.
template <bool XS>
__device__ __forceinline__ void stage_mma(PCtx& c, const __half* x, int x_ld, int M, float (&ae)[4], float (&ao)[4]) {
    const uint32_t slot = c.it % P_STAGES;
    mbar_wait(bar_full(c, slot), (c.it / P_STAGES) & 1u, c.abort_flag, c.flags, 41);
    const int g = c.lane >> 2, t = c.lane & 3;
    const uint32_t wbase = c.ring + slot * STAGE_BYTES + g * ROW_PITCH;
    uint4 lo[4], hi[4], xa[4], xb[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int kk = c.cw * 256 + u * 64 + t * 8;
        lo[u] = lds128(wbase + kk * 2);
        hi[u] = lds128(wbase + (kk + 32) * 2);
        if (XS) {
            xa[u] = lds128(c.xs + (g * XS_PITCH + kk) * 2);
            xb[u] = lds128(c.xs + (g * XS_PITCH + kk + 32) * 2);
        } else if (g < M) {
            xa[u] = ldcg128(x + (size_t)g * x_ld + kk);
            xb[u] = ldcg128(x + (size_t)g * x_ld + kk + 32);
        } else {
            xa[u] = xb[u] = make_uint4(0, 0, 0, 0);
        }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        mma_16816(ae, lo[u].x, hi[u].x, lo[u].y, hi[u].y, xa[u].x, xa[u].y);
        mma_16816(ae, lo[u].z, hi[u].z, lo[u].w, hi[u].w, xa[u].z, xa[u].w);
        mma_16816(ao, lo[u].x, hi[u].x, lo[u].y, hi[u].y, xb[u].x, xb[u].y);
        mma_16816(ao, lo[u].z, hi[u].z, lo[u].w, hi[u].w, xb[u].z, xb[u].w);
    }
    __syncwarp();
    if (c.lane == 0) mbar_arrive(bar_empty(c, slot));
    ++c.it;
}

// partial[buf][warp][sum][row][m]: valid halves are rows 0-7 of the "even" accumulators (c0, c1) and rows
// 8-15 of the "odd" ones (c2, c3)
__device__ __forceinline__ void store_partial(const PCtx& c, int sum, const float (&ae)[4], const float (&ao)[4]) {
    const int g = c.lane >> 2, t = c.lane & 3;
    float* dst = c.partial_ptr + (((c.pbuf * 8 + c.cw) * 2 + sum) * 8 + g) * 8 + 2 * t;
    dst[0] = ae[0] + ao[2];
    dst[1] = ae[1] + ao[3];
}
__device__ __forceinline__ float load_partial_sum(const PCtx& c, int buf, int sum, int rr, int m) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += c.partial_ptr[(((buf * 8 + w) * 2 + sum) * 8 + rr) * 8 + m];
    return s;
}

// ---------------------------------------------------------------------------- consumer side of the phases

// Phase A of a layer: rows [r0, r1) of [Wqkv; Wfc1] against the LayerNorm output in xs.
// qkv rows: f16(acc) + bias; fc1 rows: the same, then GELU (text_model.zig:131-160).
__device__ void phase_a(PCtx& c, const md_persist_table::Layer& L, const md_persist_params& p, int r0, int r1) {
    for (int r = r0; r < r1; r += 8) {
        float ae[4] = {0.f, 0.f, 0.f, 0.f}, ao[4] = {0.f, 0.f, 0.f, 0.f};
        stage_mma<true>(c, nullptr, 0, p.M, ae, ao);
        store_partial(c, 0, ae, ao);
        consumer_sync();
        if (c.tc < 64) {
            const int m = c.tc >> 3, rr = c.tc & 7, row = r + rr;
            if (m < p.M && row < r1) {
                float val = md_round_f16(load_partial_sum(c, c.pbuf, 0, rr, m));
                if (row < QKV_ROWS) {
                    val = md_round_f16(val + __half2float(L.bqkv[row]));
                    p.qkv[(size_t)m * QKV_ROWS + row] = __float2half_rn(val);
                } else {
                    const int n = row - QKV_ROWS;
                    val = md_round_f16(val + __half2float(L.bfc1[n]));
                    val = md_round_f16(md_gelu_f32(val));
                    p.fc1[(size_t)m * PF + n] = __float2half_rn(val);
                }
            }
        }
        c.pbuf ^= 1;
    }
}

// Phase C: output rows [r0, r1) of the out-projection (k = 2048, one stage) and of fc2 (k = 8192, four
// stages), then attn_out += mlp_out and hidden += attn_out with one f16 rounding each
// (text_model.zig:162-171).
__device__ void phase_c(PCtx& c, const md_persist_table::Layer& L, const md_persist_params& p, int r0, int r1) {
    for (int r = r0; r < r1; r += 8) {
        float a1e[4] = {0.f, 0.f, 0.f, 0.f}, a1o[4] = {0.f, 0.f, 0.f, 0.f};
        float a2e[4] = {0.f, 0.f, 0.f, 0.f}, a2o[4] = {0.f, 0.f, 0.f, 0.f};
        stage_mma<false>(c, p.attn, PD, p.M, a1e, a1o);
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) stage_mma<false>(c, p.fc1 + ch * PD, PF, p.M, a2e, a2o);
        store_partial(c, 0, a1e, a1o);
        store_partial(c, 1, a2e, a2o);
        consumer_sync();
        if (c.tc < 64) {
            const int m = c.tc >> 3, rr = c.tc & 7, n = r + rr;
            if (m < p.M && n < r1) {
                const float s1 = load_partial_sum(c, c.pbuf, 0, rr, m), s2 = load_partial_sum(c, c.pbuf, 1, rr, m);
                const float a = md_round_f16(md_round_f16(s1) + __half2float(L.bout[n]));
                const float mlp = md_round_f16(md_round_f16(s2) + __half2float(L.bfc2[n]));
                const float sum = md_round_f16(a + mlp);
                __half* h = p.hidden + (size_t)m * PD + n;
                *h = __float2half_rn(ldcg_f16(h) + sum);
            }
        }
        c.pbuf ^= 1;
    }
}

// lm_head rows [r0, r1) against the final LayerNorm output in xs: logits and the greedy-argmax key
// (text_model.zig:325-345, sampling.zig:257-273: first strict maximum of the f16 logits).
__device__ void phase_head(PCtx& c, const md_persist_table& T, const md_persist_params& p, int r0, int r1) {
    unsigned long long best = 0ull;
    for (int r = r0; r < r1; r += 8) {
        float ae[4] = {0.f, 0.f, 0.f, 0.f}, ao[4] = {0.f, 0.f, 0.f, 0.f};
        stage_mma<true>(c, nullptr, 0, p.M, ae, ao);
        store_partial(c, 0, ae, ao);
        consumer_sync();
        if (c.tc < 64) {
            const int m = c.tc >> 3, rr = c.tc & 7, n = r + rr;
            if (m < p.M && n < r1) {
                float val = md_round_f16(load_partial_sum(c, c.pbuf, 0, rr, m));
                val = md_round_f16(val + __half2float(T.lm_b[n]));
                p.logits[(size_t)m * p.vocab + n] = __float2half_rn(val);
                const unsigned bits = __float_as_uint(val);
                const unsigned ordered = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
                const unsigned long long key =
                    ((unsigned long long)ordered << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)n);
                best = key > best ? key : best;
            }
        }
        c.pbuf ^= 1;
    }
    if (c.tc < 64) {  // threads m*8 .. m*8+7 hold the candidates of request m: one atomic per CTA and request
#pragma unroll
        for (int o = 4; o; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        const int m = c.tc >> 3;
        if ((c.tc & 7) == 0 && m < p.M && best != 0ull) atomicMax(p.amax + m, best);
    }
}

// ---------------------------------------------------------------------------- attention phase

// Rotary embedding of this lane's 8 dims (dims sub*8 .. sub*8+7 of a head; rope.zig:130-216: the first
// PROT dims rotate as pairs (j, j + PROT/2), the rest pass through), result rounded to f16.
__device__ __forceinline__ void rope8(float (&x)[8], int sub, int pos, const float* tab) {
    float partner[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) partner[i] = __shfl_xor_sync(0xffffffffu, x[i], 2);  // sub 0<->2, 1<->3
    if (sub < 4) {
        const int j0 = (sub & 1) * 8;
        const float4* cs = reinterpret_cast<const float4*>(tab + ((size_t)pos * (PROT / 2) + j0) * 2);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 v = cs[i];  // (cos, sin) of j0 + 2i and j0 + 2i + 1
            const float c0 = v.x, s0 = v.y, c1 = v.z, s1 = v.w;
            if (sub < 2) {  // dd < half: x[j] * cos - x[j + half] * sin
                x[2 * i] = md_round_f16(x[2 * i] * c0 - partner[2 * i] * s0);
                x[2 * i + 1] = md_round_f16(x[2 * i + 1] * c1 - partner[2 * i + 1] * s1);
            } else {        // dd >= half: x[j] * sin + x[j + half] * cos
                x[2 * i] = md_round_f16(partner[2 * i] * s0 + x[2 * i] * c0);
                x[2 * i + 1] = md_round_f16(partner[2 * i + 1] * s1 + x[2 * i + 1] * c1);
            }
        }
    }
}

__device__ void attention_phase(const PCtx& c, const md_persist_table& T, const md_persist_table::Layer& L,
                                const md_persist_params& p) {
    int pos[MD_PERSIST_MAX_BATCH], nsplit[MD_PERSIST_MAX_BATCH], total = 0;
#pragma unroll
    for (int b = 0; b < MD_PERSIST_MAX_BATCH; ++b) {
        pos[b] = 0;
        nsplit[b] = 0;
        if (b < p.M) {
            pos[b] = *T.pos[b];
            nsplit[b] = max(1, (pos[b] + ATT_KEYS - 1) / ATT_KEYS);
            total += PH * nsplit[b];
        }
    }
    const int sub = c.lane & 7, grp = c.lane >> 3;  // 8 lanes x 16 B cover one 128-byte key row, 4 keys at a time
    const float scale = 0.125f;                      // 1/sqrt(64)
    for (int u = c.cw * gridDim.x + blockIdx.x; u < total; u += 8 * gridDim.x) {
        int b = 0, rem = u;
#pragma unroll
        for (int bb = 0; bb < MD_PERSIST_MAX_BATCH - 1; ++bb)
            if (b == bb && rem >= PH * nsplit[bb]) { rem -= PH * nsplit[bb]; b = bb + 1; }
        int my_pos = 0, my_ns = 1;
#pragma unroll
        for (int bb = 0; bb < MD_PERSIST_MAX_BATCH; ++bb)
            if (bb == b) { my_pos = pos[bb]; my_ns = nsplit[bb]; }
        const int head = rem / my_ns, split = rem % my_ns;
        const bool last = split == my_ns - 1;
        const __half* qkv = p.qkv + (size_t)b * QKV_ROWS;
        __half* kc = L.kc[0];
        __half* vc = L.vc[0];
#pragma unroll
        for (int bb = 1; bb < MD_PERSIST_MAX_BATCH; ++bb)
            if (bb == b) { kc = L.kc[bb]; vc = L.vc[bb]; }
        const size_t head_off = (size_t)head * p.max_seq * PHD;

        // keys and values of this split first (cached by earlier steps: nothing to wait for)
        constexpr int ITER = ATT_KEYS / 4;
        uint4 kreg[ITER], vreg[ITER];
        const int key0 = split * ATT_KEYS;
#pragma unroll
        for (int it = 0; it < ITER; ++it) {
            const int key = key0 + it * 4 + grp;
            kreg[it] = key < my_pos ? ldnc128(kc + head_off + (size_t)key * PHD + sub * 8) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int it = 0; it < ITER; ++it) {
            const int key = key0 + it * 4 + grp;
            vreg[it] = key < my_pos ? ldnc128(vc + head_off + (size_t)key * PHD + sub * 8) : make_uint4(0, 0, 0, 0);
        }
        float q[8];
        unpack8(ldcg128(qkv + head * PHD + sub * 8), q);
        rope8(q, sub, my_pos, p.rope_tab);
        float knew[8], vnew[8];
        if (last) {  // warp-uniform
            unpack8(ldcg128(qkv + PD + head * PHD + sub * 8), knew);
            rope8(knew, sub, my_pos, p.rope_tab);
            const uint4 vraw = ldcg128(qkv + 2 * PD + head * PHD + sub * 8);
            unpack8(vraw, vnew);
            if (grp == 0) {  // append to the cache (text_model.zig:143-149)
                uint4 kp;
                __half2* kh = reinterpret_cast<__half2*>(&kp);
#pragma unroll
                for (int i = 0; i < 4; ++i) kh[i] = __floats2half2_rn(knew[2 * i], knew[2 * i + 1]);
                *reinterpret_cast<uint4*>(kc + head_off + (size_t)my_pos * PHD + sub * 8) = kp;
                *reinterpret_cast<uint4*>(vc + head_off + (size_t)my_pos * PHD + sub * 8) = vraw;
            }
        }
        float sc[ITER], m = -INFINITY;
#pragma unroll
        for (int it = 0; it < ITER; ++it) {
            float kf[8];
            unpack8(kreg[it], kf);
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) dot = fmaf(q[i], kf[i], dot);
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            dot += __shfl_xor_sync(0xffffffffu, dot, 4);
            sc[it] = (key0 + it * 4 + grp < my_pos) ? dot * scale : -INFINITY;
            m = fmaxf(m, sc[it]);
        }
        float s_new = -INFINITY;
        if (last) {
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) dot = fmaf(q[i], knew[i], dot);
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            dot += __shfl_xor_sync(0xffffffffu, dot, 4);
            if (grp == 0) {
                s_new = dot * scale;
                m = fmaxf(m, s_new);
            }
        }
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
        const float m_use = (m == -INFINITY) ? 0.f : m;
        float l = 0.f, acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
        for (int it = 0; it < ITER; ++it) {
            const float pw = expf(sc[it] - m_use);  // exp(-inf) = 0 for absent keys
            l += pw;
            float vf[8];
            unpack8(vreg[it], vf);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(pw, vf[i], acc[i]);
        }
        if (last && grp == 0) {
            const float pw = expf(s_new - m_use);
            l += pw;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(pw, vnew[i], acc[i]);
        }
        l += __shfl_xor_sync(0xffffffffu, l, 8);
        l += __shfl_xor_sync(0xffffffffu, l, 16);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 8);
            acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 16);
        }
        __half* out = p.attn + (size_t)b * PD + head * PHD;
        if (my_ns == 1) {  // a single split: the result is final
            if (grp == 0) {
                const float inv = 1.0f / l;
                uint4 o;
                __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int i = 0; i < 4; ++i) oh[i] = __floats2half2_rn(acc[2 * i] * inv, acc[2 * i + 1] * inv);
                *reinterpret_cast<uint4*>(out + sub * 8) = o;
            }
            continue;
        }
        float* part = p.att_scratch + (((size_t)b * PH + head) * p.max_splits + split) * (PHD + 2);
        if (grp == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) part[2 + sub * 8 + i] = acc[i];
            if (sub == 0) { part[0] = m; part[1] = l; }
        }
        __threadfence();
        __syncwarp();
        unsigned ticket = 0;
        if (c.lane == 0) ticket = atomicAdd(p.att_counters + b * PH + head, 1u);
        ticket = __shfl_sync(0xffffffffu, ticket, 0);
        if (ticket == (unsigned)(my_ns - 1)) {  // the last split of this head to finish merges all of them
            __threadfence();
            const float* base = p.att_scratch + ((size_t)b * PH + head) * p.max_splits * (PHD + 2);
            float Mg = -INFINITY;
            for (int s2 = 0; s2 < my_ns; ++s2) Mg = fmaxf(Mg, __ldcg(base + s2 * (PHD + 2)));
            const float Mu = (Mg == -INFINITY) ? 0.f : Mg;
            float Lg = 0.f, o0 = 0.f, o1 = 0.f;
            for (int s2 = 0; s2 < my_ns; ++s2) {
                const float* ps = base + s2 * (PHD + 2);
                const float ms = __ldcg(ps);
                const float f = (ms == -INFINITY) ? 0.f : expf(ms - Mu);
                Lg += __ldcg(ps + 1) * f;
                const float2 ov = __ldcg(reinterpret_cast<const float2*>(ps + 2 + c.lane * 2));
                o0 += ov.x * f;
                o1 += ov.y * f;
            }
            const float inv = 1.0f / Lg;
            *reinterpret_cast<__half2*>(out + c.lane * 2) = __floats2half2_rn(o0 * inv, o1 * inv);
            if (c.lane == 0) p.att_counters[b * PH + head] = 0u;
        }
    }
}

// ---------------------------------------------------------------------------- producer side

struct Producer {
    uint32_t ring, bars, it;
    int lane;
    volatile int* abort_flag;
    md_devflags* flags;

    // One stage: rows row .. row+nv-1, `bytes_per_row` from src(row) each.  Returns false when abandoned.
    template <class SrcOf>
    __device__ __forceinline__ bool stage(int nv, SrcOf src_of) {
        const uint32_t slot = it % P_STAGES, full = bars + 8 * slot, empty = bars + 8 * (P_STAGES + slot);
        mbar_wait(empty, ((it / P_STAGES) & 1u) ^ 1u, abort_flag, flags, 42);
        if (*abort_flag) return false;
        if (lane == 0) mbar_expect_tx(full, (uint32_t)nv * 4096u);
        __syncwarp();
        if (lane < nv) bulk_load_row(ring + slot * STAGE_BYTES + lane * ROW_PITCH, src_of(lane), 4096u, full);
        ++it;
        return true;
    }
};

__device__ void produce_all(Producer& pr, const md_persist_table& T, const md_persist_params& p) {
    const int cta = blockIdx.x, n = gridDim.x;
    int a0, a1, c0, c1, h0, h1;
    row_range(A_ROWS, cta, n, a0, a1);
    row_range(PD, cta, n, c0, c1);
    row_range(p.vocab, cta, n, h0, h1);
    for (int l = 0; l < p.n_layers; ++l) {
        const md_persist_table::Layer& L = T.layers[l];
        const __half *wqkv = L.wqkv, *wfc1 = L.wfc1, *wout = L.wout, *wfc2 = L.wfc2;
        for (int r = a0; r < a1; r += 8) {
            if (!pr.stage(min(8, a1 - r), [&](int i) {
                    const int row = r + i;
                    return row < QKV_ROWS ? wqkv + (size_t)row * PD : wfc1 + (size_t)(row - QKV_ROWS) * PD;
                }))
                return;
        }
        for (int r = c0; r < c1; r += 8) {
            const int nv = min(8, c1 - r);
            if (!pr.stage(nv, [&](int i) { return wout + (size_t)(r + i) * PD; })) return;
            for (int ch = 0; ch < 4; ++ch)
                if (!pr.stage(nv, [&](int i) { return wfc2 + (size_t)(r + i) * PF + ch * PD; })) return;
        }
    }
    const __half* lm = T.lm_w;
    for (int r = h0; r < h1; r += 8)
        if (!pr.stage(min(8, h1 - r), [&](int i) { return lm + (size_t)(r + i) * PD; })) return;
}

// ---------------------------------------------------------------------------- the kernel

__global__ void __launch_bounds__(P_THREADS, 1)
decode_step_kernel(const md_persist_params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + PSmem::MISC);
    const uint32_t bars = sbase + PSmem::BARS;
    if (threadIdx.x == 0) {
        for (int s = 0; s < P_STAGES; ++s) {
            mbar_init(bars + 8 * s, 1);               // full: the producer's arrive + the copies' bytes
            mbar_init(bars + 8 * (P_STAGES + s), 8);  // empty: one arrive per consumer warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const md_persist_table& T = *p.tab;

    if (warp == 0) {
        Producer pr{sbase + PSmem::RING, bars, 0u, lane, abort_flag, p.flags};
        produce_all(pr, T, p);
        if (*abort_flag) {  // let copies in flight land before the CTA's shared memory is released
            const unsigned long long t0 = global_ns();
            while (global_ns() - t0 < 500000ull) {}
        }
        return;
    }

    PCtx c;
    c.ring = sbase + PSmem::RING;
    c.xs = sbase + PSmem::XS;
    c.partial = sbase + PSmem::PARTIAL;
    c.bars = bars;
    c.partial_ptr = reinterpret_cast<float*>(smem + PSmem::PARTIAL);
    c.red_ptr = reinterpret_cast<float*>(smem + PSmem::RED);
    c.xs_ptr = reinterpret_cast<__half*>(smem + PSmem::XS);
    c.abort_flag = abort_flag;
    c.flags = p.flags;
    c.cw = warp - 1;
    c.lane = lane;
    c.tc = threadIdx.x - 32;
    c.it = 0;
    c.pbuf = 0;

    const int cta = blockIdx.x, n = gridDim.x;
    int a0, a1, c0, c1, h0, h1;
    row_range(A_ROWS, cta, n, a0, a1);
    row_range(PD, cta, n, c0, c1);
    row_range(p.vocab, cta, n, h0, h1);
    unsigned int epoch = 0;
    for (int l = 0; l < p.n_layers; ++l) {
        const md_persist_table::Layer& L = T.layers[l];
        layernorm_to_smem(c, p.hidden, L.ln_w, L.ln_b, p.M, p.eps);
        phase_a(c, L, p, a0, a1);
        if (!grid_sync(c, p.grid_counter, ++epoch * n)) return;
        attention_phase(c, T, L, p);
        if (!grid_sync(c, p.grid_counter, ++epoch * n)) return;
        phase_c(c, L, p, c0, c1);
        if (!grid_sync(c, p.grid_counter, ++epoch * n)) return;
    }
    layernorm_to_smem(c, p.hidden, T.ln_out_w, T.ln_out_b, p.M, p.eps);
    phase_head(c, T, p, h0, h1);
}

}  // namespace

bool md_decode_persistent_supported(size_t dim, size_t hidden, size_t n_heads, size_t head_dim, size_t rot_dim,
                                    size_t vocab, size_t n_layers, size_t batch) {
    return dim == PD && hidden == PF && n_heads == PH && head_dim == PHD && rot_dim == PROT && vocab >= 1024 &&
           n_layers >= 1 && n_layers <= MD_PERSIST_MAX_LAYERS && batch >= 1 && batch <= MD_PERSIST_MAX_BATCH;
}

size_t md_decode_persistent_scratch_bytes(size_t batch, size_t max_seq) {
    const size_t max_splits = (max_seq + ATT_KEYS - 1) / ATT_KEYS;
    return batch * PH * max_splits * (PHD + 2) * sizeof(float);
}

int md_launch_decode_persistent(md_ctx* ctx, const md_persist_params& p) {
    static int configured_device = -1;
    if (configured_device != ctx->device) {
        MD_CUDA(ctx, cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PSmem::TOTAL));
        int per_sm = 0;
        MD_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel, P_THREADS, PSmem::TOTAL));
        if (per_sm < 1) return md_fail(ctx, MD_ERR_UNSUPPORTED, "decode_step_kernel does not fit on an SM of this device");
        configured_device = ctx->device;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctx->sm_count);
    cfg.blockDim = dim3(P_THREADS);
    cfg.dynamicSmemBytes = PSmem::TOTAL;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs co-resident: the grid barrier depends on it
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, decode_step_kernel, p);
    if (e != cudaSuccess)
        return md_fail(ctx, MD_ERR_CUDA, "launch of decode_step_kernel failed: %s", cudaGetErrorString(e));
    ctx->launches++;
    return MD_OK;
}
