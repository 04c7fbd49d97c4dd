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
//                barriers and through the attention phase: the ring (133 KB per SM, 20 MB in flight over
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
#include "ring_common.cuh"

namespace {

using namespace tc;
using namespace ring;

constexpr int PD = 2048, PF = 8192, PH = 32, PHD = 64, PROT = 32;  // Phi-1.5 geometry this kernel is built for
constexpr int QKV_ROWS = 3 * PD, A_ROWS = QKV_ROWS + PF;            // phase A: 14336 weight rows of 2048
constexpr int P_STAGES = 4;
constexpr int XBUF_BYTES = 8 * XS_PITCH * 2;    // 8 activation rows x 2048 k
constexpr int CONSUMERS = 256, P_THREADS = CONSUMERS + 32;
constexpr int ATT_KEYS = 32;                    // keys per attention unit (one warp): 8 K and 8 V loads in flight per lane
constexpr int MAX_Q_ROWS = 48, MAX_F_ROWS = 64, MAX_A_ROWS = MAX_Q_ROWS + MAX_F_ROWS;
constexpr int MAX_C_ROWS = 16, MAX_H_ROWS = 512;  // rows one CTA can own per phase (>= 128 CTAs)
constexpr unsigned long long GRID_WAIT_NS = 1000000000ull;

struct PSmem {
    static constexpr int RING = 0;
    static constexpr int XBUF = RING + P_STAGES * STAGE_BYTES;       // two activation buffers [8][XS_PITCH] halves
    static constexpr int PARTIAL = XBUF + 2 * XBUF_BYTES;            // [2 buffers][8 warps][2 sums][8][8] f32
    static constexpr int RED = PARTIAL + 2 * 8 * 2 * 64 * 4;         // [8 warps][8] partials, [2][8] results, decision
    static constexpr int BIAS = RED + (64 + 16 + 8) * 4;             // f32 biases of this CTA's rows in the phase
    static constexpr int POS = BIAS + MAX_H_ROWS * 4;                // pos[8], nsplit[8] (int)
    static constexpr int ROPE = POS + 16 * 4;                        // [8 requests][16][2] (cos, sin) at pos
    static constexpr int KVPTR = ROPE + 8 * 32 * 4;                  // [layers][K|V][8 requests] cache pointers
    static constexpr int BARS = KVPTR + MD_PERSIST_MAX_LAYERS * 2 * 8 * 8;  // full[4], empty[4]
    static constexpr int MISC = BARS + 2 * 8 * P_STAGES;             // abort flag
    static constexpr int TOTAL = MISC + 16;
};

struct PCtx {
    uint32_t ring, xbuf, bars;         // shared-memory addresses
    uint8_t* smem;                     // the same memory through generic pointers
    volatile int* abort_flag;
    md_devflags* flags;
    int cw, lane, tc;                  // consumer warp 0..7, lane, consumer thread 0..255
    uint32_t it;                       // stages consumed so far: slot = it % P_STAGES
    uint32_t tile;                     // tiles finished so far: partial buffer = tile & 1, epilogue warp = tile & 7
    __device__ __forceinline__ float* partial() const { return reinterpret_cast<float*>(smem + PSmem::PARTIAL); }
    __device__ __forceinline__ float* red() const { return reinterpret_cast<float*>(smem + PSmem::RED); }
    __device__ __forceinline__ float* bias() const { return reinterpret_cast<float*>(smem + PSmem::BIAS); }
    __device__ __forceinline__ int* pos() const { return reinterpret_cast<int*>(smem + PSmem::POS); }
    __device__ __forceinline__ float* rope() const { return reinterpret_cast<float*>(smem + PSmem::ROPE); }
    __device__ __forceinline__ __half** kvptr(int layer, int kv) const {
        return reinterpret_cast<__half**>(smem + PSmem::KVPTR) + (layer * 2 + kv) * 8;
    }
    __device__ __forceinline__ __half* xrow(int buf, int m) const {
        return reinterpret_cast<__half*>(smem + PSmem::XBUF + buf * XBUF_BYTES) + (size_t)m * XS_PITCH;
    }
};

__device__ __forceinline__ uint32_t bar_full(const PCtx& c, uint32_t slot) { return c.bars + 8 * slot; }
__device__ __forceinline__ uint32_t bar_empty(const PCtx& c, uint32_t slot) { return c.bars + 8 * (P_STAGES + slot); }

// Grid-wide barriers of the consumer threads (the producers never wait here), split in two halves so that
// independent work can sit between "my part is done" and "everybody's part is done".  Each barrier is a
// monotonic counter in global memory.
__device__ __forceinline__ void grid_arrive(const PCtx& c, unsigned int* counter) {
    consumer_sync();  // every consumer thread's global writes precede thread 0's fence
    if (c.tc == 0) {
        __threadfence();
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
    }
}
// Returns false once the step is being abandoned (a wait somewhere ran out of time).
__device__ bool grid_wait(const PCtx& c, const unsigned int* counter, unsigned int target) {
    if (c.tc == 0) {
        if (!*c.abort_flag) {
            const unsigned long long t0 = global_ns();
            unsigned spin = 0;
            while (ld_acquire_u32(counter) < target) {
                if ((++spin & 255u) == 0u) {
                    const bool failed_elsewhere = *reinterpret_cast<volatile unsigned int*>(&c.flags->error) != 0u;
                    if (failed_elsewhere || global_ns() - t0 > GRID_WAIT_NS) {
                        md_flag_timeout(c.flags, 40);
                        *c.abort_flag = 1;
                        break;
                    }
                }
            }
            __threadfence();
        }
        // one thread decides for all 256, so that they leave (or stay) together
        c.red()[87] = *c.abort_flag ? 0.f : 1.f;
    }
    consumer_sync();
    const bool ok = c.red()[87] != 0.f;
    consumer_sync();  // the decision word is free for the next wait
    return ok;
}

// LayerNorm (ops.zig layerNorm: two-pass f32, one rounding to f16) of the M rows of `hidden` into activation
// buffer 0; rows M..7 of the buffer are zero.  256 consumer threads, 8 elements of every row each; the M rows
// go through the two block reductions together.
__device__ void layernorm_to_smem(const PCtx& c, const __half* hidden, const __half* ln_w, const __half* ln_b, int M,
                                  float eps) {
    const uint4 gw = ldnc128(ln_w + c.tc * 8), gb = ldnc128(ln_b + c.tc * 8);
    float v[8][8], s[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        s[m] = 0.f;
        if (m < M) {
            unpack8(ldcg128(hidden + (size_t)m * PD + c.tc * 8), v[m]);
#pragma unroll
            for (int i = 0; i < 4; ++i) s[m] += v[m][2 * i] + v[m][2 * i + 1];
        }
    }
    float* red = c.red();  // [8 warps][8 rows], then [2][8] results at 64
    auto block_sum8 = [&](float (&x)[8], int slot) {
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            if (m < M) {
#pragma unroll
                for (int off = 16; off; off >>= 1) x[m] += __shfl_xor_sync(0xffffffffu, x[m], off);
            }
        }
        if (c.lane == 0) {
#pragma unroll
            for (int m = 0; m < 8; ++m) red[c.cw * 8 + m] = x[m];
        }
        consumer_sync();
        if (c.tc < 8) {
            float a = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) a += red[w * 8 + c.tc];
            red[64 + slot * 8 + c.tc] = a;
        }
        consumer_sync();
    };
    block_sum8(s, 0);
    float q[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        q[m] = 0.f;
        if (m < M) {
            const float mean = red[64 + m] * (1.0f / PD);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float d = v[m][i] - mean;
                q[m] += d * d;
            }
        }
    }
    block_sum8(q, 1);
    float wv[8], bv[8];
    unpack8(gw, wv);
    unpack8(gb, bv);
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        uint4 o = make_uint4(0, 0, 0, 0);
        if (m < M) {
            const float mean = red[64 + m] * (1.0f / PD);
            const float rstd = 1.0f / sqrtf(red[72 + m] * (1.0f / PD) + eps), mean_rstd = mean * rstd;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float y0 = (v[m][2 * i] * rstd - mean_rstd) * wv[2 * i] + bv[2 * i];
                const float y1 = (v[m][2 * i + 1] * rstd - mean_rstd) * wv[2 * i + 1] + bv[2 * i + 1];
                oh[i] = __floats2half2_rn(y0, y1);
            }
        }
        *reinterpret_cast<uint4*>(c.xrow(0, m) + c.tc * 8) = o;
    }
    consumer_sync();
}

// One ring stage (8 weight rows x 2048 k) against 8 activation rows in activation buffer `xb`: this warp's
// 256-wide k slice.
__device__ __forceinline__ void stage_mma(PCtx& c, int xb, float (&ae)[4], float (&ao)[4]) {
    const uint32_t slot = c.it % P_STAGES;
    mbar_wait(bar_full(c, slot), (c.it / P_STAGES) & 1u, c.abort_flag, c.flags, 41);
    const int g = c.lane >> 2, t = c.lane & 3;
    const uint32_t wbase = c.ring + slot * STAGE_BYTES + g * ROW_PITCH;
    const uint32_t xbase = c.xbuf + xb * XBUF_BYTES + g * (XS_PITCH * 2);
    uint4 lo[4], hi[4], xa[4], xv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int kk = c.cw * 256 + u * 64 + t * 8;
        lo[u] = lds128(wbase + kk * 2);
        hi[u] = lds128(wbase + (kk + 32) * 2);
        xa[u] = lds128(xbase + kk * 2);
        xv[u] = lds128(xbase + (kk + 32) * 2);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        mma_16816(ae, lo[u].x, hi[u].x, lo[u].y, hi[u].y, xa[u].x, xa[u].y);
        mma_16816(ae, lo[u].z, hi[u].z, lo[u].w, hi[u].w, xa[u].z, xa[u].w);
        mma_16816(ao, lo[u].x, hi[u].x, lo[u].y, hi[u].y, xv[u].x, xv[u].y);
        mma_16816(ao, lo[u].z, hi[u].z, lo[u].w, hi[u].w, xv[u].z, xv[u].w);
    }
    __syncwarp();
    if (c.lane == 0) mbar_arrive(bar_empty(c, slot));
    ++c.it;
}

// partial[buf][warp][sum][row][m]: valid halves are rows 0-7 of the "even" accumulators (c0, c1) and rows
// 8-15 of the "odd" ones (c2, c3)
__device__ __forceinline__ void store_partial(const PCtx& c, int sum, const float (&ae)[4], const float (&ao)[4]) {
    const int g = c.lane >> 2, t = c.lane & 3;
    float* dst = c.partial() + ((((c.tile & 1) * 8 + c.cw) * 2 + sum) * 8 + g) * 8 + 2 * t;
    dst[0] = ae[0] + ao[2];
    dst[1] = ae[1] + ao[3];
}
__device__ __forceinline__ float load_partial_sum(const PCtx& c, int sum, int rr, int m) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += c.partial()[((((c.tile & 1) * 8 + w) * 2 + sum) * 8 + rr) * 8 + m];
    return s;
}

// ---------------------------------------------------------------------------- consumer side of the phases

// The epilogue of a tile belongs to one warp, a different one every tile, so that no warp is on the critical
// path of every tile; its lanes cover the (request m, row rr) outputs idx = m * 8 + rr.
template <class F>
__device__ __forceinline__ void tile_epilogue(PCtx& c, int M, int rows_valid, F f) {
    consumer_sync();
    if (c.cw == (int)(c.tile & 7u)) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int idx = c.lane + 32 * h, m = idx >> 3, rr = idx & 7;
            if (m < M && rr < rows_valid) f(m, rr);
        }
    }
    ++c.tile;
}

// Biases of rows [r0, r1) of this CTA into shared memory as f32 (made visible by the phase's first barrier).
template <class BiasOf>
__device__ __forceinline__ void stage_biases(const PCtx& c, int r0, int r1, int offset, BiasOf bias_of) {
    for (int i = c.tc; i < r1 - r0; i += CONSUMERS) c.bias()[offset + i] = bias_of(r0 + i);
}

// Phase A of a layer, one weight matrix at a time: rows [r0, r1) of Wqkv (GELU false) or Wfc1 (GELU true)
// against the LayerNorm output (activation buffer 0): f16(acc) + bias, then GELU for fc1
// (text_model.zig:131-160).  `bias_off` = where this block's biases sit in the staging area.
template <bool GELU>
__device__ void phase_a(PCtx& c, const md_persist_params& p, int r0, int r1, int bias_off) {
    for (int r = r0; r < r1; r += 8) {
        float ae[4] = {0.f, 0.f, 0.f, 0.f}, ao[4] = {0.f, 0.f, 0.f, 0.f};
        stage_mma(c, 0, ae, ao);
        store_partial(c, 0, ae, ao);
        tile_epilogue(c, p.M, min(8, r1 - r), [&](int m, int rr) {
            const int row = r + rr;
            float val = md_round_f16(load_partial_sum(c, 0, rr, m));
            val = md_round_f16(val + c.bias()[bias_off + row - r0]);
            if (!GELU) {
                p.qkv[(size_t)m * QKV_ROWS + row] = __float2half_rn(val);
            } else {
                val = md_round_f16(md_gelu_f32(val));
                p.fc1[(size_t)m * PF + row] = __float2half_rn(val);
            }
        });
    }
}

// Copies 2048 activations of every request (rows x + m * ld) into activation buffer `buf`, asynchronously.
__device__ __forceinline__ void fetch_x_chunk(const PCtx& c, int buf, const __half* x, int ld, int M) {
    for (int m = 0; m < M; ++m)
        cp_async16(c.xbuf + buf * XBUF_BYTES + (m * XS_PITCH + c.tc * 8) * 2, x + (size_t)m * ld + c.tc * 8);
    cp_async_commit();
}

// Phase C: output rows [r0, r1) (at most two tiles) of fc2 (k = 8192: four stages per tile) and of the
// out-projection (k = 2048: one stage per tile), then attn_out += mlp_out and hidden += attn_out with one f16
// rounding each (text_model.zig:162-171).  fc2 comes first: it needs only the fc1 output, which has been
// complete since before the attention phase, so the wait for the slowest attention CTA hides behind four
// fifths of this phase's weight stream.  Activations are copied into shared memory one stage ahead,
// alternating between the two buffers; a piece is shared by both tiles.
struct PhaseCAcc {
    float e[2][4], o[2][4];
};
__device__ void phase_c_fc2(PCtx& c, const md_persist_params& p, int r0, int r1, PhaseCAcc& acc) {
    const int tiles = (r1 - r0 + 7) / 8;
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc.e[t][i] = acc.o[t][i] = 0.f;
    if (tiles == 0) return;
    fetch_x_chunk(c, 0, p.fc1, PF, p.M);
#pragma unroll 1
    for (int ch = 0; ch < 4; ++ch) {
        cp_async_wait_all();
        consumer_sync();  // piece ch has landed for everyone, and everyone is done with the other buffer
        if (ch + 1 < 4) fetch_x_chunk(c, (ch + 1) & 1, p.fc1 + (ch + 1) * PD, PF, p.M);
        stage_mma(c, ch & 1, acc.e[0], acc.o[0]);
        if (tiles > 1) stage_mma(c, ch & 1, acc.e[1], acc.o[1]);
    }
}
__device__ void phase_c_out(PCtx& c, const md_persist_params& p, int r0, int r1, PhaseCAcc& acc) {
    const int tiles = (r1 - r0 + 7) / 8;
    if (tiles == 0) return;
    consumer_sync();  // everyone is done with both activation buffers
    fetch_x_chunk(c, 0, p.attn, PD, p.M);
    cp_async_wait_all();
    consumer_sync();
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        if (t >= tiles) break;
        const int r = r0 + 8 * t;
        float a1e[4] = {0.f, 0.f, 0.f, 0.f}, a1o[4] = {0.f, 0.f, 0.f, 0.f};
        stage_mma(c, 0, a1e, a1o);
        store_partial(c, 0, a1e, a1o);
        store_partial(c, 1, acc.e[t], acc.o[t]);
        tile_epilogue(c, p.M, min(8, r1 - r), [&](int m, int rr) {
            const int n = r + rr;
            const float s1 = load_partial_sum(c, 0, rr, m), s2 = load_partial_sum(c, 1, rr, m);
            const float a = md_round_f16(md_round_f16(s1) + c.bias()[MAX_A_ROWS + (n - r0)]);
            const float mlp = md_round_f16(md_round_f16(s2) + c.bias()[MAX_A_ROWS + MAX_C_ROWS + (n - r0)]);
            const float sum = md_round_f16(a + mlp);
            __half* h = p.hidden + (size_t)m * PD + n;
            *h = __float2half_rn(ldcg_f16(h) + sum);
        });
    }
}

// lm_head rows [r0, r1) against the final LayerNorm output (activation buffer 0): logits and the
// greedy-argmax key (text_model.zig:325-345, sampling.zig:257-273: first strict maximum of the f16 logits).
__device__ void phase_head(PCtx& c, const md_persist_params& p, int r0, int r1) {
    unsigned long long best[2] = {0ull, 0ull};  // per lane: requests m = lane >> 3 and 4 + (lane >> 3)
    for (int r = r0; r < r1; r += 8) {
        float ae[4] = {0.f, 0.f, 0.f, 0.f}, ao[4] = {0.f, 0.f, 0.f, 0.f};
        stage_mma(c, 0, ae, ao);
        store_partial(c, 0, ae, ao);
        tile_epilogue(c, p.M, min(8, r1 - r), [&](int m, int rr) {
            const int n = r + rr;
            float val = md_round_f16(load_partial_sum(c, 0, rr, m));
            val = md_round_f16(val + c.bias()[n - r0]);
            p.logits[(size_t)m * p.vocab + n] = __float2half_rn(val);
            const unsigned bits = __float_as_uint(val);
            const unsigned ordered = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
            const unsigned long long key =
                ((unsigned long long)ordered << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)n);
            unsigned long long& b = best[m >> 2];
            b = key > b ? key : b;
        });
    }
    // every warp has been the epilogue warp of some tiles: lanes m*8 .. m*8+7 (mod 32) hold request m's candidates
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        unsigned long long b = best[h];
#pragma unroll
        for (int o = 4; o; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, b, o);
            b = other > b ? other : b;
        }
        const int m = (c.lane >> 3) + 4 * h;
        if ((c.lane & 7) == 0 && m < p.M && b != 0ull) atomicMax(p.amax + m, b);
    }
}

// ---------------------------------------------------------------------------- attention phase

// Rotary embedding of this lane's 8 dims (dims sub*8 .. sub*8+7 of a head; rope.zig:130-216: the first
// PROT dims rotate as pairs (j, j + PROT/2), the rest pass through), result rounded to f16.
// `cs` = the (cos, sin) pairs of this request's position: [16][2] floats in shared memory.
__device__ __forceinline__ void rope8(float (&x)[8], int sub, const float* cs_tab) {
    float partner[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) partner[i] = __shfl_xor_sync(0xffffffffu, x[i], 2);  // sub 0<->2, 1<->3
    if (sub < 4) {
        const int j0 = (sub & 1) * 8;
        const float4* cs = reinterpret_cast<const float4*>(cs_tab + j0 * 2);
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

__device__ void attention_phase(const PCtx& c, int layer, const md_persist_params& p) {
    int pos[MD_PERSIST_MAX_BATCH], nsplit[MD_PERSIST_MAX_BATCH], total = 0;
#pragma unroll
    for (int b = 0; b < MD_PERSIST_MAX_BATCH; ++b) {
        pos[b] = 0;
        nsplit[b] = 0;
        if (b < p.M) {
            pos[b] = c.pos()[b];
            nsplit[b] = c.pos()[8 + b];
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
        __half* kc = c.kvptr(layer, 0)[b];
        __half* vc = c.kvptr(layer, 1)[b];
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
        rope8(q, sub, c.rope() + b * 32);
        float knew[8], vnew[8];
        if (last) {  // warp-uniform
            unpack8(ldcg128(qkv + PD + head * PHD + sub * 8), knew);
            rope8(knew, sub, c.rope() + b * 32);
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
    uint64_t policy;

    // One stage: rows row .. row+nv-1, `bytes_per_row` from src(row) each.  Returns false when abandoned.
    template <class SrcOf>
    __device__ __forceinline__ bool stage(int nv, SrcOf src_of) {
        const uint32_t slot = it % P_STAGES, full = bars + 8 * slot, empty = bars + 8 * (P_STAGES + slot);
        mbar_wait(empty, ((it / P_STAGES) & 1u) ^ 1u, abort_flag, flags, 42);
        if (*abort_flag) return false;
        if (lane == 0) mbar_expect_tx(full, (uint32_t)nv * 4096u);
        __syncwarp();
        if (lane < nv) bulk_load_row(ring + slot * STAGE_BYTES + lane * ROW_PITCH, src_of(lane), 4096u, full, policy);
        ++it;
        return true;
    }
};

__device__ void produce_all(Producer& pr, const md_persist_table& T, const md_persist_params& p) {
    const int cta = blockIdx.x, n = gridDim.x;
    int q0, q1, f0, f1, c0, c1, h0, h1;
    row_range(QKV_ROWS, cta, n, q0, q1);
    row_range(PF, cta, n, f0, f1);
    row_range(PD, cta, n, c0, c1);
    row_range(p.vocab, cta, n, h0, h1);
    for (int l = 0; l < p.n_layers; ++l) {
        const md_persist_table::Layer& L = T.layers[l];
        const __half *wqkv = L.wqkv, *wfc1 = L.wfc1, *wout = L.wout, *wfc2 = L.wfc2;
        for (int r = q0; r < q1; r += 8)
            if (!pr.stage(min(8, q1 - r), [&](int i) { return wqkv + (size_t)(r + i) * PD; })) return;
        for (int r = f0; r < f1; r += 8)
            if (!pr.stage(min(8, f1 - r), [&](int i) { return wfc1 + (size_t)(r + i) * PD; })) return;
        for (int ch = 0; ch < 4; ++ch)
            for (int r = c0; r < c1; r += 8)
                if (!pr.stage(min(8, c1 - r), [&](int i) { return wfc2 + (size_t)(r + i) * PF + ch * PD; })) return;
        for (int r = c0; r < c1; r += 8)
            if (!pr.stage(min(8, c1 - r), [&](int i) { return wout + (size_t)(r + i) * PD; })) return;
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
        Producer pr{sbase + PSmem::RING, bars, 0u, lane, abort_flag, p.flags, l2_evict_first_policy()};
        produce_all(pr, T, p);
        if (*abort_flag) {  // let copies in flight land before the CTA's shared memory is released
            const unsigned long long t0 = global_ns();
            while (global_ns() - t0 < 500000ull) {}
        }
        return;
    }

    PCtx c;
    c.ring = sbase + PSmem::RING;
    c.xbuf = sbase + PSmem::XBUF;
    c.bars = bars;
    c.smem = smem;
    c.abort_flag = abort_flag;
    c.flags = p.flags;
    c.cw = warp - 1;
    c.lane = lane;
    c.tc = threadIdx.x - 32;
    c.it = 0;
    c.tile = 0;

    // per-step constants: positions, split counts and the rope (cos, sin) rows of every request;
    // activation buffer 1 starts zeroed (only rows < M are ever written)
    if (c.tc < MD_PERSIST_MAX_BATCH) {
        const int b = c.tc, pos = b < p.M ? *T.pos[b] : 0;
        c.pos()[b] = pos;
        c.pos()[8 + b] = b < p.M ? max(1, (pos + ATT_KEYS - 1) / ATT_KEYS) : 0;
    }
    {
        const int b = c.tc >> 5, i = c.tc & 31;  // 8 requests x 32 floats
        if (b < p.M) c.rope()[b * 32 + i] = p.rope_tab[(size_t)(*T.pos[b]) * PROT + i];
    }
    for (int i = c.tc; i < XBUF_BYTES / 16; i += CONSUMERS)
        *reinterpret_cast<uint4*>(smem + PSmem::XBUF + XBUF_BYTES + i * 16) = make_uint4(0, 0, 0, 0);
    for (int i = c.tc; i < p.n_layers * 16; i += CONSUMERS) {
        const int l = i >> 4, kv = (i >> 3) & 1, b = i & 7;
        c.kvptr(l, kv)[b] = kv ? T.layers[l].vc[b] : T.layers[l].kc[b];
    }

    const int cta = blockIdx.x, n = gridDim.x;
    int q0, q1, f0, f1, c0, c1, h0, h1;
    row_range(QKV_ROWS, cta, n, q0, q1);
    row_range(PF, cta, n, f0, f1);
    row_range(PD, cta, n, c0, c1);
    row_range(p.vocab, cta, n, h0, h1);
    consumer_sync();  // positions are in shared memory

    // Small operands (LayerNorm parameters, biases, the KV cache of the attention) are demand loads that
    // would queue behind ~20 MB of weight copies in flight; they are pulled into L2 one layer ahead instead.
    auto prefetch_layer = [&](int l) {
        if (l >= p.n_layers) return;
        const md_persist_table::Layer& L = T.layers[l];
        if (c.tc < 32) prefetch_l2(L.ln_w + c.tc * 64);
        else if (c.tc < 64) prefetch_l2(L.ln_b + (c.tc - 32) * 64);
        else if (c.tc < 66) prefetch_l2(L.bqkv + q0 + (c.tc - 64) * 63);   // <= 43 halves: at most two lines
        else if (c.tc < 68) prefetch_l2(L.bfc1 + f0 + (c.tc - 66) * 63);   // <= 57 halves
        else if (c.tc == 68) prefetch_l2(L.bout + c0);
        else if (c.tc == 69) prefetch_l2(L.bfc2 + c0);
        // this CTA's share of the cache rows the attention of layer l will read: 4 KB pieces of the
        // [pos x 128 B] range of every (request, K|V, head)
        for (int b = 0; b < p.M; ++b) {
            const int pos = c.pos()[b];
            const unsigned bytes = (unsigned)pos * (PHD * 2), nch = (bytes + 4095u) / 4096u;
            for (unsigned id = (unsigned)cta + (unsigned)n * (unsigned)c.tc; id < 2u * PH * nch; id += (unsigned)n * CONSUMERS) {
                const unsigned range = id / nch, j = id % nch, head = range % PH;
                const __half* base = c.kvptr(l, range < PH ? 0 : 1)[b] + (size_t)head * p.max_seq * PHD;
                const unsigned off = j * 4096u, sz = min(4096u, bytes - off) & ~15u;
                if (sz)
                    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<const char*>(base) + off),
                                 "r"(sz)
                                 : "memory");
            }
        }
    };
    prefetch_layer(0);

    int tr = 0;
    unsigned long long* trace = nullptr;
    if (p.trace && c.tc == 0 && (cta == 0 || cta == n - 1)) trace = p.trace + (cta == 0 ? 0 : 256);
    auto stamp = [&]() { if (trace && tr < 256) trace[tr++] = global_ns(); };
    unsigned int* const bar_qkv = p.grid_counter;       // this layer's q, k, v rows are written
    unsigned int* const bar_fc1 = p.grid_counter + 1;   // ... fc1 rows
    unsigned int* const bar_att = p.grid_counter + 2;   // ... attention output
    unsigned int* const bar_hid = p.grid_counter + 3;   // ... hidden state
    stamp();
    for (int l = 0; l < p.n_layers; ++l) {
        const md_persist_table::Layer& L = T.layers[l];
        const unsigned target = (unsigned)(l + 1) * (unsigned)n;
        // this thread's share of the layer's biases: requested now, parked in shared memory after the LayerNorm
        // (one memory round trip for everything the layer start needs)
        float bq = 0.f, bf = 0.f, bo = 0.f, b2 = 0.f;
        if (c.tc < q1 - q0) bq = ldnc_f16(L.bqkv + q0 + c.tc);
        if (c.tc < f1 - f0) bf = ldnc_f16(L.bfc1 + f0 + c.tc);
        if (c.tc < c1 - c0) {
            bo = ldnc_f16(L.bout + c0 + c.tc);
            b2 = ldnc_f16(L.bfc2 + c0 + c.tc);
        }
        layernorm_to_smem(c, p.hidden, L.ln_w, L.ln_b, p.M, p.eps);
        if (c.tc < q1 - q0) c.bias()[c.tc] = bq;
        if (c.tc < f1 - f0) c.bias()[MAX_Q_ROWS + c.tc] = bf;
        if (c.tc < c1 - c0) {
            c.bias()[MAX_A_ROWS + c.tc] = bo;
            c.bias()[MAX_A_ROWS + MAX_C_ROWS + c.tc] = b2;
        }
        prefetch_layer(l + 1);
        stamp();
        phase_a<false>(c, p, q0, q1, 0);
        grid_arrive(c, bar_qkv);
        phase_a<true>(c, p, f0, f1, MAX_Q_ROWS);
        grid_arrive(c, bar_fc1);
        stamp();
        if (!grid_wait(c, bar_qkv, target)) return;
        stamp();
        attention_phase(c, l, p);
        grid_arrive(c, bar_att);
        stamp();
        if (!grid_wait(c, bar_fc1, target)) return;
        stamp();
        PhaseCAcc acc;
        phase_c_fc2(c, p, c0, c1, acc);
        if (!grid_wait(c, bar_att, target)) return;
        phase_c_out(c, p, c0, c1, acc);
        stamp();
        grid_arrive(c, bar_hid);
        if (!grid_wait(c, bar_hid, target)) return;
        stamp();
    }
    {
        const __half* lm_b = T.lm_b;
        stage_biases(c, h0, h1, 0, [&](int row) { return ldnc_f16(lm_b + row); });
    }
    layernorm_to_smem(c, p.hidden, T.ln_out_w, T.ln_out_b, p.M, p.eps);
    stamp();
    phase_head(c, p, h0, h1);
    stamp();
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
    // the per-CTA row ranges must fit the bias staging area
    const int n = ctx->sm_count;
    if (n < 1 || (A_ROWS + n - 1) / n + 1 > MAX_A_ROWS || (PD + n - 1) / n + 1 > MAX_C_ROWS ||
        (p.vocab + n - 1) / n + 1 > MAX_H_ROWS || (QKV_ROWS + n - 1) / n + 1 > MAX_Q_ROWS ||
        (PF + n - 1) / n + 1 > MAX_F_ROWS)
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "decode_step_kernel: %d SMs are too few for its row partition", n);
    static int configured_device = -1;
    if (configured_device != ctx->device) {
        MD_CUDA(ctx, cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PSmem::TOTAL));
        int per_sm = 0;
        MD_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel, P_THREADS, PSmem::TOTAL));
        if (per_sm < 1) return md_fail(ctx, MD_ERR_UNSUPPORTED, "decode_step_kernel does not fit on an SM of this device");
        configured_device = ctx->device;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)n);
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
