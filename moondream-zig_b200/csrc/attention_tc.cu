// Multi-query attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// Replaces attention.multiMasklessSDPA (attention.zig:125-234: ViT, 729 tokens, d = 72) and
// attention.multiMaskedSDPA (attention.zig:416-541: decoder prefill, d = 64, causal) for the layouts
// TMA can address; sdpa_mma_kernel (attention.cu) remains the path for everything else.
//
// A work item = 128 queries of one (batch, head).  The grid is at most two CTAs per SM (224 threads each); a CTA
// takes one item per round of gridDim.x items and keeps its barriers, its tensor memory and its rings across
// them, so that from the second item on nothing of a CTA's start-up (launch, barrier set-up, TMEM allocation,
// descriptor fetch, first loads) is paid again: the producer fetches the next item's Q as soon as the softmax warps
// have moved the current one into tensor memory, and its K / V tiles as ring stages come free.  Rounds alternate
// direction over the CTAs, so the CTA with the longest causal item of one round gets the shortest of the next.
//   warp 0      TMA producer: per item Q, then K tiles of 64 keys through a ring of three stages and V tiles through
//               a ring of two, K one tile ahead of V (a K stage is free with S(j), a V stage only with PV(j)).
//   warp 1      one lane issues S = Q K^T (tcgen05.mma, 128 x 64 x d, into one of two S buffers in tensor memory);
//   warp 6      one lane issues O += P V (128 x d x 64, accumulated in tensor memory over all key tiles).
//               Both products read their A operand (Q, P) from tensor memory as packed f16 and only K and V from
//               shared memory: with A in shared memory every k-step of 16 re-read 4 KB of Q or P for 2 KB of K or
//               V, and those reads, the P stores and the TMA fills together kept the shared-memory port busy for
//               the whole tile.  tcgen05.commit signals completion.
//   warps 2..5  one thread per query row.  Per item: its row of Q from the swizzled shared-memory tile into tensor
//               memory (tcgen05.st).  Per tile: tcgen05.ld of its S row, mask / running max / exp2 in f32 registers
//               (no shuffles: a row lives in one thread), P as packed f16 written over the first half of the S
//               buffer it came from (tcgen05.st).
// O stays in tensor memory.  The exponent reference of a row moves only when the row maximum has grown by more
// than 2^8 since it was last set; only then do the softmax warps rescale that row of O (rare after the first
// tiles), so the usual tile costs one read of S and no read of O.  P therefore holds values up to 2^8, well inside
// f16, and the row sum is kept in f32 on the same reference.
// S(j+1) is issued while the softmax warps work on tile j (it needs PV(j-1), whose P it overwrites, to have
// completed), and the second CTA of the SM fills the remaining gaps.
// End of an item: O into registers (which frees it for the next item), the next item's Q into tensor memory (so its
// first S product runs meanwhile), then the rows are packed in shared memory and leave as one TMA store per 32 rows.
//
// Operands are addressed through 4-D tensor maps (d, row, head, batch) whose extents are exactly the
// valid data, so everything outside (rows past kv_len, dims past d) is zero-filled by TMA: no stale
// cache rows or neighbouring heads ever reach the tensor cores.
// d = 72: dims 0-63 travel as a 128B-swizzled tile.  For Q and K (K-major operands of S) dims 64-79 (64-71 data, the
// rest zero fill) follow as a second, 32B-swizzled tile of 16 dims, one more k-step of S.  For V (the MN-major B
// operand of the PV product) the tail is a second 128B-swizzled atom (dims 64-127 of the box, all but 8 of them zero
// fill and never read) right behind the main tile, so that one MMA with N = 80 covers both: an MMA this small costs
// about the same 45-50 cycles whatever its N, so a separate N = 16 product for the tail would nearly double the time
// of the PV product.
//
// Numerics as the reference: scores, probability sums and the output accumulate in f32, one rounding
// to f16 at the end (attention.zig:199-202,505-508); P is rounded to f16 for the PV product.
// Every mbarrier wait is bounded (tc_common.cuh); a wait that gives up is reported through the
// context's error word and the kernel still runs to its end and frees its TMEM.
#include <algorithm>
#include <climits>

#include "md_internal.cuh"
#include "tc_common.cuh"

int md_make_map_4d(md_ctx* ctx, CUtensorMap* map, const void* ptr, const uint64_t dims[4], const uint64_t strides_bytes[3],
                   uint32_t box0, const uint32_t box_d[3], int swizzle_bytes);

namespace {

using namespace tc;

constexpr int ABQ = 128, ABKV = 64;
constexpr int ATTN_THREADS = 224;   // producer, S issuer, 4 softmax warps, PV issuer
constexpr float LOG2E_F = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units a row maximum may grow before O is rescaled

struct AttnTcParams {
    int q_len, kv_len, causal_pos;
    float scale_log2;
    const uint8_t* mask;  // [q_len, kv_len] or null
    // 4-D tensor maps (dim 0 = head dimension d; dims 1..3 = row, head, batch in order of ascending stride):
    // which map dimension carries the row / head / batch index, for q and for k, v
    int q_dim_row, q_dim_head, q_dim_batch, kv_dim_row, kv_dim_head, kv_dim_batch;
    int o_dim_row, o_dim_head, o_dim_batch;
    int n_qblk, n_heads, n_batch, n_items;   // items = n_qblk * n_heads * n_batch
};

// Item w -> (query block, head, batch).  Causal: the last query blocks see the most keys, so they come first
// (longest items first when a CTA takes several); otherwise the query blocks of one (batch, head) are neighbours,
// so the CTAs that run together share K and V in L2.
__device__ __forceinline__ void attn_item(const AttnTcParams& p, int w, int& qblk, int& head, int& batch) {
    const int hb = p.n_heads * p.n_batch;
    int r;
    if (p.causal_pos >= 0) { qblk = p.n_qblk - 1 - w / hb; r = w % hb; }
    else { qblk = w % p.n_qblk; r = w / p.n_qblk; }
    head = r % p.n_heads;
    batch = r / p.n_heads;
}
// The item a CTA takes in its round `it` (-1: none, and none later): rounds alternate direction over the CTAs, so the
// CTA that got the longest causal item of one round gets the shortest of the next.
__device__ __forceinline__ int attn_walk(const AttnTcParams& p, int it) {
    const int c = (it & 1) ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
    const long long w = (long long)it * gridDim.x + c;
    return w < p.n_items ? (int)w : -1;
}
__device__ __forceinline__ int attn_tiles(const AttnTcParams& p, int q0) {
    int kv_end = p.kv_len;
    if (p.causal_pos >= 0) kv_end = min(kv_end, p.causal_pos + min(q0 + ABQ, p.q_len));
    return (kv_end + ABKV - 1) / ABKV;
}

struct AttnTcMaps {
    CUtensorMap q, k, v;     // dims 0-63, 128B swizzle
    CUtensorMap qt, kt, vt;  // dims 64-79 (d = 72 only), 32B swizzle
    CUtensorMap o;           // the output, boxes of 32 rows x d, no swizzle
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
                 "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void tc_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tc_st_32x8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D> struct AttnCfg {
    static constexpr bool TAIL = D > 64;                     // dims 64.. of d = 72
    static constexpr int DPAD = TAIL ? 80 : 64;              // MMA extent of the head dimension
    static constexpr int STAGES = 3, V_STAGES = 2;           // depth of the K ring and of the V ring
    static constexpr int Q_MAIN = ABQ * 128, Q_TAIL = TAIL ? ABQ * 32 : 0;
    static constexpr int KV_MAIN = ABKV * 128, KV_TAIL = TAIL ? ABKV * 32 : 0;
    static constexpr int Q_BYTES = Q_MAIN + Q_TAIL;
    static constexpr int STAGE_BYTES = KV_MAIN + KV_TAIL;    // one K tile: main | 32B-swizzled tail
    static constexpr int V_STAGE_BYTES = KV_MAIN + (TAIL ? KV_MAIN : 0);   // one V tile: main | second 128B atom
    static constexpr int OUT_ROW = D * 2;                    // one output row, packed
    static constexpr int OUT_BYTES = ABQ * OUT_ROW;          // staging of an item's output for the TMA stores
    static constexpr int SMEM = 1024 + Q_BYTES + STAGES * STAGE_BYTES + V_STAGES * V_STAGE_BYTES + OUT_BYTES + 256;  // 101.25 / 73.25 KB
};

template <int D>
__global__ void __launch_bounds__(ATTN_THREADS, 2)
attn_tc_kernel(const __grid_constant__ AttnTcMaps tm, AttnTcParams p, md_devflags* flags) {
    using Cfg = AttnCfg<D>;
    constexpr int ST = Cfg::STAGES, STV = Cfg::V_STAGES;
    constexpr bool TAIL = Cfg::TAIL;
    // Tensor memory, 256 columns: two S buffers of 64 (P, as packed f16, takes the first 32 columns of the buffer its
    // S came from), O (64 or 80), Q as packed f16 (32 or 40)
    constexpr uint32_t TMEM_COLS = 256, T_O = 128, T_Q = 208;
    static_assert(T_O + Cfg::DPAD <= T_Q && T_Q + Cfg::DPAD / 2 <= TMEM_COLS, "tensor memory layout");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t sm_q = base, sm_qt = sm_q + Cfg::Q_MAIN;
    // K and V travel through separate rings: a K stage is free again as soon as S(j) has been computed,
    // a V stage only after PV(j), two MMAs later; one shared ring would hold the next K load back
    const uint32_t sm_k = sm_q + Cfg::Q_BYTES, sm_v = sm_k + ST * Cfg::STAGE_BYTES;  // per stage: main | tail
    const uint32_t sm_out = sm_v + STV * Cfg::V_STAGE_BYTES;
    uint8_t* out_ptr = base_ptr + Cfg::Q_BYTES + ST * Cfg::STAGE_BYTES + STV * Cfg::V_STAGE_BYTES;
    const uint32_t bars = sm_out + Cfg::OUT_BYTES;
    uint8_t* bars_ptr = out_ptr + Cfg::OUT_BYTES;
    const uint32_t b_qfull = bars, b_kfull = bars + 8, b_kempty = b_kfull + 8 * ST, b_vfull = b_kempty + 8 * ST;
    const uint32_t b_vempty = b_vfull + 8 * STV;
    const uint32_t b_sfull = b_vempty + 8 * STV;  // S(j) is in tensor memory
    const uint32_t b_pfull = b_sfull + 16;       // the softmax warps have written P(j) over it
    const uint32_t b_pvdone = b_pfull + 16;      // PV(j) has completed: O is current, the S / P buffer is free
    const uint32_t b_qcopied = b_pvdone + 16;    // the softmax warps have moved Q from shared to tensor memory
    const uint32_t b_oempty = b_qcopied + 8;     // ... and have read an item's O out of tensor memory
    // ends at bars + 8 + 16 * (ST + STV) + 48 + 16 <= bars + 168
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars_ptr + 176);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_ptr + 180);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    md_pdl_launch_dependents();
    if (threadIdx.x == 0) {
        // the descriptors are kernel parameters: fetching them does not depend on the predecessor kernel
        tma_prefetch_map(&tm.q);
        tma_prefetch_map(&tm.k);
        tma_prefetch_map(&tm.v);
        tma_prefetch_map(&tm.o);
        if (TAIL) {
            tma_prefetch_map(&tm.qt);
            tma_prefetch_map(&tm.kt);
            tma_prefetch_map(&tm.vt);
        }
        mbar_init(b_qfull, 1);
        mbar_init(b_qcopied, 4);
        mbar_init(b_oempty, 4);
        for (int s = 0; s < ST; ++s) {
            mbar_init(b_kfull + 8 * s, 1);
            mbar_init(b_kempty + 8 * s, 1);
        }
        for (int s = 0; s < STV; ++s) {
            mbar_init(b_vfull + 8 * s, 1);
            mbar_init(b_vempty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(b_sfull + 8 * b, 1);
            mbar_init(b_pfull + 8 * b, 4);
            mbar_init(b_pvdone + 8 * b, 1);
        }
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
    md_pdl_wait();

    // Every role walks the same items in the same order.  Ring slots, the S / P buffer of a tile and the wait
    // parities run on over the items: `g` counts the key tiles this CTA has handled before the current item.
    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t kst = 0, kpar = 1, vst = 0, vpar = 1;  // ring slots and the parities that say "slot free"
            int ck[4] = {0, 0, 0, 0};
            auto load_k = [&](int j) {
                ck[p.kv_dim_row] = j * ABKV;
                mbar_wait(b_kempty + 8 * kst, kpar, abort_flag, flags, 11);
                const uint32_t kfull = b_kfull + 8 * kst, kdst = sm_k + kst * Cfg::STAGE_BYTES;
                mbar_expect_tx(kfull, Cfg::STAGE_BYTES);
                tma_load_4d(kdst, &tm.k, kfull, 0, ck[1], ck[2], ck[3]);
                if (TAIL) tma_load_4d(kdst + Cfg::KV_MAIN, &tm.kt, kfull, 64, ck[1], ck[2], ck[3]);
                if (++kst == ST) { kst = 0; kpar ^= 1u; }
            };
            int it = 0;
            for (int w; (w = attn_walk(p, it)) >= 0; ++it) {
                int qblk, head, batch;
                attn_item(p, w, qblk, head, batch);
                const int q0 = qblk * ABQ, nt = attn_tiles(p, q0);
                int cq[4] = {0, 0, 0, 0};
                cq[p.q_dim_row] = q0; cq[p.q_dim_head] = head; cq[p.q_dim_batch] = batch;
                ck[p.kv_dim_head] = head; ck[p.kv_dim_batch] = batch;
                if (it > 0) mbar_wait(b_qcopied, (uint32_t)((it - 1) & 1), abort_flag, flags, 9);
                mbar_expect_tx(b_qfull, Cfg::Q_BYTES);
                tma_load_4d(sm_q, &tm.q, b_qfull, 0, cq[1], cq[2], cq[3]);
                if (TAIL) tma_load_4d(sm_qt, &tm.qt, b_qfull, 64, cq[1], cq[2], cq[3]);
                // K runs one tile ahead of V: a K stage comes free with S(j), a V stage only with PV(j)
                if (nt > 0) load_k(0);
                for (int j = 0; j < nt; ++j) {
                    if (j + 1 < nt) load_k(j + 1);
                    ck[p.kv_dim_row] = j * ABKV;
                    mbar_wait(b_vempty + 8 * vst, vpar, abort_flag, flags, 10);
                    const uint32_t vfull = b_vfull + 8 * vst, vdst = sm_v + vst * Cfg::V_STAGE_BYTES;
                    mbar_expect_tx(vfull, Cfg::V_STAGE_BYTES);
                    tma_load_4d(vdst, &tm.v, vfull, 0, ck[1], ck[2], ck[3]);
                    if (TAIL) tma_load_4d(vdst + Cfg::KV_MAIN, &tm.vt, vfull, 64, ck[1], ck[2], ck[3]);
                    if (++vst == STV) { vst = 0; vpar ^= 1u; }
                }
            }
            if (*abort_flag) {  // let copies in flight land before the CTA's shared memory is released
                const unsigned long long t0 = global_ns();
                while (global_ns() - t0 < 500000ull) {}
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ issuer of the S products
        // Both products take their A operand (Q, P: K-major, packed f16) from tensor memory, 8 columns per k-step of
        // 16; only K and V are read from shared memory.  Issuing a tile's nine MMAs and four commits from one thread
        // took longer than the softmax of the tile, so the two products have a thread each; what orders them across
        // the two threads are the barriers (S(j) waits for PV(j-2), whose P it overwrites; PV(j) waits for P(j)).
        if (lane == 0) {
            const uint32_t idesc_s = (1u << 4) | ((uint32_t)(ABKV >> 3) << 17) | ((uint32_t)(ABQ >> 4) << 24);
            // descriptors as 32-bit halves (tc_common.cuh): constant high words, low words advanced by adds; ring
            // slots and their wait parities are running counters
            const uint32_t hi128 = desc_hi(1024, 2), hi32 = desc_hi(256, 6);
            const uint32_t k_lo0 = desc_lo(sm_k, 16), kt_lo0 = desc_lo(sm_k + Cfg::KV_MAIN, 16);
            constexpr uint32_t STAGE16 = Cfg::STAGE_BYTES >> 4;
            const uint32_t t_q = tmem_base + T_Q;
            uint32_t st = 0, par = 0;        // ring slot and parity of the next S product
            uint32_t g = 0;                  // key tiles of earlier items
            int it = 0;
            for (int w; (w = attn_walk(p, it)) >= 0; ++it) {
                int qblk, head, batch;
                attn_item(p, w, qblk, head, batch);
                const int nt = attn_tiles(p, qblk * ABQ);
                if (nt > 0) mbar_wait(b_qcopied, (uint32_t)(it & 1), abort_flag, flags, 14);
                for (int j = 0; j < nt; ++j) {
                    const uint32_t gj = g + (uint32_t)j, sb = gj & 1u;
                    mbar_wait(b_kfull + 8 * st, par, abort_flag, flags, 15);
                    // the buffer still holds P of two tiles back until that PV product has completed
                    mbar_wait(b_pvdone + 8 * sb, ((gj >> 1) & 1u) ^ 1u, abort_flag, flags, 16);
                    tc_fence_after();
                    const uint32_t t_s = tmem_base + sb * 64u, k_lo = k_lo0 + st * STAGE16;
                    tc_mma_f16_ts<false>(t_s, t_q, k_lo, hi128, idesc_s);
#pragma unroll
                    for (int ks = 1; ks < 4; ++ks) tc_mma_f16_ts<true>(t_s, t_q + ks * 8, k_lo + ks * 2, hi128, idesc_s);
                    if (TAIL) tc_mma_f16_ts<true>(t_s, t_q + 32, kt_lo0 + st * STAGE16, hi32, idesc_s);
                    tc_commit(b_sfull + 8 * sb);
                    tc_commit(b_kempty + 8 * st);
                    if (++st == ST) { st = 0; par ^= 1u; }
                }
                g += (uint32_t)nt;
            }
        }
    } else if (warp == 6) {
        // ------------------------------------------------------------------ issuer of the PV products
        if (lane == 0) {
            const uint32_t idesc_pv =
                (1u << 4) | (1u << 16) | ((uint32_t)(Cfg::DPAD >> 3) << 17) | ((uint32_t)(ABQ >> 4) << 24);
            const uint32_t hi128 = desc_hi(1024, 2);
            // V: MN-major, 64 dims contiguous per key; the next atom along the dims (d = 72) lies one main tile further
            const uint32_t v_lo0 = desc_lo(sm_v, ABKV * 128);
            constexpr uint32_t VSTAGE16 = Cfg::V_STAGE_BYTES >> 4;
            uint32_t st = 0, par = 0;        // ring slot and parity of the next PV product
            uint32_t g = 0;
            int it = 0;
            for (int w; (w = attn_walk(p, it)) >= 0; ++it) {
                int qblk, head, batch;
                attn_item(p, w, qblk, head, batch);
                const int nt = attn_tiles(p, qblk * ABQ);
                for (int j = 0; j < nt; ++j) {
                    const uint32_t gj = g + (uint32_t)j, pb = gj & 1u;
                    mbar_wait(b_vfull + 8 * st, par, abort_flag, flags, 13);
                    mbar_wait(b_pfull + 8 * pb, (gj >> 1) & 1u, abort_flag, flags, 12);
                    // the first product of an item overwrites O: the previous item's output must have left tensor memory
                    if (j == 0 && it > 0) mbar_wait(b_oempty, (uint32_t)((it - 1) & 1), abort_flag, flags, 17);
                    tc_fence_after();
                    const uint32_t t_p = tmem_base + pb * 64u, v_lo = v_lo0 + st * VSTAGE16;
                    // 16 keys = 8 columns of P and 2048 B of V per k-step (in every atom)
                    if (j == 0) tc_mma_f16_ts<false>(tmem_base + T_O, t_p, v_lo, hi128, idesc_pv);
                    else tc_mma_f16_ts<true>(tmem_base + T_O, t_p, v_lo, hi128, idesc_pv);
#pragma unroll
                    for (int ks = 1; ks < ABKV / 16; ++ks)
                        tc_mma_f16_ts<true>(tmem_base + T_O, t_p + ks * 8, v_lo + ks * 128, hi128, idesc_pv);
                    tc_commit(b_pvdone + 8 * pb);
                    tc_commit(b_vempty + 8 * st);
                    if (++st == STV) { st = 0; par ^= 1u; }
                }
                g += (uint32_t)nt;
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax + output (warps 2..5)
        const int quad = warp & 3, row = quad * 32 + lane;
        const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
        const uint8_t* q_row = base_ptr + row * 128;
        const uint8_t* qt_row = base_ptr + Cfg::Q_MAIN + row * 32;
        uint8_t* stage_row = out_ptr + row * Cfg::OUT_ROW;                       // this row in the output staging
        const uint32_t stage_warp = sm_out + (uint32_t)(quad * 32 * Cfg::OUT_ROW);  // this warp's 32 rows of it
        // This row of Q of the CTA's item number `item`: out of the swizzled tile (16-byte chunk c of a 128-byte row
        // sits at c ^ (row & 7); of a 32-byte row at c ^ ((row >> 2) & 1)) into tensor memory, two dims per column.
        // Called once every S product of the item before has completed (its last PV product was waited for).
        auto copy_q = [&](int item) {
            mbar_wait(b_qfull, (uint32_t)(item & 1), abort_flag, flags, 22);
            uint32_t qa[16];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint4 v = *reinterpret_cast<const uint4*>(q_row + (((4 * h + c) ^ (row & 7)) << 4));
                    qa[4 * c] = v.x; qa[4 * c + 1] = v.y; qa[4 * c + 2] = v.z; qa[4 * c + 3] = v.w;
                }
                tc_st_32x16(t_lane + T_Q + 16 * h, qa);
            }
            if (TAIL) {
                uint32_t qc[8];
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const uint4 v = *reinterpret_cast<const uint4*>(qt_row + ((c ^ ((row >> 2) & 1)) << 4));
                    qc[4 * c] = v.x; qc[4 * c + 1] = v.y; qc[4 * c + 2] = v.z; qc[4 * c + 3] = v.w;
                }
                tc_st_32x8(t_lane + T_Q + 32, qc);
            }
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(b_qcopied);
        };
        uint32_t g = 0;
        int it = 0;
        if (attn_walk(p, 0) >= 0) copy_q(0);
        for (int w; (w = attn_walk(p, it)) >= 0; ++it) {
            int qblk, head, batch;
            attn_item(p, w, qblk, head, batch);
            const int q0 = qblk * ABQ, nt = attn_tiles(p, q0), qi = q0 + row;
            const bool row_ok = qi < p.q_len;
            float m_run = -INFINITY, l_run = 0.f;  // exponent reference (log2 units) and row sum on that reference

            for (int j = 0; j < nt; ++j) {
                const uint32_t gj = g + (uint32_t)j;
                const int sb = (int)(gj & 1u), key0 = j * ABKV;
                mbar_wait(b_sfull + 8 * sb, (gj >> 1) & 1u, abort_flag, flags, 19);
                tc_fence_after();
                uint32_t s0[32], s1[32];
                tc_ld_32x32(t_lane + (uint32_t)(sb * 64), s0);
                tc_ld_32x32(t_lane + (uint32_t)(sb * 64 + 32), s1);
                tc_wait_ld();

                // tiles wholly inside the valid, visible region (all but the last ones) skip the per-key tests
                const bool interior = !p.mask && key0 + ABKV <= p.kv_len &&
                                      (p.causal_pos < 0 || key0 + ABKV - 1 <= p.causal_pos + q0 + quad * 32);
                if (!interior && !p.mask) {
                    // the visible keys of a row are a prefix of the tile: the first n_vis of its 64
                    int n_vis = p.kv_len - key0;
                    if (p.causal_pos >= 0) n_vis = min(n_vis, p.causal_pos + qi - key0 + 1);
                    if (!row_ok) n_vis = 0;
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        if (e >= n_vis) s0[e] = 0xff800000u;  // -inf
                        if (e + 32 >= n_vis) s1[e] = 0xff800000u;
                    }
                } else if (!interior) {
#pragma unroll
                    for (int e = 0; e < 64; ++e) {
                        const int key = key0 + e;
                        bool vis = row_ok && key < p.kv_len;
                        if (p.causal_pos >= 0) vis = vis && key <= p.causal_pos + qi;
                        if (vis && p.mask) vis = p.mask[(long long)qi * p.kv_len + key] != 0;
                        if (!vis) {
                            if (e < 32) s0[e] = 0xff800000u; else s1[e - 32] = 0xff800000u;  // -inf
                        }
                    }
                }
                // three-input max (two new values per instruction), eight independent chains of four
                float mx[8];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    mx[c] = fmaxf(__uint_as_float(s0[8 * c]), __uint_as_float(s0[8 * c + 1]));
                    mx[4 + c] = fmaxf(__uint_as_float(s1[8 * c]), __uint_as_float(s1[8 * c + 1]));
                }
#pragma unroll
                for (int e = 2; e < 8; e += 2) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        mx[c] = max3(mx[c], __uint_as_float(s0[8 * c + e]), __uint_as_float(s0[8 * c + e + 1]));
                        mx[4 + c] = max3(mx[4 + c], __uint_as_float(s1[8 * c + e]), __uint_as_float(s1[8 * c + e + 1]));
                    }
                }
                const float mt = fmaxf(max3(mx[0], mx[1], mx[2]), max3(max3(mx[3], mx[4], mx[5]), mx[6], mx[7])) *
                                 p.scale_log2;  // -inf stays -inf (scale > 0)

                if (j == 0) {
                    m_run = mt;
                } else if (__any_sync(0xffffffffu, mt > m_run + RESCALE_THRESHOLD)) {
                    // move this warp's rows to their new maxima: O(row) *= 2^(old - new), once PV(j-1) has landed
                    const float m_new = fmaxf(m_run, mt);
                    const float corr = (m_new == -INFINITY) ? 1.f : ex2_fast(m_run - m_new);
                    l_run *= corr;
                    m_run = m_new;
                    mbar_wait(b_pvdone + 8 * ((gj - 1) & 1u), ((gj - 1) >> 1) & 1u, abort_flag, flags, 21);
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < Cfg::DPAD / 16; ++c) {
                        uint32_t r[16];
                        tc_ld_32x16(t_lane + T_O + c * 16, r);
                        tc_wait_ld();
#pragma unroll
                        for (int e = 0; e < 16; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * corr);
                        tc_st_32x16(t_lane + T_O + c * 16, r);
                    }
                }
                const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;

                float rs[8];   // eight independent partial sums
#pragma unroll
                for (int c = 0; c < 8; ++c) rs[c] = 0.f;
                uint32_t pa[16], pb[16];   // P as packed f16: column c = keys 2c, 2c + 1
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const float a0 = ex2_fast(fmaf(__uint_as_float(s0[2 * e]), p.scale_log2, neg_m));
                    const float a1 = ex2_fast(fmaf(__uint_as_float(s0[2 * e + 1]), p.scale_log2, neg_m));
                    const float b0 = ex2_fast(fmaf(__uint_as_float(s1[2 * e]), p.scale_log2, neg_m));
                    const float b1 = ex2_fast(fmaf(__uint_as_float(s1[2 * e + 1]), p.scale_log2, neg_m));
                    rs[(e & 1) * 4] += a0; rs[(e & 1) * 4 + 1] += a1; rs[(e & 1) * 4 + 2] += b0; rs[(e & 1) * 4 + 3] += b1;
                    const __half2 ha = __floats2half2_rn(a0, a1), hb = __floats2half2_rn(b0, b1);
                    pa[e] = *reinterpret_cast<const uint32_t*>(&ha);
                    pb[e] = *reinterpret_cast<const uint32_t*>(&hb);
                }
                l_run += ((rs[0] + rs[1]) + (rs[2] + rs[3])) + ((rs[4] + rs[5]) + (rs[6] + rs[7]));

                // P over the first half of the S buffer it came from (this thread has its whole S row in registers)
                tc_st_32x16(t_lane + (uint32_t)(sb * 64), pa);
                tc_st_32x16(t_lane + (uint32_t)(sb * 64 + 16), pb);
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(b_pfull + 8 * sb);
            }

            // The item's output: out of tensor memory into registers first.  That frees O, and with it the next
            // item can start: its Q goes into tensor memory now, so its first S product runs while this item's
            // output is converted and stored.
            uint32_t o[Cfg::DPAD / 16][16];
            if (nt > 0) {
                const uint32_t gl = g + (uint32_t)nt - 1u;
                mbar_wait(b_pvdone + 8 * (gl & 1u), (gl >> 1) & 1u, abort_flag, flags, 18);
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < Cfg::DPAD / 16; ++c) tc_ld_32x16(t_lane + T_O + c * 16, o[c]);
                tc_wait_ld();
                tc_fence_before();
            } else {
#pragma unroll
                for (int c = 0; c < Cfg::DPAD / 16; ++c)
#pragma unroll
                    for (int e = 0; e < 16; ++e) o[c][e] = 0u;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(b_oempty);
            if (attn_walk(p, it + 1) >= 0) copy_q(it + 1);

            // One row per thread would be 32 scattered 16-byte pieces per store instruction; instead the warp's 32
            // rows are packed in shared memory and leave as one TMA store (rows past q_len are clipped by the map).
            if (lane == 0) tma_store_wait_read<0>();   // the previous item's store has read the staging rows
            __syncwarp();
            const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll
            for (int c = 0; c < Cfg::DPAD / 16; ++c) {
#pragma unroll
                for (int h8 = 0; h8 < 2; ++h8) {
                    if (c * 16 + h8 * 8 < D) {
                        uint32_t wv[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __half2 h = __floats2half2_rn(__uint_as_float(o[c][h8 * 8 + 2 * e]) * inv,
                                                                __uint_as_float(o[c][h8 * 8 + 2 * e + 1]) * inv);
                            wv[e] = *reinterpret_cast<const uint32_t*>(&h);
                        }
                        *reinterpret_cast<uint4*>(stage_row + (c * 16 + h8 * 8) * 2) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                    }
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0 && q0 + quad * 32 < p.q_len) {
                int co[4] = {0, 0, 0, 0};
                co[p.o_dim_row] = q0 + quad * 32; co[p.o_dim_head] = head; co[p.o_dim_batch] = batch;
                tma_store_4d(&tm.o, stage_warp, 0, co[1], co[2], co[3]);
                tma_store_commit();
            }
            g += (uint32_t)nt;
        }
        if (lane == 0) tma_store_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                     : "memory");
    }
}

}  // namespace

namespace {

// Orders (row, head, batch) by ascending stride for a 4-D tensor map whose dim 0 is the head dimension.
// An extent of 1 never moves, so its stride is free: it goes last with a stride past everything else.
struct MapPlan {
    uint64_t dims[4], strides_bytes[3];
    int dim_of[3];  // map dimension (1..3) of row, head, batch
};

bool plan_map(MapPlan& mp, size_t d, const size_t extent[3], const size_t stride[3]) {
    int order[3] = {0, 1, 2};
    auto key = [&](int r) { return extent[r] == 1 ? ~0ull : (unsigned long long)stride[r]; };
    for (int i = 0; i < 3; ++i)
        for (int j = i + 1; j < 3; ++j)
            if (key(order[j]) < key(order[i])) { int t = order[i]; order[i] = order[j]; order[j] = t; }
    mp.dims[0] = d;
    unsigned long long next_free = (d + 7) / 8 * 8;  // stride (elements) that clears every dimension placed so far
    for (int i = 0; i < 3; ++i) {
        const int r = order[i];
        unsigned long long st = extent[r] == 1 ? next_free : (unsigned long long)stride[r];
        if (st == 0 || (st % 8) != 0 || st * 2 >= (1ull << 40) || extent[r] == 0 || extent[r] > (1ull << 31)) return false;
        mp.dims[i + 1] = extent[r];
        mp.strides_bytes[i] = st * 2;
        mp.dim_of[r] = i + 1;
        const unsigned long long span = st * extent[r];
        if (span > next_free) next_free = (span + 7) / 8 * 8;
    }
    return true;
}

template <int D>
int launch_attn_tc(md_ctx* ctx, const AttnTcMaps& maps, const AttnTcParams& p, dim3 grid) {
    auto kern = attn_tc_kernel<D>;
    const uint32_t cfg_bit = 1u << (D == 64 ? 8 : 9);
    if (!(ctx->tc_configured & cfg_bit)) {
        MD_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnCfg<D>::SMEM));
        ctx->tc_configured |= cfg_bit;
    }
    return md_launch_ex(ctx, kern, grid, dim3(ATTN_THREADS), AttnCfg<D>::SMEM, "attn_tc_kernel", maps, p, ctx->flags);
}

}  // namespace

// True when the tcgen05 attention can address these operands: d = 64 or 72, 16-byte aligned bases and strides.
bool md_sdpa_tc_supported(const void* q, const void* k, const void* v, const void* out, size_t d, size_t q_row,
                          size_t q_head, size_t q_batch, size_t kv_row, size_t kv_head, size_t kv_batch, size_t o_row,
                          size_t o_head, size_t o_batch, size_t n_heads, size_t batch) {
    if (d != 64 && d != 72) return false;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
         reinterpret_cast<uintptr_t>(out)) & 15)
        return false;
    const size_t st[] = {q_row, kv_row, o_row, n_heads > 1 ? q_head : 8, n_heads > 1 ? kv_head : 8,
                         n_heads > 1 ? o_head : 8, batch > 1 ? q_batch : 8, batch > 1 ? kv_batch : 8,
                         batch > 1 ? o_batch : 8};
    for (size_t s : st)
        if (s == 0 || (s % 8) != 0) return false;
    return n_heads <= 65535 && batch <= 65535;
}

int md_launch_sdpa_tc(md_ctx* ctx, const __half* q, const __half* k, const __half* v, const uint8_t* mask, __half* out,
                      size_t n_heads, size_t q_len, size_t kv_len, size_t d, size_t q_row, size_t q_head, size_t kv_row,
                      size_t kv_head, size_t o_row, size_t o_head, size_t batch, size_t q_batch, size_t kv_batch,
                      size_t o_batch, int causal_pos) {
    if (!md_sdpa_tc_supported(q, k, v, out, d, q_row, q_head, q_batch, kv_row, kv_head, kv_batch, o_row, o_head, o_batch,
                              n_heads, batch))
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "tcgen05 attention needs d = 64 or 72 and 16-byte aligned operands");
    MapPlan mq, mk;
    const size_t eq[3] = {q_len, n_heads, batch}, sq[3] = {q_row, q_head, q_batch};
    const size_t ek[3] = {kv_len, n_heads, batch}, sk[3] = {kv_row, kv_head, kv_batch};
    if (!plan_map(mq, d, eq, sq) || !plan_map(mk, d, ek, sk))
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "tcgen05 attention: strides not addressable by a tensor map");
    AttnTcMaps maps;
    uint32_t boxq[3] = {1, 1, 1}, boxk[3] = {1, 1, 1};
    boxq[mq.dim_of[0] - 1] = ABQ;
    boxk[mk.dim_of[0] - 1] = ABKV;
    MD_TRY(md_make_map_4d(ctx, &maps.q, q, mq.dims, mq.strides_bytes, 64, boxq, 128));
    MD_TRY(md_make_map_4d(ctx, &maps.k, k, mk.dims, mk.strides_bytes, 64, boxk, 128));
    MD_TRY(md_make_map_4d(ctx, &maps.v, v, mk.dims, mk.strides_bytes, 64, boxk, 128));
    if (d > 64) {
        MD_TRY(md_make_map_4d(ctx, &maps.qt, q, mq.dims, mq.strides_bytes, 16, boxq, 32));
        MD_TRY(md_make_map_4d(ctx, &maps.kt, k, mk.dims, mk.strides_bytes, 16, boxk, 32));
        MD_TRY(md_make_map_4d(ctx, &maps.vt, v, mk.dims, mk.strides_bytes, 64, boxk, 128));   // dims 64..127: 72.. zero fill
    } else {
        maps.qt = maps.q; maps.kt = maps.k; maps.vt = maps.v;
    }
    MapPlan mo;
    const size_t eo[3] = {q_len, n_heads, batch}, so[3] = {o_row, o_head, o_batch};
    if (!plan_map(mo, d, eo, so))
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "tcgen05 attention: output strides not addressable by a tensor map");
    uint32_t boxo[3] = {1, 1, 1};
    boxo[mo.dim_of[0] - 1] = 32;
    MD_TRY(md_make_map_4d(ctx, &maps.o, out, mo.dims, mo.strides_bytes, (uint32_t)d, boxo, 0));
    AttnTcParams p;
    p.q_len = (int)q_len; p.kv_len = (int)kv_len; p.causal_pos = causal_pos;
    p.scale_log2 = (1.0f / sqrtf((float)d)) * LOG2E_F;
    p.mask = mask;
    p.q_dim_row = mq.dim_of[0]; p.q_dim_head = mq.dim_of[1]; p.q_dim_batch = mq.dim_of[2];
    p.kv_dim_row = mk.dim_of[0]; p.kv_dim_head = mk.dim_of[1]; p.kv_dim_batch = mk.dim_of[2];
    p.o_dim_row = mo.dim_of[0]; p.o_dim_head = mo.dim_of[1]; p.o_dim_batch = mo.dim_of[2];
    p.n_qblk = (int)((q_len + ABQ - 1) / ABQ); p.n_heads = (int)n_heads; p.n_batch = (int)batch;
    const size_t n_items = (size_t)p.n_qblk * n_heads * batch;
    if (n_items > (size_t)INT_MAX) return md_fail(ctx, MD_ERR_UNSUPPORTED, "tcgen05 attention: too many query blocks");
    p.n_items = (int)n_items;
    // at most two CTAs per SM (what fits); option attn_ctas_per_sm = 0 gives every item its own CTA
    size_t ctas = n_items;
    if (ctx->attn_ctas_per_sm > 0) ctas = std::min(n_items, (size_t)ctx->attn_ctas_per_sm * (size_t)ctx->sm_count);
    dim3 grid((unsigned)ctas);
    return d == 64 ? launch_attn_tc<64>(ctx, maps, p, grid) : launch_attn_tc<72>(ctx, maps, p, grid);
}
