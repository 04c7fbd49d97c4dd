// Internal declarations shared by the translation units of libmoondream_b200.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/moondream_b200.h"

// Device-side error word: bit 0 = a bounded wait gave up.  One word per context,
// zeroed at md_init and re-zeroed by md_sync after it has been reported.
struct md_devflags {
    unsigned int error;
    unsigned int where;    // site id of the first wait that gave up
    unsigned int* mirror;  // word in mapped pinned host memory, set to 1 together with `error`: the host can
                           // tell "nothing went wrong" after a stream synchronize without a copy
};
#ifdef __CUDACC__
// Record that a bounded device-side wait gave up at `site` (first site wins).
__device__ __forceinline__ void md_flag_timeout(md_devflags* flags, unsigned site) {
    if (atomicOr(&flags->error, 1u) == 0u) {
        flags->where = site;
        if (flags->mirror) {
            *reinterpret_cast<volatile unsigned int*>(flags->mirror) = 1u;
            __threadfence_system();
        }
    }
}
#endif

struct md_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
};

constexpr size_t MD_COUNTER_WORDS = 256;
constexpr size_t MD_SPLITK_TICKETS = 1024;   // tiles of a split-K GEMM (one arrival ticket each)

struct md_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    md_devflags* flags = nullptr;       // device
    md_devflags* flags_host = nullptr;  // pinned host copy of *flags (read back when the mirror word is set)
    unsigned int* mirror_host = nullptr;  // pinned, mapped: the word md_devflags::mirror points at
    std::string last_error;
    uint64_t launches = 0;
    int gemm_mode = 0;
    // staging buffers for host-pointer ("drop-in") calls, grown on demand
    struct Stage { void* ptr = nullptr; size_t cap = 0; };
    std::vector<Stage> stage;
    // split-K GEMM: f32 partial tiles and arrival tickets, one set per stream that has used it (the two chains of a
    // forked layer run such products at the same time); tickets are zero between launches
    struct SplitK { cudaStream_t stream = nullptr; float* part = nullptr; size_t cap = 0; unsigned* tickets = nullptr; };
    std::vector<SplitK> splitk;
    int push_tma = 1;           // md_set_option("push_tma"): column-split GEMM pushes by TMA stores from the epilogue's staging
                                // buffers (1, default) or by the push warps' plain stores (0)
    int tc_splitk = 0;          // md_set_option("tc_splitk"): 0 never (default), -1 the cost model decides, n >= 2 always n ranges
    // scratch for kernels that need global memory beyond inputs and outputs
    void* scratch = nullptr;
    size_t scratch_cap = 0;
    // per-head arrival counters of the split-KV decode attention (MD_COUNTER_WORDS words): zero between launches
    unsigned int* counters = nullptr;
    // cuTensorMapEncodeTiled resolved through the runtime (no link against libcuda)
    void* encode_tiled = nullptr;
    uint32_t pair_configured = 0;  // the same for the instantiations of gemm_pair_kernel
    uint32_t tc_configured = 0;  // tcgen05 kernels whose dynamic shared memory limit has been raised
    int skinny = 1;          // md_set_option("skinny"): 8 < M <= 64 takes the swapped-operand split-K kernel
    int skinny_splits = 0;   // md_set_option("skinny_splits"): 0 = automatic, else the number of K splits (tests)
    bool sdpa_mma_configured = false;  // the same for the mma.sync attention kernels
    // (cos, sin) table shared by the fused attention calls: [rope_rows][rope_dim/2][2] f32
    float* rope_tab = nullptr;
    size_t rope_rows = 0, rope_dim = 0;
    float rope_theta = 0.f;
    bool capturing = false;  // between md_graph_begin and md_graph_end
    // Bumped whenever something a captured graph may have baked in changes: the scratch buffer or the rope table
    // moved (md_scratch / md_rope_cached reallocated them) or an option that selects kernels was set.  The model
    // runners store the value with every graph they keep and capture again when it differs.
    uint64_t generation = 0;
    int gemv_variant = 0;    // md_set_option("gemv_variant")
    int gemv_ksplit = 0;     // md_set_option("gemv_ksplit"): 0 = automatic, 1 / 2 / 4 / 8 = K splits of the GEMV kernel
    int tc_block_n = 0;      // md_set_option("tc_block_n")
    int tc_pair = -1;        // md_set_option("tc_pair"): 1 = every tcgen05 GEMM runs on CTA pairs, 0 = never, -1 = by shape
    int last_tc_tile = 0;    // md_get_option("last_tc_tile"): tile of the last tcgen05 GEMM launch (64/128/256, 512 = 256 x 256)
    int decode_cluster_ok = -1;    // -1 unknown, 0/1: 16-CTA clusters usable for the decode attention merge
    int decode_cluster_mode = -1;  // md_set_option("decode_cluster"): 0 forces the scratch-based merge
    int dualk_variant = 0;   // md_set_option("dualk_variant"): (warps, unroll) of gemv_dual_k_kernel
    int fused_decode = 1;    // md_set_option("fused_decode"): decode layers as 3 fused kernels
    int pdl = 0;             // md_set_option("pdl"): programmatic dependent launch for the GEMV kernels
    int prefill_fork = 1;       // md_set_option("prefill_fork"): prefill layers run the MLP beside the attention
    int decode_split_ln = 5;    // md_set_option("decode_split_ln"): from this many rows on a decode step runs the LayerNorm once
    int decode_fork = 1;        // md_set_option("decode_fork"): a decode layer runs as two concurrent kernel chains
    int attn_ctas_per_sm = 2;   // md_set_option("attn_ctas_per_sm"): grid of the tcgen05 attention = this many CTAs per SM, each
                                // walking several (query block, head, batch) items; 0 = one CTA per item
    int decode_loop = -1;       // md_set_option("decode_loop"): batched decode attention as one CTA per (head, request) when there
                                // are at least this many pairs; -1 = 128, 0 = never
    int decode_mlp_split = 2;   // md_set_option("decode_mlp_split"): single-request decode runs the MLP as 2 or 4 chains (0 = one)
    cudaStream_t side_stream = nullptr;  // second chain of the forked decode layer
    cudaStream_t mlp_stream[3] = {};     // further chains when the MLP is split (its first part runs on side_stream)
    cudaEvent_t ev_fork = nullptr, ev_side = nullptr, ev_mlp[3] = {};
    int attn_tc = -1;        // md_set_option("attn_tc"): -1 auto, 0 mma.sync attention only, 1 tcgen05 attention only
};

int md_fail(md_ctx* ctx, int status, const char* fmt, ...);
#define MD_CUDA(ctx, expr)                                                                      \
    do {                                                                                        \
        cudaError_t _e = (expr);                                                                \
        if (_e != cudaSuccess)                                                                  \
            return md_fail((ctx), _e == cudaErrorMemoryAllocation ? MD_ERR_OOM : MD_ERR_CUDA,   \
                           "%s failed: %s", #expr, cudaGetErrorString(_e));                     \
    } while (0)
#define MD_TRY(expr)                    \
    do {                                \
        int _s = (expr);                \
        if (_s != MD_OK) return _s;     \
    } while (0)

// Launch through cudaLaunchKernelEx so that the context's launch attributes apply: with ctx->pdl the kernel
// is programmatically dependent on its predecessor in the stream (it may start while that one drains; it must
// execute griddepcontrol.wait before touching anything an earlier kernel produces or still reads).
#ifdef __CUDACC__
template <class... KArgs, class... Args>
int md_launch_ex(md_ctx* ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, const char* name,
                 Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) return md_fail(ctx, MD_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e));
    ctx->launches++;
    return MD_OK;
}
// Device side of the protocol: let the successor start its prologue, then wait for the predecessor.
__device__ __forceinline__ void md_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void md_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif


// The context's rope table for (rot_dim, theta), covering at least `rows` positions; built on first use.
int md_rope_cached(md_ctx* ctx, size_t rot_dim, float theta, size_t rows, const float** out);
// Ensure ctx->scratch holds at least `bytes`.
int md_scratch(md_ctx* ctx, size_t bytes, void** out);
int md_splitk_workspace(md_ctx* ctx, size_t bytes, float** part, unsigned** tickets);

// Host-or-device argument resolution for drop-in calls.
bool md_is_device_ptr(const void* p);
struct md_arg {
    const void* user = nullptr;
    void* dev = nullptr;
    size_t bytes = 0;
    bool staged = false;
    bool mapped = false;  // output written by the kernel straight into mapped pinned host memory
};
// Bring an input to the device (no-op for device pointers). slot selects the staging buffer.
int md_stage_in(md_ctx* ctx, int slot, const void* user, size_t bytes, md_arg* out);
// Reserve device space for an output (no-op for device pointers).
int md_stage_out(md_ctx* ctx, int slot, void* user, size_t bytes, md_arg* out);
// As md_stage_out, but a small output in pinned, mapped host memory is handed to the kernel directly
// (only for kernels that write with plain stores).
int md_stage_out_mapped(md_ctx* ctx, int slot, void* user, size_t bytes, md_arg* out);
// Copy a staged output back and wait; for device outputs nothing happens.
int md_finish_out(md_ctx* ctx, md_arg* out);
// After a drop-in call whose output was a host buffer: check the device error word.
int md_check_flags(md_ctx* ctx);

// ---- kernel launchers (device pointers only) ------------------------------------
struct md_epilogue {
    const __half* bias = nullptr;       // [N] or null
    const __half* residual = nullptr;   // [M,N] (or [residual_rows,N] repeated every residual_rows rows) or null
    const __half* residual2 = nullptr;  // [M,N] or null, added after `residual`
    int gelu = 0;
    int residual_rows = 0;              // > 0: row m reads residual row m % residual_rows (broadcast over batches)
    // GEMV kernels only (the decode layer whose MLP runs as two half-width chains):
    float* out_f32 = nullptr;           // store the raw f32 sums [M,N] here instead of the f16 result (no glue)
    const float* parts = nullptr;       // n_parts f32 partial products [M,N] (part_stride floats apart) of another
    int n_parts = 0;                    //   projection and its bias: f16(f16(sum of the parts) + bias2) is added where
    int part_stride = 0;                //   `residual` would be
    const __half* bias2 = nullptr;
};

// Column-split GEMM: finished C chunks are also stored into the other GPUs' buffers.
struct md_push {
    int n = 0;                 // number of peers (0 = none)
    long long ld = 0;          // row stride of the peers' C in elements
    __half* base[7] = {};      // peer pointers to element (0, 0) of this rank's column block
    const __half* self = nullptr;  // the same element of this rank's own C (the push warps read the tile back from it)
    int tma = 0;               // 1: the epilogue warps send each staged chunk to the peers with TMA stores (no push warps)
};

// Tensor maps over the peers' copies of this rank's column block (column-split GEMM with TMA pushes).
struct md_peer_maps {
    CUtensorMap m[7];
};

// gemv.cu: C[M,N] = A[M,K] . Bt[N,K]^T for M <= 8, K % 8 == 0.
int md_launch_gemv_nt(md_ctx* ctx, const __half* a, const __half* bt, __half* c, size_t M, size_t N, size_t K,
                      const md_epilogue& ep, size_t ldb = 0);  // ldb: row stride of Bt in elements (0 = K)
// gemv_fused.cu: the decode layer's GEMVs fused with the glue around them (M <= 8 rows).
//   ln_dual: y = LayerNorm(hidden); out1 = y W1^T + b1; out2 = gelu(y W2^T + b2)      (K = 2048)
//   dual_k : hidden += (x1 W1^T + b1) + (x2 W2^T + b2), with the reference's f16 rounding points
bool md_gemv_ln_dual_supported(size_t M, size_t K, size_t n1, size_t n2);
int md_launch_gemv_ln_dual(md_ctx* ctx, const __half* hidden, const __half* ln_w, const __half* ln_b, float eps,
                           const __half* w1, const __half* b1, __half* out1, size_t n1, const __half* w2,
                           const __half* b2, __half* out2, size_t n2, size_t M, size_t K,
                           unsigned long long* amax = nullptr,  // amax: optional [M] argmax keys of out1
                           bool gelu1 = false);                 // GELU on segment 1 too
bool md_gemv_dual_k_supported(size_t M, size_t N, size_t k1, size_t k2);
int md_launch_gemv_dual_k(md_ctx* ctx, const __half* x1, const __half* w1, const __half* b1, size_t k1,
                          const __half* x2, const __half* w2, const __half* b2, size_t k2, __half* hidden, size_t N,
                          size_t M);
// gemm_simt.cu: any shape; b_layout 0 = [K,N], 1 = [N,K].
int md_launch_gemm_simt(md_ctx* ctx, const __half* a, const __half* b, __half* c, size_t M, size_t N, size_t K,
                        int b_layout, const md_epilogue& ep);
// gemm_tc.cu: tcgen05 + TMA; returns MD_ERR_UNSUPPORTED when alignment rules are not met.
bool md_gemm_tc_supported(const void* a, const void* b, const void* c, size_t M, size_t N, size_t K, int b_layout);
int md_launch_gemm_tc(md_ctx* ctx, const __half* a, const __half* b, __half* c, size_t M, size_t N, size_t K,
                      int b_layout, const md_epilogue& ep);
// as above with an output row stride ldc >= N (C is a column block of a wider matrix) and peer pushes
int md_launch_gemm_tc_ex(md_ctx* ctx, const __half* a, const __half* b, __half* c, size_t M, size_t N, size_t K,
                         int b_layout, const md_epilogue& ep, size_t ldc, const md_push& push);

// comm.cu: gathered [world][M][n_local] -> c [M][world * n_local] (n_local % 8 == 0, 16-byte aligned)
int md_launch_gather_colblocks(md_ctx* ctx, const uint16_t* gathered, uint16_t* c, size_t world, size_t M, size_t n_local);

// gemm_skinny.cu: 8 < M <= 64, weights as the MMA's M side, split-K over a thread-block cluster
bool md_gemm_skinny_supported(const void* a, const void* b, const void* c, size_t M, size_t N, size_t K);
int md_launch_gemm_skinny(md_ctx* ctx, const __half* a, const __half* b, __half* c, size_t M, size_t N, size_t K,
                          int b_layout, const md_epilogue& ep);

// gemm_pair.cu: 256 x 256 tiles on CTA pairs (tcgen05 cta_group::2); same operand rules as md_launch_gemm_tc
int md_launch_gemm_pair(md_ctx* ctx, const __half* a, const __half* b, __half* c, size_t M, size_t N, size_t K, int b_layout,
                        const md_epilogue& ep, size_t ldc, const md_push& push);

// gemm_tc.cu: a kernel whose bounded wait runs out on purpose (md_selftest_bounded_wait)
int md_launch_selftest_wait(md_ctx* ctx, unsigned limit_ms);

// attention.cu
int md_launch_sdpa(md_ctx* ctx, const __half* q, const __half* k, const __half* v, const uint8_t* mask, __half* out,
                   size_t n_heads, size_t q_len, size_t kv_len, size_t d,
                   // strides in elements: q/out row stride and head stride, k/v row stride and head stride
                   size_t q_row, size_t q_head, size_t kv_row, size_t kv_head, size_t o_row, size_t o_head,
                   size_t batch, size_t q_batch, size_t kv_batch, size_t o_batch, int causal_pos);
// attention_tc.cu: the same contract on tcgen05 tensor cores (d = 64 or 72, 16-byte aligned operands)
bool md_sdpa_tc_supported(const void* q, const void* k, const void* v, const void* out, size_t d, size_t q_row,
                          size_t q_head, size_t q_batch, size_t kv_row, size_t kv_head, size_t kv_batch, size_t o_row,
                          size_t o_head, size_t o_batch, size_t n_heads, size_t batch);
int md_launch_sdpa_tc(md_ctx* ctx, const __half* q, const __half* k, const __half* v, const uint8_t* mask, __half* out,
                      size_t n_heads, size_t q_len, size_t kv_len, size_t d, size_t q_row, size_t q_head, size_t kv_row,
                      size_t kv_head, size_t o_row, size_t o_head, size_t batch, size_t q_batch, size_t kv_batch,
                      size_t o_batch, int causal_pos);
int md_launch_sdpa_single(md_ctx* ctx, const __half* q, const __half* k, const __half* v, const uint8_t* mask,
                          __half* out, size_t kv_len);
int md_launch_sdpa_decode_fused(md_ctx* ctx, const __half* qkv_row, __half* kc, __half* vc, __half* out,
                                size_t n_heads, size_t d, size_t max_seq, size_t pos, size_t rot_dim, float theta);
int md_launch_rope_cache_write(md_ctx* ctx, const __half* qkv, __half* q_rot, __half* kc, __half* vc, size_t S,
                               size_t n_heads, size_t d, size_t max_seq, size_t pos, size_t rot_dim, float theta);

// glue.cu
int md_launch_layernorm(md_ctx* ctx, const __half* x, const __half* w, const __half* b, __half* y, size_t rows,
                        size_t cols, float eps);
int md_launch_gelu(md_ctx* ctx, __half* x, size_t n);
int md_launch_bias_add(md_ctx* ctx, __half* a, const __half* b, size_t rows, size_t cols);
int md_launch_add(md_ctx* ctx, __half* a, const __half* b, size_t n);
int md_launch_argmax(md_ctx* ctx, const __half* x, size_t n, unsigned long long* idx_dev);
int md_launch_argmax_rows(md_ctx* ctx, const __half* x, size_t n, size_t stride, size_t rows, unsigned long long* idx_dev);
int md_launch_patchify(md_ctx* ctx, const uint8_t* img, __half* out, size_t crops, size_t h, size_t w, size_t patch,
                       size_t out_stride);
int md_launch_rope_table(md_ctx* ctx, float* table, size_t dim, size_t end, float theta);
int md_launch_rope_apply(md_ctx* ctx, const __half* x, __half* out, size_t n_heads, size_t seq_len, size_t d,
                         const float* freqs, const unsigned long long* pos, size_t rot_dim);
int md_launch_mask(md_ctx* ctx, uint8_t* mask, size_t pos, size_t seq_len);
int md_launch_kv_update(md_ctx* ctx, __half* kc, __half* vc, const __half* k, const __half* v, size_t n_heads,
                        size_t max_seq, size_t d, size_t cur_len, size_t seq_len);
int md_launch_kv_active(md_ctx* ctx, const __half* kc, const __half* vc, __half* k, __half* v, size_t n_heads,
                        size_t max_seq, size_t d, size_t cur_len);

#define MD_LAUNCH_CHECK(ctx, name)                                                             \
    do {                                                                                       \
        cudaError_t _e = cudaGetLastError();                                                   \
        if (_e != cudaSuccess)                                                                 \
            return md_fail((ctx), MD_ERR_CUDA, "launch of %s failed: %s", name,                \
                           cudaGetErrorString(_e));                                            \
        (ctx)->launches++;                                                                     \
    } while (0)

// ---- device helpers ----------------------------------------------------------------
#ifdef __CUDACC__
// The reference's rounding points for the glue fused into GEMM epilogues.
__device__ __forceinline__ float md_round_f16(float v) { return __half2float(__float2half_rn(v)); }

__device__ __forceinline__ float md_gelu_f32(float v) {
    // ops.zig:1641-1642: sqrt(2/pi) and 0.044715 are f16 constants in the reference.
    const float c = 0.7978515625f, a = 0.044708251953125f;
    const float inner = c * (v + a * (v * v * v));
    return 0.5f * v * (1.0f + tanhf(inner));
}

// The same GELU with the hardware tanh (tanh.approx.f32, one special-function op; absolute error about 5e-4 on the
// tanh, i.e. at most 0.5 * |x| * 5e-4 on the result, a fraction of the f16 spacing at |x| and far inside the parity
// bar), for the GEMM epilogues where tanhf, or an exp and a divide, would cost more than the tile's MMAs: with the
// exp / divide form the bias + GELU epilogue of a 128 x 256 tile took longer than its 18 k-blocks of MMAs.
__device__ __forceinline__ float md_gelu_fast_f32(float v) {
    const float c = 0.7978515625f, a = 0.044708251953125f;
    const float inner = c * (v + a * (v * v * v));
    float th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(inner));
    const float hv = 0.5f * v;
    return fmaf(hv, th, hv);
}

// acc (f32 accumulator) -> f16 value after the fused glue, as f32 holding an f16-representable value.
__device__ __forceinline__ float md_apply_epilogue(float acc, float bias, bool has_bias, bool gelu, float resid,
                                                   bool has_resid) {
    float v = md_round_f16(acc);
    if (has_bias) v = md_round_f16(v + bias);
    if (gelu) v = md_round_f16(md_gelu_f32(v));
    if (has_resid) v = md_round_f16(v + resid);
    return v;
}

// The fused glue for output element (m, n): f16(acc) -> +bias -> gelu -> +residual -> +residual2, one
// rounding to f16 after every step, exactly where the reference's separate ops round.
__device__ __forceinline__ float md_epilogue_value(const md_epilogue& ep, float acc, int m, int n, int N) {
    float v = md_round_f16(acc);
    if (ep.bias) v = md_round_f16(v + __half2float(ep.bias[n]));
    if (ep.gelu) v = md_round_f16(md_gelu_f32(v));
    if (ep.residual) {
        const int rm = ep.residual_rows > 0 ? m % ep.residual_rows : m;
        v = md_round_f16(v + __half2float(__ldcg(ep.residual + (size_t)rm * N + n)));
    }
    if (ep.parts) {
        // the other projection arrives as parts of its K sum: one rounding of the sum, then its bias
        float r = 0.f;
        for (int i = 0; i < ep.n_parts; ++i) r += __ldcg(ep.parts + (size_t)i * ep.part_stride + (size_t)m * N + n);
        r = md_round_f16(md_round_f16(r) + __half2float(ep.bias2[n]));
        v = md_round_f16(v + r);
    }
    if (ep.residual2) v = md_round_f16(v + __half2float(__ldcg(ep.residual2 + (size_t)m * N + n)));
    return v;
}
#endif
