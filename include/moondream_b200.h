/*
 * moondream_b200 — C ABI of the B200 (sm_100a) replacement for moondream-zig's
 * FP16 matmul + attention hot path (src/core/{hgemm,hgemm_trans,attention,rope}.zig
 * and the glue ops of src/core/ops.zig that sit between the GEMMs).
 *
 * Conventions
 *  - f16 tensors are IEEE binary16 passed as `const uint16_t*` / `uint16_t*`,
 *    row-major, with explicit sizes (`size_t`, the reference's `usize`).  The
 *    reference's `Tensor(T)` struct is never passed: the Zig shim hands over
 *    `tensor.data.ptr` and the dims.
 *  - Every data pointer may be a HOST pointer or a DEVICE pointer of the
 *    context's GPU (decided per pointer with cudaPointerGetAttributes):
 *      host   -> "drop-in" mode: the call stages the buffer through device memory
 *                owned by the context and returns when the result is back in the
 *                caller's buffer (the reference's calls are synchronous).
 *      device -> "resident" mode: the kernel is enqueued on the context's stream
 *                and the call returns immediately; md_sync() waits.
 *    A call whose OUTPUT is a host buffer always returns completed.
 *  - Weights live for the whole process in the reference (preslice_text.zig:53-79);
 *    upload them once with md_upload() and pass the returned device pointer to
 *    the GEMM entry points.  Nothing is cached by host address (the reference's
 *    slab allocator recycles addresses, slab_reusing_allocator.zig:141-156).
 *  - Every function returns an md_status; md_last_error() describes the last failure.
 *  - One context per GPU, used from one thread at a time.  No entry point ever
 *    falls back to the CPU: without a usable sm_100a device md_init fails.
 */
#ifndef MOONDREAM_B200_H
#define MOONDREAM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum md_status {
    MD_OK = 0,
    MD_ERR_INVALID_ARG = 1,      /* null pointer, zero size */
    MD_ERR_INVALID_DIMENSION = 2,/* error.InvalidTensorDimension / InvalidInputDimensions */
    MD_ERR_SHAPE = 3,            /* error.IncompatibleTensorShapes */
    MD_ERR_SEQUENCE_TOO_LONG = 4,/* error.SequenceTooLong (attention.zig:769, text_model.zig:478) */
    MD_ERR_INVALID_ROT_DIM = 5,  /* error.InvalidRotationDimension (rope.zig:141-143) */
    MD_ERR_UNSUPPORTED = 6,
    MD_ERR_OOM = 7,              /* error.OutOfMemory */
    MD_ERR_CUDA = 8,
    MD_ERR_TIMEOUT = 9,          /* a bounded device-side wait gave up; results are invalid */
    MD_ERR_NO_DEVICE = 10,
    MD_ERR_IO = 11,              /* a file could not be opened, mapped or read to its stated length (error.InvalidRead) */
    MD_ERR_FORMAT = 12,          /* a weight file that is not what weights.zig accepts; md_last_error names the Zig error */
    MD_ERR_NCCL = 13             /* NCCL is missing or one of its calls failed (column-split GEMM across GPUs only) */
} md_status;

typedef struct md_ctx md_ctx;

/* ---- context, memory, streams ------------------------------------------------ */

/* Create a context on CUDA device `device`.  Fails with MD_ERR_NO_DEVICE when the
 * device is absent or is not compute capability 10.x. */
int md_init(md_ctx** out, int device);
int md_destroy(md_ctx* ctx);
/* Human-readable description of the last error on this context ("" if none).
 * ctx may be NULL: then the last md_init failure is described. */
const char* md_last_error(const md_ctx* ctx);
/* Wait for everything enqueued on the context's stream; reports MD_ERR_TIMEOUT if
 * any kernel since the last md_sync gave up on a bounded wait. */
int md_sync(md_ctx* ctx);
/* Self-test of the failure path (no counterpart in the reference): enqueues one small kernel whose only
 * thread waits on a barrier that nothing ever completes.  The wait is bounded like every wait in this
 * library: it gives up after `limit_ms` milliseconds (1..2000), records the failure and the kernel ends
 * normally.  The next md_sync() (or the next call with a host output) then returns MD_ERR_TIMEOUT, after
 * which the context is clean and usable again.  Nothing faults or hangs. */
int md_selftest_bounded_wait(md_ctx* ctx, unsigned limit_ms);
/* Use an existing cudaStream_t (e.g. the harness's stream) instead of the
 * context's own.  NULL restores the context's own stream. */
int md_set_stream(md_ctx* ctx, void* cuda_stream);
/* Device memory owned by the caller until md_free. */
int md_alloc(md_ctx* ctx, size_t bytes, void** dev_out);
int md_free(md_ctx* ctx, void* dev);
/* md_alloc + host->device copy: the "register a weight once" call. */
int md_upload(md_ctx* ctx, const void* host, size_t bytes, void** dev_out);
int md_memcpy_h2d(md_ctx* ctx, void* dev, const void* host, size_t bytes);
int md_memcpy_d2h(md_ctx* ctx, void* host, const void* dev, size_t bytes);
/* Number of kernels of this library launched on the context since md_init. */
int md_launch_count(const md_ctx* ctx, uint64_t* count_out);
/* Select the GEMM kernel: 0 = automatic (tcgen05 when the operands meet the TMA
 * alignment rules, SIMT otherwise), 1 = force the SIMT kernel, 2 = force tcgen05
 * (MD_ERR_UNSUPPORTED when the shape cannot take it).  For tests and profiling. */
int md_set_gemm_mode(md_ctx* ctx, int mode);

/* Tuning knobs for tests and profiling; unknown keys return MD_ERR_INVALID_ARG.
 *   "gemv_variant"  0 = automatic, 1..6 = a fixed (warps, unroll) configuration of the GEMV kernel
 *   "gemv_ksplit"   0 = automatic, 1 / 2 / 4 / 8 = number of K splits of the GEMV kernel (the CTAs of a thread-block
 *                   cluster stream K / S each and add their sums through distributed shared memory)
 *   "tc_block_n"    0 = automatic, 64 / 128 / 256 = fixed tile width of the tcgen05 GEMM (128-row tiles),
 *                   512 = the 256 x 256 tile
 *   "tc_pair"       -1 (default) = shapes that would take the 128 x 256 tile and have more than 256 rows run
 *                   256 x 256 tiles on CTA pairs (tcgen05 cta_group::2: each CTA of a cluster of two loads its 128 rows
 *                   of A and half of the B tile, one thread issues the MMAs for both); 1 = every tcgen05 GEMM does;
 *                   0 = single-CTA tiles only.  Same results bit for bit
 *   "skinny"        1 (default) = products with 8 < M <= 64 rows take the swapped-operand split-K kernel (weights on
 *                   the MMA's M side, K split over the CTAs of a thread-block cluster, ~2 CTAs per SM, partials
 *                   added through distributed shared memory)
 *   "skinny_splits" 0 = automatic, else the number of K splits of that kernel (rounded down to 1, 2, 4 or 8)
 *   "pdl"           1 = launch the GEMV kernels with programmatic dependent launch: a kernel starts
 *                   streaming its weights while its predecessor on the stream drains.  Only for streams
 *                   on which no earlier kernel writes the weight matrices (registered weights).
 *   "fused_decode"  1 (default) = a decode layer runs as three fused kernels, 0 = one kernel per reference op
 *   "dualk_variant" 0..4 = (warps, unroll) of the out-proj + fc2 kernel of the fused decode layer
 *   "decode_cluster" 1 = merge the key splits of the decode attention through the shared memory of a 16-CTA cluster;
 *                   0 / -1 (default) = through global scratch and an arrival ticket
 *   "decode_split_ln" n (default 5): a decode step over >= n rows runs each LayerNorm once as its own kernel followed by
 *                   plain GEMVs with fused epilogues, instead of the kernels that recompute it in every CTA; 0 = never
 *   "attn_tc"       -1 (default) = tcgen05 attention when the operands allow it and q_len > 64,
 *                   0 = mma.sync attention only, 1 = tcgen05 only (MD_ERR_UNSUPPORTED otherwise)
 *   "prefill_fork"  1 (default) = a prefill layer runs fc1 -> fc2 as a second kernel chain beside the attention
 *   "decode_fork"   1 (default) = the fused decode layer runs as two concurrent kernel chains (q/k/v projection ->
 *                   attention -> out-projection | fc1 -> fc2) joined by events, 0 = three kernels in a row
 *   "push_tma"      how md_hgemm_colsplit_push / _fused send a finished tile to the peers: 1 (default) = the epilogue warps issue
 *                   one more TMA store per peer from the shared-memory chunk they have just staged for this GPU's C;
 *                   0 = eight extra warps read the tile back from this GPU's C and store it with plain 16-byte stores
 *   "tc_splitk"     0 (default): never; -1: the tcgen05 GEMM splits K over several CTAs per tile where its cost model
 *                   expects a gain (fewer 128 x 256 tiles than SMs and a long K; f32 partial tiles added up in a fixed
 *                   order by the CTA that finishes last); 2..8: always that many ranges where the shape allows.
 *                   Faster for such a product alone (761 x 2048 x 8192: 42.6 -> 33.4 us), slower inside the forked
 *                   prefill layer, where the other chain's kernels already fill the SMs it leaves idle
 *   "attn_ctas_per_sm" 2 (default), 1: the tcgen05 attention runs that many CTAs per SM, each walking several
 *                   (query block, head, batch) items with its barriers, rings and TMEM kept; 0: one CTA per item
 *   "decode_loop"   n: the attention of a batched decode step with at least n (head, request) pairs runs one CTA per
 *                   pair that walks all of its keys (nothing to merge across CTAs); -1 (default) = 128 (four requests of 32 heads), 0 = never
 *   "decode_mlp_split" 2 (default) or 4 = with decode_fork and a single request, the MLP chain runs as that many
 *                   independent chains (a slice of fc1's rows, then that slice of fc2's K sum as f32 partial sums) which
 *                   the out-projection's epilogue adds with the reference's roundings; 0 = one MLP chain */
int md_set_option(md_ctx* ctx, const char* key, long value);
/* Read back a knob or a diagnostic (no counterpart in the reference): "gemv_variant", "tc_block_n", "pdl", and
 *   "last_tc_tile"  the tile the last tcgen05 GEMM launch of this context used: 64 / 128 / 256 = width of a
 *                   128-row tile, 512 = the 256 x 256 tile, 2256 = a 256 x 256 tile on a CTA pair, 1000 + S = the
 *                   skinny kernel with S splits of K,
 *                   0 = none yet.  Lets a test see which tile the
 *                   cost model picked for a shape (e.g. for the column-split GEMM with peers). */
int md_get_option(md_ctx* ctx, const char* key, long* value_out);

/* ---- CUDA graphs -------------------------------------------------------------------
 * A decode step is ~170 small kernels; replaying them as one graph removes the launch
 * overhead.  Between md_graph_begin and md_graph_end every entry point called with DEVICE
 * pointers only is recorded instead of executed (host-pointer calls are rejected with
 * MD_ERR_UNSUPPORTED, they would need a synchronous copy).  Run the same calls once before
 * capturing so that scratch memory and kernel attributes are already set up. */
typedef struct md_graph md_graph;
int md_graph_begin(md_ctx* ctx);
int md_graph_end(md_ctx* ctx, md_graph** out);
int md_graph_launch(md_ctx* ctx, md_graph* graph);
int md_graph_destroy(md_ctx* ctx, md_graph* graph);

/* ---- matmul -------------------------------------------------------------------- */

/* Replaces hgemm.matmul(a, b, allocator) — src/core/hgemm.zig:362-426.
 * C[M,N] = A[M,K] . B[K,N]; f16 in/out, f32 accumulate, one rounding to f16. */
int md_hgemm_nn(md_ctx* ctx, const uint16_t* a, const uint16_t* b, uint16_t* c, size_t M, size_t N, size_t K);

/* Replaces hgemm_trans.matmul(a, b_transposed, allocator) — src/core/hgemm_trans.zig:400-488.
 * C[M,N] = A[M,K] . B_t[N,K]^T.  M <= 8 takes the weight-streaming GEMV kernel
 * (the reference has a dedicated path for M == 1 only, hgemm_trans.zig:430-455). */
int md_hgemm_nt(md_ctx* ctx, const uint16_t* a, const uint16_t* b_t, uint16_t* c, size_t M, size_t N, size_t K);

/* Shape checks of hgemm.zig:369-381 / hgemm_trans.zig:408-420 for callers that hold
 * full shapes: rank != 2 -> MD_ERR_INVALID_DIMENSION, inner dims differ -> MD_ERR_SHAPE. */
int md_check_matmul_shapes(const size_t* a_shape, size_t a_rank, const size_t* b_shape, size_t b_rank,
                           int b_transposed);

/* The GEMMs above with the glue the reference applies right after them fused into the
 * epilogue, keeping the reference's rounding points: c = f16(acc); if bias: c = f16(c + bias[n])
 * (ops.broadcast_add_simd, ops.zig:1780-1953); if gelu: c = gelu(c) (ops.gelu, ops.zig:1635-1774);
 * if residual: c = f16(c + residual[m,n]) (ops.add, ops.zig:312-323).  bias/residual may be NULL.
 * b_layout: 0 = B is [K,N] (hgemm), 1 = B is [N,K] (hgemm_trans).  All pointers device-resident. */
int md_hgemm_fused(md_ctx* ctx, const uint16_t* a, const uint16_t* b, uint16_t* c, size_t M, size_t N, size_t K,
                   int b_layout, const uint16_t* bias, int gelu, const uint16_t* residual);

/* ---- column-split GEMM across the GPUs of one box (the one exchange step of the path) ----------
 * C[M, N_total] = A[M,K] . B with N split over `world` GPUs: this rank computes the column block
 * [col_offset, col_offset + N_local) from the full A and its slice of B (hgemm.zig / hgemm_trans.zig
 * have no distributed counterpart; the arithmetic per block is md_hgemm_nn / md_hgemm_nt).
 *
 * md_hgemm_colsplit_push fuses the exchange into the GEMM: every finished chunk of the block is stored
 * into this rank's full C (c_full, row stride N_total) and, with plain peer stores over NVLink, into the
 * same place of the n_peers other ranks' full C buffers (peer_c_full: device pointers that are mapped
 * into this process, e.g. from symmetric memory or CUDA IPC).  When every rank has run the call and a
 * cross-rank barrier has passed, every C holds all column blocks; no separate all-gather runs.
 * b is this rank's slice: [K, N_local] (b_layout 0) or [N_local, K] (b_layout 1).  n_peers <= 7. */
int md_hgemm_colsplit_push(md_ctx* ctx, const uint16_t* a, const uint16_t* b_slice, uint16_t* c_full, size_t M,
                           size_t N_local, size_t K, int b_layout, size_t N_total, size_t col_offset, size_t n_peers,
                           uint16_t* const* peer_c_full);

/* The re-layout step of the all-gather baseline: gathered [world][M][N_local] (what an all-gather of the
 * ranks' contiguous blocks produces) -> c [M][world * N_local].  Device pointers. */
int md_gather_colblocks(md_ctx* ctx, const uint16_t* gathered, uint16_t* c, size_t world, size_t M, size_t N_local);

/* ---- the exchange step for hosts that run one process per GPU -----------------------------------
 * The reference has no distributed code (hgemm.zig:396-423 spawns threads only), so nothing here replaces a
 * reference function; the arithmetic per column block is md_hgemm_nn / md_hgemm_nt.  A communicator binds a
 * context to `world` <= 8 ranks of one box.  NCCL is looked up at run time (libnccl.so.2): a process that
 * already carries one shares it, a machine without it gets MD_ERR_NCCL from md_comm_unique_id / md_comm_init.
 * Every call below except md_comm_unique_id is collective: all ranks make it, in the same order. */
#define MD_COMM_ID_BYTES 128
typedef struct md_comm md_comm;
/* Rank 0 creates the id (ncclGetUniqueId) and hands the 128 bytes to the other ranks by any means. */
int md_comm_unique_id(md_ctx* ctx, void* id_out);
/* ncclCommInitRank on the context's device + a small peer-mapped signal pad for md_comm_barrier. */
int md_comm_init(md_ctx* ctx, const void* unique_id, int rank, int world, md_comm** out);
int md_comm_destroy(md_comm* comm);
/* A zeroed device buffer of `bytes` on every rank, mapped into every other rank (CUDA IPC handles all-gathered
 * over the communicator), so that this library's kernels can store into the peers' copies over NVLink. */
int md_comm_symm_alloc(md_comm* comm, size_t bytes, void** local_out);
int md_comm_symm_free(md_comm* comm, void* local);
/* Stream-ordered barrier across the ranks' GPUs: one small kernel per rank, no host round trip.  A peer that
 * does not arrive within two seconds makes the next md_sync return MD_ERR_TIMEOUT (site 200 + peer rank). */
int md_comm_barrier(md_comm* comm);
/* C[M, N_total] = A[M,K] . B with N split evenly over the ranks (N_total / world a multiple of 8); b_slice is
 * this rank's slice, [K, N_total/world] (b_layout 0) or [N_total/world, K] (b_layout 1); every rank ends up with
 * the whole C.  Device pointers only.
 *   _allgather  the baseline: GEMM into a contiguous block, ncclAllGather of the blocks, one re-layout kernel.
 *   _fused      md_hgemm_colsplit_push between two md_comm barriers: the GEMM kernel's push warps store every
 *               finished tile into all ranks' C while the following tiles are computed; c_symm must come from
 *               md_comm_symm_alloc (at least M * N_total * 2 bytes).  No collective and no re-layout runs. */
int md_hgemm_colsplit_allgather(md_comm* comm, const uint16_t* a, const uint16_t* b_slice, uint16_t* c_full, size_t M,
                                size_t N_total, size_t K, int b_layout);
int md_hgemm_colsplit_fused(md_comm* comm, const uint16_t* a, const uint16_t* b_slice, uint16_t* c_symm, size_t M,
                            size_t N_total, size_t K, int b_layout);

/* ---- attention ----------------------------------------------------------------- */

/* Replaces attention.multiMasklessSDPA(n_heads, head_dim, q, k, v, allocator) —
 * src/core/attention.zig:125-234.  q,out [n_heads,q_len,d]; k,v [n_heads,kv_len,d]. */
int md_sdpa_maskless(md_ctx* ctx, const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* out,
                     size_t n_heads, size_t q_len, size_t kv_len, size_t head_dim);

/* Replaces attention.createAttentionMask(allocator, pos, seq_len) — attention.zig:256-281.
 * mask is one byte per entry, [seq_len, pos+seq_len]. */
int md_create_attention_mask(md_ctx* ctx, uint8_t* mask, size_t pos, size_t seq_len);

/* Replaces attention.multiMaskedSDPA(q,k,v,mask,n_heads,head_dim,allocator) — attention.zig:416-541.
 * mask [q_len, kv_len] bytes, 0 = masked out. */
int md_sdpa_masked(md_ctx* ctx, const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint8_t* mask,
                   uint16_t* out, size_t n_heads, size_t q_len, size_t kv_len, size_t head_dim);

/* Replaces attention.singleMaskedSDPA(q,k,v,mask,allocator) — attention.zig:759-811.
 * 32 heads x 64 dims fixed; q,out [32,1,64]; k,v [32,kv_len,64] contiguous; mask [kv_len];
 * kv_len > 2048 -> MD_ERR_SEQUENCE_TOO_LONG. */
int md_sdpa_single(md_ctx* ctx, const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint8_t* mask,
                   uint16_t* out, size_t kv_len);

/* md_sdpa_single for callers that must not allocate.  It has no counterpart in the reference: it
 * exists for hosts that cannot call cudaMalloc once they are running — a serving process that gave
 * all of HBM to its own arena at start-up, or a latency-critical decode loop that cannot afford the
 * device-wide synchronisation cudaMalloc/cudaFree imply.  It takes no context and calls no cudaMalloc,
 * cudaFree or allocating library routine: the split-KV scratch is a 135,424-byte device array built
 * into the library (held by every GPU that loads it until the process exits).
 *   - same arithmetic and layouts as md_sdpa_single (32 heads x 64 dims), DEVICE pointers only;
 *   - kv_len > 2048 (the scratch's maximum) -> MD_ERR_SEQUENCE_TOO_LONG; a message is written to
 *     err[0..err_cap) when err is not NULL;
 *   - enqueues on cuda_stream (NULL = the default stream) and returns without waiting;
 *   - the tensors must live on the device that is current when the call is made (a tensor on another
 *     GPU -> MD_ERR_INVALID_ARG; managed memory is accepted);
 *   - the first call on a device looks up the scratch's device address; make that call with the
 *     device current, before any stream capture begins, and at start-up before the host reserves the
 *     rest of HBM (with lazy module loading the first use of the library on a device is what places
 *     its code and the scratch array in device memory);
 *   - every call on a device shares the one scratch array: calls that overlap on the GPU race,
 *     so keep them on one stream or order them with events. */
int md_sdpa_single_noalloc(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint8_t* mask,
                           uint16_t* out, size_t kv_len, void* cuda_stream, char* err, size_t err_cap);

/* The decode-step attention the GPU path uses instead of the sequence
 * rope.applyRotEmb x2 -> LayerCache.updateCache -> getActiveCache -> createAttentionMask ->
 * singleMaskedSDPA (text_model.zig:228-290): reads q,k,v of the new token from one row of the
 * fused qkv projection ([3*n_heads*d]: q | k | v), rotates q and k at position `pos` in-kernel
 * (partial rotary on the first rot_dim dims), appends k,v to the cache in place
 * (layout [n_heads][max_seq][d], text_model.zig:392,485) and attends over positions 0..pos.
 * out [n_heads*d].  Device pointers only.  pos >= max_seq -> MD_ERR_SEQUENCE_TOO_LONG. */
int md_sdpa_decode_fused(md_ctx* ctx, const uint16_t* qkv_row, uint16_t* key_cache, uint16_t* value_cache,
                         uint16_t* out, size_t n_heads, size_t head_dim, size_t max_seq, size_t pos,
                         size_t rot_dim, float theta);

/* The prefill attention the GPU path uses instead of the same sequence with multiMaskedSDPA
 * (text_model.zig:228-290): qkv [S, 3*n_heads*d]; rotates q and k at positions pos..pos+S-1,
 * appends k,v to the cache, causal attention over 0..pos+i for row i; out [S, n_heads*d]
 * (already in the "transposed back" layout of text_model.zig:293-294).  Device pointers only. */
int md_sdpa_prefill_fused(md_ctx* ctx, const uint16_t* qkv, uint16_t* key_cache, uint16_t* value_cache,
                          uint16_t* out, size_t S, size_t n_heads, size_t head_dim, size_t max_seq, size_t pos,
                          size_t rot_dim, float theta);

/* ViT attention straight from the fused qkv projection (replaces the split / reshape / transposeAxes /
 * multiMasklessSDPA / transposeAxes chain of vision_model.zig:285-330): qkv [crops*tokens, 3*n_heads*d],
 * attention per crop over `tokens` keys, out [crops*tokens, n_heads*d].  Device pointers only. */
int md_sdpa_vit_fused(md_ctx* ctx, const uint16_t* qkv, uint16_t* out, size_t crops, size_t tokens,
                      size_t n_heads, size_t head_dim);

/* ---- rope ---------------------------------------------------------------------- */

/* Replaces rope.precomputeFreqsCis(f32, allocator, dim, end, theta) — src/core/rope.zig:32-128.
 * table f32 [end, dim/2, 2] = (cos, sin). */
int md_rope_table(md_ctx* ctx, float* table, size_t dim, size_t end, float theta);

/* Replaces rope.applyRotEmb(allocator, x, n_heads, head_dim, freqs_cis, position_ids, rot_dim) —
 * rope.zig:130-272.  x,out f16 [n_heads,seq_len,head_dim]; freqs_cis f32 [*, freqs_half, 2];
 * position_ids u64 [seq_len] (the reference's usize).  rot_dim != 2*freqs_half -> MD_ERR_INVALID_ROT_DIM. */
int md_rope_apply(md_ctx* ctx, const uint16_t* x, uint16_t* out, size_t n_heads, size_t seq_len, size_t head_dim,
                  const float* freqs_cis, size_t freqs_half, const uint64_t* position_ids, size_t rot_dim);

/* ---- KV cache (text_model.zig:383-516) ------------------------------------------- */

/* LayerCache.updateCache — text_model.zig:476-515. k_new,v_new [n_heads,seq_len,d]. */
int md_kv_update(md_ctx* ctx, uint16_t* key_cache, uint16_t* value_cache, const uint16_t* k_new,
                 const uint16_t* v_new, size_t n_heads, size_t max_seq, size_t head_dim, size_t cur_len,
                 size_t seq_len);
/* LayerCache.getActiveCache — text_model.zig:436-474. */
int md_kv_active(md_ctx* ctx, const uint16_t* key_cache, const uint16_t* value_cache, uint16_t* k_out,
                 uint16_t* v_out, size_t n_heads, size_t max_seq, size_t head_dim, size_t cur_len);

/* ---- glue ops between the GEMMs (src/core/ops.zig) ------------------------------- */

/* ops.layerNorm(f16, x, w, b, eps) — ops.zig:1063-1070,1152-1419. eps is given as the f16 bits. */
int md_layernorm(md_ctx* ctx, const uint16_t* x, const uint16_t* w, const uint16_t* b, uint16_t* y, size_t rows,
                 size_t cols, uint16_t eps_f16);
/* ops.gelu(f16, &x) in place — ops.zig:1635-1774. */
int md_gelu(md_ctx* ctx, uint16_t* x, size_t n);
/* ops.broadcast_add_simd(&a, b) in place — ops.zig:1780-1953; a [rows,cols] += b [cols]. */
int md_bias_add(md_ctx* ctx, uint16_t* a, const uint16_t* b, size_t rows, size_t cols);
/* ops.add(f16, &a, b) in place — ops.zig:312-323. */
int md_add(md_ctx* ctx, uint16_t* a, const uint16_t* b, size_t n);
/* sampling.argmax — src/utils/sampling.zig:257-273; first strict maximum. idx_out: host or device u64. */
int md_argmax(md_ctx* ctx, const uint16_t* x, size_t n, uint64_t* idx_out);
/* createPatches tail + convertBHWCtoBCHW + /255 + normalizePatch + rearrangeBCHWtoBTC
 * (vision_model.zig:137-183, reshape_handler.zig:5-129): uint8 [crops,H,W,3] ->
 * f16 [crops*(H/p)*(W/p), out_stride] with the first 3*p*p columns filled in (c,ph,pw) order and
 * columns 3*p*p..out_stride-1 zeroed (out_stride >= 3*p*p lets the caller pad K for TMA). */
int md_preprocess_patchify(md_ctx* ctx, const uint8_t* img, uint16_t* out, size_t crops, size_t height,
                           size_t width, size_t patch, size_t out_stride);

#ifdef __cplusplus
}
#endif
#endif /* MOONDREAM_B200_H */
