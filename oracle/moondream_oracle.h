/*
 * CPU oracle for the moondream-zig FP16 matmul + attention hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a C++ restatement of the reference's CPU
 * algorithms (Zig, AVX2 `@Vector(8,f32)` + std.Thread).  It is the checker the
 * GPU library is compared against and the timed CPU baseline; nothing in the
 * product library links, imports or calls it.
 *
 * Parity status: the reference is Zig 0.13 and cannot be compiled where this is
 * built, so the oracle is pinned only by what the reference's own tests pin:
 *   - hgemm (NN) against the in-test naive f32-accumulate product with the
 *     tolerances of src/core/matmul_test.zig:108-152 and the cases at :154-367
 *   - sgemm 2x2 known answer, src/core/matmul_test.zig:371-400
 *   - LayerNorm (normalised rows, zero variance) and broadcast add (bias,
 *     positional embedding, general), src/core/ops_test.zig:1773-1866,
 *     1886-1935, 2547-2640
 * hgemm_trans (NT + GEMV), the three SDPA variants, rope, softmax, GELU,
 * the KV cache and argmax have NO reference test: for those rows
 * PARITY IS UNPINNED; they are validated against float64 restatements of the
 * formulas and algebraic properties.
 *
 * All f16 buffers are IEEE binary16 passed as uint16_t*.  Every function
 * returns 0 on success or a negative orc_status.
 */
#ifndef MOONDREAM_ORACLE_H
#define MOONDREAM_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum orc_status {
    ORC_OK = 0,
    ORC_ERR_INVALID_DIMENSION = -1, /* error.InvalidTensorDimension / InvalidInputDimensions */
    ORC_ERR_INCOMPATIBLE_SHAPES = -2, /* error.IncompatibleTensorShapes */
    ORC_ERR_SEQUENCE_TOO_LONG = -3, /* error.SequenceTooLong */
    ORC_ERR_INVALID_ROT_DIM = -4, /* error.InvalidRotationDimension */
    ORC_ERR_INVALID_ARG = -5,
};

/* Number of worker threads the matmuls spawn per call; 0 = one per hardware
 * thread, which is what the reference does (hgemm.zig:396). */
void orc_set_threads(int n);
int orc_get_threads(void);

/* hgemm.zig:362-426 — C[M,N] = A[M,K] . B[K,N], f16 storage, f32 accumulate,
 * 168x168x168 tiles, 8x8 FMA micro-kernel, one rounding to f16 at the end. */
int orc_hgemm_nn(const uint16_t* a, const uint16_t* b, uint16_t* c, size_t M, size_t N, size_t K);

/* hgemm_trans.zig:400-488 — C[M,N] = A[M,K] . B_t[N,K]^T.  M==1 takes the
 * vector path of hgemm_trans.zig:55-134 (4 x 8-lane accumulators, work items
 * of 32 outputs); everything else the tiled path (:257-398). */
int orc_hgemm_nt(const uint16_t* a, const uint16_t* b_t, uint16_t* c, size_t M, size_t N, size_t K);

/* matmul_test.zig:83-106 — the naive product the reference's tests compare
 * hgemm against: f32 accumulate in k order (mul then add), one f16 rounding. */
int orc_naive_matmul_f16(const uint16_t* a, const uint16_t* b, uint16_t* c, size_t M, size_t N, size_t K);

/* sgemm_inplace.zig:48-87,225-322 — f32 C[M,N] = A[M,K] . B[K,N] (result zeroed first). */
int orc_sgemm(const float* a, const float* b, float* c, size_t M, size_t N, size_t K);

/* ops.zig:1548-1633 — in-place row softmax over the last dim: row max,
 * e = (v-max > -88) ? exp(v-max) : 0, normalise only when the sum is > 0. */
int orc_softmax_rows(float* data, size_t rows, size_t cols);

/* attention.zig:125-234 — softmax(Q K^T / sqrt(d)) V per head, no mask.
 * q [n_heads,q_len,d], k,v [n_heads,kv_len,d], out [n_heads,q_len,d]. */
int orc_sdpa_maskless(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* out,
                      size_t n_heads, size_t q_len, size_t kv_len, size_t head_dim);

/* attention.zig:256-281 — bool mask [seq_len, pos+seq_len]: columns < pos are
 * true, then lower-triangular (j <= i). One byte per entry. */
int orc_create_attention_mask(uint8_t* mask, size_t pos, size_t seq_len);

/* attention.zig:416-541 — as maskless, scores scaled then masked (false -> -inf). */
int orc_sdpa_masked(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint8_t* mask,
                    uint16_t* out, size_t n_heads, size_t q_len, size_t kv_len, size_t head_dim);

/* attention.zig:564-642,759-811 — one query token, 32 heads x 64 dims fixed,
 * exact exp softmax, kv_len <= 2048 else ORC_ERR_SEQUENCE_TOO_LONG.
 * q [32,1,64], k,v [32,kv_len,64] contiguous, mask [kv_len], out [32,1,64]. */
int orc_sdpa_single(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint8_t* mask,
                    uint16_t* out, size_t kv_len);

/* rope.zig:32-128 — table[end][dim/2][2] = (cos, sin)(p * theta^(-2j/dim)), f32. */
int orc_rope_table(float* table, size_t dim, size_t end, float theta);

/* rope.zig:130-272 — x,out f16 [n_heads,seq_len,head_dim]; pairs (x[j], x[j+rot_dim/2]);
 * dims >= rot_dim copied; freqs_half = number of (cos,sin) pairs per position in the table. */
int orc_rope_apply(const uint16_t* x, uint16_t* out, size_t n_heads, size_t seq_len, size_t head_dim,
                   const float* freqs_cis, size_t freqs_half, const size_t* position_ids, size_t rot_dim);

/* ops.zig:1063-1070,1152-1419 — LayerNorm over the last dim; f32 mean and biased
 * variance, y = (x*rstd - mean*rstd)*w + b, f16 out. eps is the f16 value the caller holds. */
int orc_layernorm(const uint16_t* x, const uint16_t* w, const uint16_t* b, uint16_t* y,
                  size_t rows, size_t cols, uint16_t eps_f16);

/* ops.zig:1635-1774 — tanh GELU in f32 with both constants rounded to f16 first. In place. */
int orc_gelu(uint16_t* x, size_t n);

/* ops.zig:1780-1953 — a[row][j] = f16(f32(a[row][j]) + f32(b[j])). In place on a. */
int orc_bias_add(uint16_t* a, const uint16_t* b, size_t rows, size_t cols);

/* ops.zig:312-323 — a += b elementwise in f16. */
int orc_add(uint16_t* a, const uint16_t* b, size_t n);

/* sampling.zig:257-273 — index of the first strict maximum of f16 logits widened to f32. */
int orc_argmax_f16(const uint16_t* x, size_t n, size_t* idx_out);

/* text_model.zig:476-515 — append seq_len rows per head into the flat cache
 * [n_heads][max_seq][head_dim] at position cur_len. k_new,v_new [n_heads,seq_len,head_dim]. */
int orc_kv_update(uint16_t* key_cache, uint16_t* value_cache, const uint16_t* k_new, const uint16_t* v_new,
                  size_t n_heads, size_t max_seq, size_t head_dim, size_t cur_len, size_t seq_len);

/* text_model.zig:436-474 — copy the active prefix out as contiguous [n_heads,cur_len,head_dim]. */
int orc_kv_active(const uint16_t* key_cache, const uint16_t* value_cache, uint16_t* k_out, uint16_t* v_out,
                  size_t n_heads, size_t max_seq, size_t head_dim, size_t cur_len);

/* vision_model.zig:137-183 + reshape_handler.zig:5-129 — uint8 [crops,H,W,3] ->
 * f16(u8) / f16(255) -> (v-0.5)/0.5 (every step in f16) -> patches [crops, (H/p)*(W/p), 3*p*p]
 * with patch element order (c, ph, pw). */
int orc_preprocess_patchify(const uint8_t* img, uint16_t* out, size_t crops, size_t height, size_t width,
                            size_t patch);

/* ---- model-level restatements (host control flow of the reference) ---- */

/* Phi-1.5-style text decoder weights; every matrix is [out,in] row-major f16
 * (weights.zig:439-478), per-layer tensors are arrays of n_layers pointers. */
typedef struct orc_text_weights {
    size_t n_layers, dim, hidden, n_heads, head_dim, vocab, max_seq;
    const uint16_t* const* ln_w;  const uint16_t* const* ln_b;
    const uint16_t* const* wqkv;  const uint16_t* const* bqkv;
    const uint16_t* const* wout;  const uint16_t* const* bout;
    const uint16_t* const* wfc1;  const uint16_t* const* bfc1;
    const uint16_t* const* wfc2;  const uint16_t* const* bfc2;
    const uint16_t* ln_out_w; const uint16_t* ln_out_b;
    const uint16_t* lm_w; const uint16_t* lm_b;
    const uint16_t* wte; /* [vocab, dim] */
} orc_text_weights;

/* text_model.zig:139-180 — one text_decoder call over S rows of embeddings with the
 * per-layer caches key/value[n_layers] (flat [n_heads][max_seq][head_dim]) holding
 * cur_len tokens.  hidden_io [S,dim] is overwritten with the output; caches are
 * appended in place. */
int orc_text_decoder(const orc_text_weights* w, uint16_t* hidden_io, size_t S,
                     uint16_t* const* key_cache, uint16_t* const* value_cache, size_t cur_len);

/* text_model.zig:325-345 — LN(last row) . lm_w^T + lm_b -> logits [vocab]. */
int orc_lm_head(const orc_text_weights* w, const uint16_t* hidden, size_t S, uint16_t* logits);

/* SigLIP-style vision encoder weights; every matrix is [in,out] row-major f16
 * (weights.py:209-246), per-layer tensors are arrays of n_layers pointers. */
typedef struct orc_vision_weights {
    size_t n_layers, dim, n_heads, head_dim, hidden, tokens, patch_dim, proj_hidden, proj_out;
    const uint16_t* patch_w; const uint16_t* patch_b; const uint16_t* pos_emb; /* [588,1152],[1152],[729,1152] */
    const uint16_t* const* ln1_w; const uint16_t* const* ln1_b;
    const uint16_t* const* wqkv;  const uint16_t* const* bqkv;
    const uint16_t* const* wout;  const uint16_t* const* bout;
    const uint16_t* const* ln2_w; const uint16_t* const* ln2_b;
    const uint16_t* const* wfc1;  const uint16_t* const* bfc1;
    const uint16_t* const* wfc2;  const uint16_t* const* bfc2;
    const uint16_t* norm_w; const uint16_t* norm_b;
    const uint16_t* proj_fc1_w; const uint16_t* proj_fc1_b; /* [2304,8192] */
    const uint16_t* proj_fc2_w; const uint16_t* proj_fc2_b; /* [8192,2048] */
} orc_vision_weights;

/* vision_model.zig:204-272 — patches [crops*tokens, patch_dim] -> features [crops*tokens, dim].
 * joint_attention != 0 runs attention over all crops as ONE sequence, which is what the
 * reference does for its two identical crops (vision_model.zig:36-38,308-316); 0 runs it per crop. */
int orc_vision_encoder(const orc_vision_weights* w, const uint16_t* patches, size_t crops,
                       int joint_attention, uint16_t* features);

/* vision_model.zig:189-195,366-387 — concat(features of crop a, crop b) on the last dim ->
 * fc1 + bias -> GELU -> fc2 + bias -> [tokens, proj_out]. */
int orc_vision_projection(const orc_vision_weights* w, const uint16_t* feat_a, const uint16_t* feat_b,
                          uint16_t* out);

#ifdef __cplusplus
}
#endif
#endif
