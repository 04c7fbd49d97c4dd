/*
 * moondream_b200_model — the callers on either side of the hot path, device-resident.
 *
 * These entry points restate the host control flow of src/model/text_model.zig and
 * src/model/vision_model.zig on top of the kernels of moondream_b200.h, so that a request runs
 * end to end without returning to the host between layers: weights registered once, activations
 * and the KV cache resident in HBM, one CUDA graph per decode step.  Names follow the reference:
 * text_encoder / text_decoder / lm_head (text_model.zig:106,139,325), KVCache (text_model.zig:349),
 * vision_encoder / encode_mlp (vision_model.zig:204,366).
 *
 * All weight pointers are DEVICE pointers (md_upload) to f16 tensors laid out as the reference
 * holds them: text matrices [out,in], vision / projection matrices [in,out] (weights.zig:439-478).
 */
#ifndef MOONDREAM_B200_MODEL_H
#define MOONDREAM_B200_MODEL_H

#include "moondream_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- text decoder (Phi-1.5 style, text_model.zig) --------------------------------------- */

typedef struct md_text_weights {
    size_t n_layers, dim, hidden, n_heads, head_dim, vocab, max_seq, rot_dim;
    float rope_theta;
    uint16_t eps_f16;            /* LayerNorm epsilon as f16 bits (text_model.zig:28) */
    /* arrays of n_layers device pointers (the arrays themselves are host memory) */
    const uint16_t* const* ln_w;   const uint16_t* const* ln_b;
    const uint16_t* const* wqkv;   const uint16_t* const* bqkv;   /* [3*dim, dim], [3*dim] */
    const uint16_t* const* wout;   const uint16_t* const* bout;   /* [dim, dim] */
    const uint16_t* const* wfc1;   const uint16_t* const* bfc1;   /* [hidden, dim] */
    const uint16_t* const* wfc2;   const uint16_t* const* bfc2;   /* [dim, hidden] */
    const uint16_t* ln_out_w; const uint16_t* ln_out_b;
    const uint16_t* lm_w; const uint16_t* lm_b;                   /* [vocab, dim], [vocab] */
    const uint16_t* wte;                                          /* [vocab, dim] token embedding */
} md_text_weights;

typedef struct md_text_model md_text_model;
/* One request = one KVCache (text_model.zig:349-539: per layer key/value [n_heads][max_seq][head_dim])
 * plus the activation buffers of a step. */
typedef struct md_text_request md_text_request;

int md_text_model_create(md_ctx* ctx, const md_text_weights* w, md_text_model** out);
int md_text_model_destroy(md_text_model* model);
int md_text_request_create(md_text_model* model, md_text_request** out);
int md_text_request_destroy(md_text_request* req);
/* KVCache.reset (text_model.zig:533-537). */
int md_text_request_reset(md_text_request* req);
/* Current number of cached tokens (LayerCache.getCurrentLen). */
int md_text_request_len(const md_text_request* req, size_t* len_out);

/* text_encoder (text_model.zig:106-137): embedding lookup. ids host u32 [n]; out f16 [n, dim], host or device.
 * An id >= vocab returns MD_ERR_INVALID_ARG (error.TokenIdOutOfBounds). */
int md_text_encoder(md_text_model* model, const uint32_t* ids, size_t n, uint16_t* out);

/* text_decoder + lm_head + greedy sampling for a block of S >= 1 embedding rows
 * (text_model.zig:139-180, 325-345; sampling.zig:257-273): appends S tokens to the request's cache.
 * embeds [S, dim] host or device.  Optional outputs (NULL to skip), host or device:
 *   hidden_out [S, dim]  the decoder output,  logits_out [vocab]  lm_head of the last row,
 *   token_out            argmax of the logits (u64).
 * cache overflow -> MD_ERR_SEQUENCE_TOO_LONG. */
int md_text_forward(md_text_model* model, md_text_request* req, const uint16_t* embeds, size_t S,
                    uint16_t* hidden_out, uint16_t* logits_out, uint64_t* token_out);

/* Greedy generation entirely on the device (the hot loop of moondream.zig:323-368 without eos
 * handling): starting from token `first` (normally the token md_text_forward returned for the
 * prompt), run n_steps decode steps; step i embeds the previous token, runs the decoder over one row,
 * lm_head, argmax.  One CUDA graph is captured on the first call and replayed per step; the position
 * and the token live in device memory so the graph never changes.
 *   tokens_out   host u32 [n_steps]: the token produced by each step
 *   forced       optional host u32 [n_steps]: teacher forcing — step i consumes forced[i-1] instead of
 *                its own previous output (step 0 consumes `first`)
 *   logits_out   optional host f16 [n_steps, vocab] */
int md_text_generate(md_text_model* model, md_text_request* req, uint32_t first, size_t n_steps,
                     uint32_t* tokens_out, const uint32_t* forced, uint16_t* logits_out);

/* The same loop for up to 8 independent requests advanced together: every GEMV runs with M = batch rows
 * (BASELINE config 5a batches concurrent decode streams as M <= 8 GEMVs); attention runs per request.
 * All requests must hold caches of the same model; their lengths may differ.
 *   first [batch], tokens_out [batch, n_steps] (host). */
int md_text_generate_batch(md_text_model* model, md_text_request* const* reqs, size_t batch, const uint32_t* first,
                           size_t n_steps, uint32_t* tokens_out);

/* ---- vision encoder (SigLIP-style ViT, vision_model.zig) --------------------------------- */

typedef struct md_vision_weights {
    size_t n_layers, dim, n_heads, head_dim, hidden, tokens, patch, img, proj_hidden, proj_out;
    uint16_t eps_f16;
    const uint16_t* patch_w; const uint16_t* patch_b;   /* [3*patch*patch, dim], [dim] */
    const uint16_t* pos_emb;                            /* [tokens, dim] */
    const uint16_t* const* ln1_w; const uint16_t* const* ln1_b;
    const uint16_t* const* wqkv;  const uint16_t* const* bqkv;   /* [dim, 3*dim] */
    const uint16_t* const* wout;  const uint16_t* const* bout;   /* [dim, dim] */
    const uint16_t* const* ln2_w; const uint16_t* const* ln2_b;
    const uint16_t* const* wfc1;  const uint16_t* const* bfc1;   /* [dim, hidden] */
    const uint16_t* const* wfc2;  const uint16_t* const* bfc2;   /* [hidden, dim] */
    const uint16_t* norm_w; const uint16_t* norm_b;
    const uint16_t* proj_fc1_w; const uint16_t* proj_fc1_b;     /* [2*dim, proj_hidden] */
    const uint16_t* proj_fc2_w; const uint16_t* proj_fc2_b;     /* [proj_hidden, proj_out] */
} md_vision_weights;

typedef struct md_vision_model md_vision_model;

int md_vision_model_create(md_ctx* ctx, const md_vision_weights* w, size_t max_crops, md_vision_model** out);
int md_vision_model_destroy(md_vision_model* model);

/* encode_image without the file decode (vision_model.zig:160-202): uint8 crops [crops, img, img, 3]
 * (host or device) -> normalise + patchify -> vision_encoder (27 pre-LN blocks, per-crop attention) ->
 * features [crops, tokens, dim] -> concat(crop a, crop b) on the feature dim -> encode_mlp ->
 * out [tokens, proj_out].  The reference always encodes two identical crops (a = 0, b = 1); with one crop
 * pass crop_b = 0.  features_out (optional, [crops*tokens, dim]) and out may be host or device. */
int md_vision_encode(md_vision_model* model, const uint8_t* crops_u8, size_t crops, size_t crop_a, size_t crop_b,
                     uint16_t* features_out, uint16_t* out);

#ifdef __cplusplus
}
#endif
#endif /* MOONDREAM_B200_MODEL_H */
