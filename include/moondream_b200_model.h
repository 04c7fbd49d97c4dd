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
 * (concurrent decode streams batched as M <= 8 GEMVs); the attention of all requests runs in one launch, each request
 * against its own cache.
 * All requests must hold caches of the same model; their lengths may differ.
 *   first [batch], tokens_out [batch, n_steps] (host). */
int md_text_generate_batch(md_text_model* model, md_text_request* const* reqs, size_t batch, const uint32_t* first,
                           size_t n_steps, uint32_t* tokens_out);
/* The batched loop under teacher forcing: forced host u32 [batch, n_steps], request b consumes forced[b][i-1] at
 * step i instead of its own previous output (step 0 consumes first[b]); tokens_out still holds what every step
 * produced.  For parity checks of batched decoding against a reference that generated the forced tokens. */
int md_text_generate_batch_forced(md_text_model* model, md_text_request* const* reqs, size_t batch, const uint32_t* first,
                                  size_t n_steps, uint32_t* tokens_out, const uint32_t* forced);

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

/* `n_images` (<= max_crops) independent images of one crop each in one pass: the encoder's GEMMs run over
 * n_images * tokens rows, attention stays per image, and image i is projected from concat(features[i], features[i])
 * — what md_vision_encode gives for the reference's two identical crops of one image (vision_model.zig:137-155) —
 * into outs[i] ([tokens, proj_out], host or device).  images_u8 [n_images, img, img, 3], host or device.  For hosts
 * that serve several requests at once (the reference encodes one image per process run). */
int md_vision_encode_images(md_vision_model* model, const uint8_t* images_u8, size_t n_images, uint16_t* const* outs);

/* ---- moondream.bin weight file (read: weights.zig:61-207; written by weights.py:82-246) --------------
 *
 * Layout, little-endian: u32 magic 0x4D4F4F4E ("MOON"), u32 version 2, then records until end of file:
 *   u32 name_length (<= 256), u32 shape_length (<= 4), u32 data_length (element count; written, never read),
 *   name bytes, shape_length x u64 dims, prod(dims) x f16.
 * The 36 tensor names and their expected shapes follow from the model configuration (weights.zig:439-478);
 * per-layer tensors are stacked on a leading n_layers axis.
 *
 * md_weight_file_open parses and validates on the host only (no device, no context): the file is mapped
 * read-only and every record is checked in the reference's order.  Failures and the Zig error each stands for
 * (the name is the first word of md_last_error(NULL)):
 *   MD_ERR_IO      FileNotFound (open / map failed), InvalidRead (file ends inside a field)
 *   MD_ERR_FORMAT  InvalidMagicNumber, InvalidVersion, InvalidHeader (1..11 trailing bytes), InvalidNameLength,
 *                  InvalidShapeLength, UnknownTensorName, ShapeMismatch
 * A name that occurs twice keeps its last occurrence, as the reference does.  Unlike the reference, which leaves
 * the field undefined, a tensor that never occurs is reported (MissingTensor, MD_ERR_FORMAT) by
 * md_weight_file_text / md_weight_file_vision. */

typedef struct md_model_config {     /* config.zig:3-27, 86-112 */
    size_t vocab, dim, hidden_dim, n_layers, n_heads, head_dim, seq_len;
    float rope_theta, partial_rotary_factor;
    size_t img_channels, img_dim, patch_size, num_patches, vit_dim, n_vit_layers, n_vit_heads, vit_head_dim,
        hidden_features;
} md_model_config;
/* MODEL_CONFIG of config.zig:3-27. */
int md_model_config_default(md_model_config* cfg);

typedef struct md_weight_file md_weight_file;

/* cfg NULL = md_model_config_default. */
int md_weight_file_open(const char* path, const md_model_config* cfg, md_weight_file** out);
int md_weight_file_close(md_weight_file* wf);   /* also frees what md_weight_file_upload allocated */
/* The records in file order.  name is NUL-terminated and lives as long as the file object; host_data points into
 * the read-only mapping; shape receives `rank` dims (at most 4). */
int md_weight_file_count(const md_weight_file* wf, size_t* n_out);
int md_weight_file_tensor(const md_weight_file* wf, size_t index, const char** name, size_t* rank, size_t shape[4],
                          const uint16_t** host_data);
/* Copy every tensor to the context's device, byte for byte, through a double-buffered pinned staging area; one
 * device allocation per tensor, so the layers of a stacked tensor are contiguous.  Returns when the copies are done. */
int md_weight_file_upload(md_weight_file* wf, md_ctx* ctx);
/* Fill the weight tables of the two models from an uploaded file.  The per-layer pointer arrays belong to the
 * file object; the models keep the device pointers, so close the file after the models are destroyed.
 * rot_dim = head_dim * partial_rotary_factor, max_seq = seq_len, eps = f16(1e-5) (text_model.zig:28,
 * vision_model.zig:35).  The projection's input width is checked as vit_head_dim * n_heads, the expression of
 * weights.zig:470 (2304 = 2 * vit_dim for the shipped configuration). */
int md_weight_file_text(md_weight_file* wf, md_text_weights* out);
int md_weight_file_vision(md_weight_file* wf, md_vision_weights* out);

#ifdef __cplusplus
}
#endif
#endif /* MOONDREAM_B200_MODEL_H */
