// Interface of the persistent decode-step kernel (decode_persistent.cu) towards the text model (model.cu).
#pragma once
#include "md_internal.cuh"

constexpr int MD_PERSIST_MAX_LAYERS = 32;
constexpr int MD_PERSIST_MAX_BATCH = 8;

// Lives in device memory: every pointer the step needs, per layer and per request.
struct md_persist_table {
    struct Layer {
        const __half *ln_w, *ln_b, *wqkv, *bqkv, *wfc1, *bfc1, *wout, *bout, *wfc2, *bfc2;
        __half* kc[MD_PERSIST_MAX_BATCH];  // key cache of this layer, per request: [32][max_seq][64]
        __half* vc[MD_PERSIST_MAX_BATCH];
    } layers[MD_PERSIST_MAX_LAYERS];
    const __half *ln_out_w, *ln_out_b, *lm_w, *lm_b;
    const int* pos[MD_PERSIST_MAX_BATCH];  // device-resident position of every request
};

struct md_persist_params {
    const md_persist_table* tab;
    __half* hidden;            // [M][2048] in: embeddings of the current tokens; updated layer by layer
    __half* qkv;               // [M][6144]
    __half* attn;              // [M][2048]
    __half* fc1;               // [M][8192]
    __half* logits;            // [M][vocab]
    unsigned long long* amax;  // [M] greedy-argmax keys (value, then lower index), zero before the step
    float* att_scratch;        // [M][32][max_splits][66] partial (max, sum, out[64]) of the attention splits
    unsigned int* att_counters;  // [M * 32] arrival tickets, zero before and after the step
    unsigned int* grid_counter;  // [4] grid barriers, zero before the step
    const float* rope_tab;     // [max_seq][16][2] (cos, sin)
    int M, n_layers, vocab, max_seq, max_splits;
    float eps;
    md_devflags* flags;
    unsigned long long* trace;  // optional [2][256] timestamps (ns) of the first and last CTA, for tuning
};

// True when the model has the geometry the kernel is specialised for.
bool md_decode_persistent_supported(size_t dim, size_t hidden, size_t n_heads, size_t head_dim, size_t rot_dim,
                                    size_t vocab, size_t n_layers, size_t batch);
// Scratch the attention phase needs, in bytes, and the launch itself (cooperative, one CTA per SM).
size_t md_decode_persistent_scratch_bytes(size_t batch, size_t max_seq);
int md_launch_decode_persistent(md_ctx* ctx, const md_persist_params& p);
