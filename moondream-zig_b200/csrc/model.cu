// Device-resident restatement of the reference's model control flow on top of the hot-path
// kernels: text_model.zig:106-345 (text_encoder, text_decoder, lm_head, KVCache) and
// vision_model.zig:160-387 (normalise, patchify, vision_encoder, encode_mlp), plus the greedy
// generation loop of moondream.zig:323-368.  Host code + a few tiny kernels; every matmul goes
// through md_gemm_dispatch (GEMV for <= 8 rows, tcgen05 GEMM otherwise) with the reference's
// glue fused into the epilogue at the reference's rounding points.
#include "md_internal.cuh"

#include "../../include/moondream_b200_model.h"

#include <cstring>

extern "C" int md_gemm_dispatch(md_ctx* ctx, const __half* a, const __half* b, __half* c, size_t M, size_t N, size_t K,
                                int b_layout, const md_epilogue& ep);
int md_launch_sdpa_decode_fused_devpos_batch(md_ctx* ctx, const __half* qkv, size_t qkv_stride, __half* const* kc,
                                             __half* const* vc, __half* out, size_t out_stride, size_t batch,
                                             size_t n_heads, size_t d, size_t max_seq, const int* const* pos_dev,
                                             size_t rot_dim, float theta);

namespace {

// hidden[r, :] = wte[token[r], :]   (text_model.zig:106-137), tokens in device memory
__global__ void embed_kernel(const __half* __restrict__ wte, const unsigned long long* __restrict__ tokens,
                             __half* __restrict__ out, int dim, int vocab) {
    const unsigned long long tok = tokens[blockIdx.x];
    const __half* src = wte + (size_t)(tok < (unsigned long long)vocab ? tok : 0) * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) out[(size_t)blockIdx.x * dim + i] = src[i];
}

// End of a decode step for `batch` requests: record the sampled tokens, choose the next input
// (teacher forcing or the sample), advance positions and the step counter, and gather the next
// step's embeddings (text_model.zig:106-137) so the step needs no separate embedding kernel.
// `sampled` holds token indices, or (keys != 0) the 64-bit argmax keys the fused lm_head leaves:
// (ordered value << 32) | (0xFFFFFFFF - index); the keys are cleared for the next step.
__global__ void __launch_bounds__(256)
advance_kernel(unsigned long long* cur_tokens, unsigned long long* sampled, int keys, int batch,
               unsigned int* tokens_out, int n_steps, const unsigned int* forced, int* step, int* const* pos_ptrs,
               const __half* __restrict__ wte, __half* __restrict__ hidden, int dim, int vocab) {
    __shared__ unsigned long long next_tok[8];
    const int b = threadIdx.x;
    const int s = *step;
    if (b < batch) {
        unsigned long long tok = sampled[b];
        if (keys) {
            tok = 0xFFFFFFFFull - (tok & 0xFFFFFFFFull);
            sampled[b] = 0ull;
        }
        if (s < n_steps) tokens_out[(size_t)b * n_steps + s] = (unsigned int)tok;
        const unsigned long long nxt =
            (forced && s < n_steps) ? (unsigned long long)forced[(size_t)b * n_steps + s] : tok;
        cur_tokens[b] = nxt;
        next_tok[b] = nxt < (unsigned long long)vocab ? nxt : 0ull;
        *pos_ptrs[b] += 1;
    }
    __syncthreads();
    if (b == 0) *step = s + 1;
    // the embedding rows of the next tokens; 16 bytes per thread where the rows allow it, all rows requested at once
    if ((dim & 7) == 0 && ((reinterpret_cast<uintptr_t>(wte) | reinterpret_cast<uintptr_t>(hidden)) & 15) == 0) {
        const int vec = dim >> 3;
        for (int i = threadIdx.x; i < batch * vec; i += blockDim.x) {
            const int r = i / vec, c = i - r * vec;
            reinterpret_cast<uint4*>(hidden)[(size_t)r * vec + c] =
                __ldg(reinterpret_cast<const uint4*>(wte + (size_t)next_tok[r] * dim) + c);
        }
    } else {
        for (int r = 0; r < batch; ++r) {
            const __half* src = wte + (size_t)next_tok[r] * dim;
            for (int i = threadIdx.x; i < dim; i += blockDim.x) hidden[(size_t)r * dim + i] = src[i];
        }
    }
}

__global__ void copy_logits_kernel(const __half* __restrict__ logits, __half* __restrict__ all, int vocab,
                                   const int* step) {
    __half* dst = all + (size_t)(*step) * vocab;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) dst[i] = logits[i];
}

__global__ void set_int_kernel(int* p, int v) { *p = v; }

struct DevPtr {
    void* p = nullptr;
    size_t cap = 0;
    ~DevPtr() { if (p) cudaFree(p); }
    int ensure(md_ctx* ctx, size_t bytes) {
        if (cap >= bytes) return MD_OK;
        if (ctx->capturing) return md_fail(ctx, MD_ERR_UNSUPPORTED, "buffer growth during graph capture");
        if (p) {
            MD_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            MD_CUDA(ctx, cudaFree(p));
            p = nullptr;
            cap = 0;
        }
        MD_CUDA(ctx, cudaMalloc(&p, bytes));
        cap = bytes;
        return MD_OK;
    }
    template <class T> T* as() const { return reinterpret_cast<T*>(p); }
};

template <class T> std::vector<T> copy_ptrs(const T* src, size_t n) { return std::vector<T>(src, src + n); }

int copy_out(md_ctx* ctx, void* user, const void* dev, size_t bytes) {
    if (!user || !bytes) return MD_OK;
    const cudaMemcpyKind kind = md_is_device_ptr(user) ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost;
    MD_CUDA(ctx, cudaMemcpyAsync(user, dev, bytes, kind, ctx->stream));
    return MD_OK;
}

}  // namespace

// ------------------------------------------------------------------------------------ text

struct md_text_model {
    md_ctx* ctx;
    md_text_weights w;
    std::vector<const uint16_t*> ln_w, ln_b, wqkv, bqkv, wout, bout, wfc1, bfc1, wfc2, bfc2;
};

struct md_text_request {
    md_text_model* model;
    std::vector<__half*> kc, vc;  // per layer [n_heads][max_seq][head_dim]
    size_t pos = 0;               // host mirror of *pos_dev
    int* pos_dev = nullptr;
    // activations of one forward over `rows` rows
    DevPtr hidden, ln, qkv, attn, attn_out, fc1, logits, ln_last;
    DevPtr mlp_part;  // up to four f32 [8, dim] partial products of fc2 (the decode layer whose MLP runs as two half-width chains)
    // device-side generation state
    DevPtr cur_token, sampled, tokens_out, forced, step, logits_all, pos_ptrs;
    md_graph* graph = nullptr;
    uint64_t graph_gen = 0, prefill_graph_gen = 0;  // md_ctx::generation the graphs were captured under
    size_t graph_steps = 0;
    bool graph_forced = false, graph_logits = false;
    // a prefill of the same shape at the same position seen twice is captured and replayed
    md_graph* prefill_graph = nullptr;
    size_t prefill_S = 0, prefill_pos = 0, seen_S = 0, seen_pos = ~(size_t)0;
};

namespace {

// While alive, the kernels that implement the programmatic-dependent-launch protocol (GEMV, tcgen05 GEMM and
// attention, LayerNorm, rope) are launched dependent on their predecessor: each starts its set-up while the
// previous one drains and waits (griddepcontrol.wait) before touching global memory.
struct PdlScope {
    md_ctx* c;
    int old;
    explicit PdlScope(md_ctx* cc) : c(cc), old(cc->pdl) { c->pdl = 1; }
    ~PdlScope() { c->pdl = old; }
};

// Overrides the automatic (warps, unroll) choice of the GEMV kernel for a scope, unless the caller fixed one.
struct GemvVariantScope {
    md_ctx* c;
    int old;
    GemvVariantScope(md_ctx* cc, int variant) : c(cc), old(cc->gemv_variant) {
        if (old == 0 && variant) c->gemv_variant = variant;
    }
    ~GemvVariantScope() { c->gemv_variant = old; }
};

const __half* H(const uint16_t* p) { return reinterpret_cast<const __half*>(p); }
__half* H(uint16_t* p) { return reinterpret_cast<__half*>(p); }

float eps_of(uint16_t bits) {
    __half_raw r;
    r.x = bits;
    return __half2float(__half(r));
}

int ensure_rows(md_text_request* r, size_t rows) {
    md_ctx* ctx = r->model->ctx;
    const md_text_weights& w = r->model->w;
    if (r->graph && r->hidden.cap < rows * w.dim * 2) {
        // the buffers are about to move: a captured decode step that points at them is stale
        md_graph_destroy(ctx, r->graph);
        r->graph = nullptr;
    }
    if (r->prefill_graph && r->hidden.cap < rows * w.dim * 2) {
        md_graph_destroy(ctx, r->prefill_graph);
        r->prefill_graph = nullptr;
    }
    MD_TRY(r->hidden.ensure(ctx, rows * w.dim * 2));
    MD_TRY(r->ln.ensure(ctx, rows * w.dim * 2));
    MD_TRY(r->qkv.ensure(ctx, rows * 3 * w.dim * 2));
    MD_TRY(r->attn.ensure(ctx, rows * w.dim * 2));
    MD_TRY(r->attn_out.ensure(ctx, rows * w.dim * 2));
    MD_TRY(r->fc1.ensure(ctx, rows * w.hidden * 2));
    MD_TRY(r->logits.ensure(ctx, 8 * w.vocab * 2));
    MD_TRY(r->ln_last.ensure(ctx, 8 * w.dim * 2));
    MD_TRY(r->mlp_part.ensure(ctx, 4 * 8 * w.dim * sizeof(float)));
    return MD_OK;
}

// One decoder layer over `rows` rows held in bufs->hidden (text_model.zig:150-172).
//   prefill: rows = S tokens of one request, host-known position
//   decode : rows = batch requests, one token each, positions in device memory
struct LayerIO {
    __half *hidden, *ln, *qkv, *attn, *attn_out, *fc1;
    float* mlp_part;
};

// Attention of one decode step: every request's new token against its own cache, one launch for the batch.
int decode_attention(md_text_model* m, size_t layer, const LayerIO& io, size_t rows, md_text_request* const* reqs) {
    const md_text_weights& w = m->w;
    __half *kc[8], *vc[8];
    const int* pos[8];
    for (size_t b = 0; b < rows; ++b) {
        kc[b] = reqs[b]->kc[layer];
        vc[b] = reqs[b]->vc[layer];
        pos[b] = reqs[b]->pos_dev;
    }
    return md_launch_sdpa_decode_fused_devpos_batch(m->ctx, io.qkv, 3 * w.dim, kc, vc, io.attn, w.dim, rows, w.n_heads,
                                                    w.head_dim, w.max_seq, pos, w.rot_dim, w.rope_theta);
}

int text_layer(md_text_model* m, size_t layer, const LayerIO& io, size_t rows, bool decode,
               md_text_request* const* reqs, size_t prefill_pos) {
    md_ctx* ctx = m->ctx;
    const md_text_weights& w = m->w;
    const size_t D = w.dim, F = w.hidden;
    // The fused kernels recompute the LayerNorm of all rows in every CTA; with many rows that costs registers
    // (one CTA per SM instead of two) and L2 reads, so from ctx->decode_split_ln rows on the LayerNorm runs once
    // as its own kernel and plain GEMVs with fused epilogues follow (the generic path below, forked the same way).
    const bool ln_once = ctx->decode_split_ln > 0 && rows >= (size_t)ctx->decode_split_ln;
    if (decode && ctx->fused_decode && !ln_once && md_gemv_ln_dual_supported(rows, D, 3 * D, F) &&
        md_gemv_dual_k_supported(rows, D, D, F)) {
        if (ctx->decode_fork) {
            // Two concurrent chains per layer, so that the weight stream of the MLP fills the time the attention
            // chain spends on latency (q/k/v projection -> attention -> out-projection move 33 MB, the MLP 67 MB):
            //   main: [LayerNorm + qkv] -> attention ------------------> [out-proj + bias + mlp_out + hidden]
            //   side: [LayerNorm + fc1 + GELU] -> [fc2 + bias -> mlp_out] --^
            // Same rounding points as the reference: attn_out = f16(f16(acc) + b), mlp_out likewise,
            // attn_out += mlp_out, hidden += attn_out (text_model.zig:162-171).
            if (!ctx->side_stream) {
                MD_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->side_stream, cudaStreamNonBlocking));
                MD_CUDA(ctx, cudaEventCreateWithFlags(&ctx->ev_fork, cudaEventDisableTiming));
                MD_CUDA(ctx, cudaEventCreateWithFlags(&ctx->ev_side, cudaEventDisableTiming));
            }
            cudaStream_t main_stream = ctx->stream;
            MD_CUDA(ctx, cudaEventRecord(ctx->ev_fork, main_stream));            // hidden of the previous layer is final
            const int parts = ctx->decode_mlp_split;
            if (rows == 1 && (parts == 2 || parts == 4) && io.mlp_part && (F % (32 * parts)) == 0) {
                // Single request: the MLP chain (fc1 -> fc2, 67 MB) is the longest path of the layer, so it runs as
                // 2 or 4 independent chains: chain h computes rows h*F/parts.. of fc1 (+ bias + GELU) and then the part
                // of fc2's K sum over those features, as raw f32 sums; the out-projection's epilogue adds the parts,
                // rounds once, adds fc2's bias and continues as before (mlp_out = f16(f16(acc) + b)).
                const size_t Fh = F / parts;
                int st = MD_OK;
                for (int h = 0; h < parts && st == MD_OK; ++h) {
                    if (h > 0 && !ctx->mlp_stream[h - 1]) {
                        MD_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->mlp_stream[h - 1], cudaStreamNonBlocking));
                        MD_CUDA(ctx, cudaEventCreateWithFlags(&ctx->ev_mlp[h - 1], cudaEventDisableTiming));
                    }
                    cudaStream_t ss = h ? ctx->mlp_stream[h - 1] : ctx->side_stream;
                    if (cudaStreamWaitEvent(ss, ctx->ev_fork, 0) != cudaSuccess) st = md_fail(ctx, MD_ERR_CUDA, "cudaStreamWaitEvent failed");
                    ctx->stream = ss;
                    if (st == MD_OK)
                        st = md_launch_gemv_ln_dual(ctx, io.hidden, H(m->ln_w[layer]), H(m->ln_b[layer]), eps_of(w.eps_f16),
                                                    H(m->wfc1[layer]) + h * Fh * D, H(m->bfc1[layer]) + h * Fh, io.fc1 + h * Fh,
                                                    Fh, nullptr, nullptr, nullptr, 0, rows, D, nullptr, true);
                    if (st == MD_OK) {
                        md_epilogue e_part;
                        e_part.out_f32 = io.mlp_part + h * 8 * D;
                        st = md_launch_gemv_nt(ctx, io.fc1 + h * Fh, H(m->wfc2[layer]) + h * Fh, io.attn_out, rows, D, Fh, e_part, F);
                    }
                    if (st == MD_OK && cudaEventRecord(h ? ctx->ev_mlp[h - 1] : ctx->ev_side, ss) != cudaSuccess)
                        st = md_fail(ctx, MD_ERR_CUDA, "cudaEventRecord on a side stream failed");
                }
                ctx->stream = main_stream;
                MD_TRY(st);
                MD_TRY(md_launch_gemv_ln_dual(ctx, io.hidden, H(m->ln_w[layer]), H(m->ln_b[layer]), eps_of(w.eps_f16),
                                              H(m->wqkv[layer]), H(m->bqkv[layer]), io.qkv, 3 * D, nullptr, nullptr, nullptr, 0,
                                              rows, D));
                MD_TRY(decode_attention(m, layer, io, rows, reqs));
                MD_CUDA(ctx, cudaStreamWaitEvent(main_stream, ctx->ev_side, 0));
                for (int h = 1; h < parts; ++h) MD_CUDA(ctx, cudaStreamWaitEvent(main_stream, ctx->ev_mlp[h - 1], 0));
                md_epilogue e_out;
                e_out.bias = H(m->bout[layer]);
                e_out.parts = io.mlp_part;
                e_out.n_parts = parts;
                e_out.part_stride = (int)(8 * D);
                e_out.bias2 = H(m->bfc2[layer]);
                e_out.residual2 = io.hidden;    // updated in place: every element is read and written by one thread
                return md_launch_gemv_nt(ctx, io.attn, H(m->wout[layer]), io.hidden, rows, D, D, e_out);
            }
            MD_CUDA(ctx, cudaStreamWaitEvent(ctx->side_stream, ctx->ev_fork, 0));
            ctx->stream = ctx->side_stream;
            int st = md_launch_gemv_ln_dual(ctx, io.hidden, H(m->ln_w[layer]), H(m->ln_b[layer]), eps_of(w.eps_f16),
                                            H(m->wfc1[layer]), H(m->bfc1[layer]), io.fc1, F, nullptr, nullptr, nullptr, 0,
                                            rows, D, nullptr, true);
            if (st == MD_OK) {
                md_epilogue e_fc2;
                e_fc2.bias = H(m->bfc2[layer]);
                st = md_launch_gemv_nt(ctx, io.fc1, H(m->wfc2[layer]), io.attn_out, rows, D, F, e_fc2);
            }
            if (st == MD_OK && cudaEventRecord(ctx->ev_side, ctx->side_stream) != cudaSuccess)
                st = md_fail(ctx, MD_ERR_CUDA, "cudaEventRecord on the side stream failed");
            ctx->stream = main_stream;
            MD_TRY(st);
            // (launch priorities for either chain were measured and made the step slower: both chains run at
            // the stream's priority)
            MD_TRY(md_launch_gemv_ln_dual(ctx, io.hidden, H(m->ln_w[layer]), H(m->ln_b[layer]), eps_of(w.eps_f16),
                                          H(m->wqkv[layer]), H(m->bqkv[layer]), io.qkv, 3 * D, nullptr, nullptr, nullptr, 0,
                                          rows, D));
            MD_TRY(decode_attention(m, layer, io, rows, reqs));
            MD_CUDA(ctx, cudaStreamWaitEvent(main_stream, ctx->ev_side, 0));
            md_epilogue e_out;
            e_out.bias = H(m->bout[layer]);
            e_out.residual = io.attn_out;   // mlp_out
            e_out.residual2 = io.hidden;    // updated in place: every element is read and written by one thread
            return md_launch_gemv_nt(ctx, io.attn, H(m->wout[layer]), io.hidden, rows, D, D, e_out);
        }
        // Three kernels per layer: [LayerNorm + qkv + fc1] -> attention -> [out-proj + fc2 + residuals]
        MD_TRY(md_launch_gemv_ln_dual(ctx, io.hidden, H(m->ln_w[layer]), H(m->ln_b[layer]), eps_of(w.eps_f16),
                                      H(m->wqkv[layer]), H(m->bqkv[layer]), io.qkv, 3 * D, H(m->wfc1[layer]),
                                      H(m->bfc1[layer]), io.fc1, F, rows, D));
        MD_TRY(decode_attention(m, layer, io, rows, reqs));
        return md_launch_gemv_dual_k(ctx, io.attn, H(m->wout[layer]), H(m->bout[layer]), D, io.fc1, H(m->wfc2[layer]),
                                     H(m->bfc2[layer]), F, io.hidden, D, rows);
    }
    MD_TRY(md_launch_layernorm(ctx, io.hidden, H(m->ln_w[layer]), H(m->ln_b[layer]), io.ln, rows, D, eps_of(w.eps_f16)));
    // Prefill: the MLP of a Phi layer reads the same LayerNorm output as the attention, so fc1 -> fc2 run as a
    // second kernel chain beside qkv -> rope -> attention; the GEMMs of one chain that cover only part of the SMs
    // (96 tiles for the 2048-wide outputs at 761 rows) leave the rest to the other chain.  The chains meet in the
    // out-projection's epilogue (same roundings as the sequential form, text_model.zig:162-171).
    const bool fork_prefill = ctx->prefill_fork && (decode ? ctx->decode_fork != 0 : rows > 8);
    if (fork_prefill) {
        if (!ctx->side_stream) {
            MD_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->side_stream, cudaStreamNonBlocking));
            MD_CUDA(ctx, cudaEventCreateWithFlags(&ctx->ev_fork, cudaEventDisableTiming));
            MD_CUDA(ctx, cudaEventCreateWithFlags(&ctx->ev_side, cudaEventDisableTiming));
        }
        cudaStream_t main_stream = ctx->stream;
        MD_CUDA(ctx, cudaEventRecord(ctx->ev_fork, main_stream));  // LayerNorm output ready
        MD_CUDA(ctx, cudaStreamWaitEvent(ctx->side_stream, ctx->ev_fork, 0));
        ctx->stream = ctx->side_stream;
        md_epilogue e_fc1, e_fc2;
        e_fc1.bias = H(m->bfc1[layer]);
        e_fc1.gelu = 1;
        e_fc2.bias = H(m->bfc2[layer]);
        int st = md_gemm_dispatch(ctx, io.ln, H(m->wfc1[layer]), io.fc1, rows, F, D, 1, e_fc1);
        if (st == MD_OK) st = md_gemm_dispatch(ctx, io.fc1, H(m->wfc2[layer]), io.attn_out, rows, D, F, 1, e_fc2);
        if (st == MD_OK && cudaEventRecord(ctx->ev_side, ctx->side_stream) != cudaSuccess)
            st = md_fail(ctx, MD_ERR_CUDA, "cudaEventRecord on the side stream failed");
        ctx->stream = main_stream;
        MD_TRY(st);
    }
    md_epilogue e_qkv;
    e_qkv.bias = H(m->bqkv[layer]);
    MD_TRY(md_gemm_dispatch(ctx, io.ln, H(m->wqkv[layer]), io.qkv, rows, 3 * D, D, 1, e_qkv));
    if (decode) {
        MD_TRY(decode_attention(m, layer, io, rows, reqs));
    } else {
        md_text_request* r = reqs[0];
        void* q_rot = nullptr;
        MD_TRY(md_scratch(ctx, rows * D * 2, &q_rot));
        MD_TRY(md_launch_rope_cache_write(ctx, io.qkv, (__half*)q_rot, r->kc[layer], r->vc[layer], rows, w.n_heads,
                                          w.head_dim, w.max_seq, prefill_pos, w.rot_dim, w.rope_theta));
        MD_TRY(md_launch_sdpa(ctx, (const __half*)q_rot, r->kc[layer], r->vc[layer], nullptr, io.attn, w.n_heads, rows,
                              prefill_pos + rows, w.head_dim, D, w.head_dim, w.head_dim, w.max_seq * w.head_dim, D,
                              w.head_dim, 1, 0, 0, 0, (int)prefill_pos));
    }
    md_epilogue e_out;
    e_out.bias = H(m->bout[layer]);
    if (fork_prefill) {
        // join the MLP chain: attn_out = f16(f16(acc) + b); attn_out += mlp_out; hidden += attn_out
        MD_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->ev_side, 0));
        e_out.residual = io.attn_out;  // mlp_out, written by the side chain
        e_out.residual2 = io.hidden;   // updated in place
        return md_gemm_dispatch(ctx, io.attn, H(m->wout[layer]), io.hidden, rows, D, D, 1, e_out);
    }
    MD_TRY(md_gemm_dispatch(ctx, io.attn, H(m->wout[layer]), io.attn_out, rows, D, D, 1, e_out));
    md_epilogue e_fc1;
    e_fc1.bias = H(m->bfc1[layer]);
    e_fc1.gelu = 1;
    MD_TRY(md_gemm_dispatch(ctx, io.ln, H(m->wfc1[layer]), io.fc1, rows, F, D, 1, e_fc1));
    // fc2 + bias, then attn_out += mlp_out, then hidden += attn_out (text_model.zig:170-171),
    // each with its own f16 rounding, written back into hidden.
    md_epilogue e_fc2;
    e_fc2.bias = H(m->bfc2[layer]);
    e_fc2.residual = io.attn_out;
    e_fc2.residual2 = io.hidden;
    MD_TRY(md_gemm_dispatch(ctx, io.fc1, H(m->wfc2[layer]), io.hidden, rows, D, F, 1, e_fc2));
    return MD_OK;
}

LayerIO io_of(md_text_request* r) {
    return LayerIO{r->hidden.as<__half>(), r->ln.as<__half>(), r->qkv.as<__half>(), r->attn.as<__half>(),
                   r->attn_out.as<__half>(), r->fc1.as<__half>(), r->mlp_part.as<float>()};
}

// lm_head over `rows` hidden rows (text_model.zig:325-345 takes the last row of one request; the
// batched decode applies it to one row per request) followed by the greedy sample of each row.
int text_lm_head(md_text_model* m, const __half* hidden_rows, size_t rows, __half* ln_buf, __half* logits,
                 unsigned long long* sampled) {
    md_ctx* ctx = m->ctx;
    const md_text_weights& w = m->w;
    MD_TRY(md_launch_layernorm(ctx, hidden_rows, H(w.ln_out_w), H(w.ln_out_b), ln_buf, rows, w.dim, eps_of(w.eps_f16)));
    md_epilogue e;
    e.bias = H(w.lm_b);
    MD_TRY(md_gemm_dispatch(ctx, ln_buf, H(w.lm_w), logits, rows, w.vocab, w.dim, 1, e));
    MD_TRY(md_launch_argmax_rows(ctx, logits, w.vocab, w.vocab, rows, sampled));
    return MD_OK;
}

}  // namespace

extern "C" {

int md_text_model_create(md_ctx* ctx, const md_text_weights* w, md_text_model** out) {
    if (!ctx) return MD_ERR_INVALID_ARG;
    if (!w || !out) return md_fail(ctx, MD_ERR_INVALID_ARG, "md_text_model_create: null argument");
    if (w->dim != w->n_heads * w->head_dim || w->head_dim != 64)
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "text model needs dim == n_heads * head_dim and head_dim == 64");
    if (w->rot_dim > w->head_dim || (w->rot_dim & 1)) return md_fail(ctx, MD_ERR_INVALID_ROT_DIM, "rot_dim %zu", w->rot_dim);
    md_text_model* m = new md_text_model();
    m->ctx = ctx;
    m->w = *w;
    const size_t L = w->n_layers;
    m->ln_w = copy_ptrs(w->ln_w, L); m->ln_b = copy_ptrs(w->ln_b, L);
    m->wqkv = copy_ptrs(w->wqkv, L); m->bqkv = copy_ptrs(w->bqkv, L);
    m->wout = copy_ptrs(w->wout, L); m->bout = copy_ptrs(w->bout, L);
    m->wfc1 = copy_ptrs(w->wfc1, L); m->bfc1 = copy_ptrs(w->bfc1, L);
    m->wfc2 = copy_ptrs(w->wfc2, L); m->bfc2 = copy_ptrs(w->bfc2, L);
    *out = m;
    return MD_OK;
}

int md_text_model_destroy(md_text_model* model) {
    delete model;
    return MD_OK;
}

int md_text_request_create(md_text_model* model, md_text_request** out) {
    if (!model || !out) return MD_ERR_INVALID_ARG;
    md_ctx* ctx = model->ctx;
    const md_text_weights& w = model->w;
    md_text_request* r = new md_text_request();
    r->model = model;
    const size_t cache_bytes = w.n_heads * w.max_seq * w.head_dim * 2;
    for (size_t l = 0; l < w.n_layers; ++l) {
        void *k = nullptr, *v = nullptr;
        if (cudaMalloc(&k, cache_bytes) != cudaSuccess || cudaMalloc(&v, cache_bytes) != cudaSuccess) {
            cudaGetLastError();
            if (k) cudaFree(k);
            md_text_request_destroy(r);
            return md_fail(ctx, MD_ERR_OOM, "KV cache allocation failed (layer %zu)", l);
        }
        r->kc.push_back((__half*)k);
        r->vc.push_back((__half*)v);
    }
    if (cudaMalloc((void**)&r->pos_dev, sizeof(int)) != cudaSuccess) {
        md_text_request_destroy(r);
        return md_fail(ctx, MD_ERR_OOM, "request state allocation failed");
    }
    cudaMemsetAsync(r->pos_dev, 0, sizeof(int), ctx->stream);
    int st = ensure_rows(r, 8);
    if (st == MD_OK) st = r->cur_token.ensure(ctx, 8 * sizeof(unsigned long long));
    if (st == MD_OK) st = r->sampled.ensure(ctx, 8 * sizeof(unsigned long long));
    if (st == MD_OK) st = r->step.ensure(ctx, sizeof(int));
    if (st != MD_OK) {
        md_text_request_destroy(r);
        return st;
    }
    *out = r;
    return MD_OK;
}

int md_text_request_destroy(md_text_request* req) {
    if (!req) return MD_OK;
    md_ctx* ctx = req->model->ctx;
    cudaStreamSynchronize(ctx->stream);
    if (req->graph) md_graph_destroy(ctx, req->graph);
    if (req->prefill_graph) md_graph_destroy(ctx, req->prefill_graph);
    for (auto p : req->kc) cudaFree(p);
    for (auto p : req->vc) cudaFree(p);
    if (req->pos_dev) cudaFree(req->pos_dev);
    delete req;
    return MD_OK;
}

int md_text_request_reset(md_text_request* req) {
    if (!req) return MD_ERR_INVALID_ARG;
    md_ctx* ctx = req->model->ctx;
    req->pos = 0;
    MD_CUDA(ctx, cudaMemsetAsync(req->pos_dev, 0, sizeof(int), ctx->stream));
    return MD_OK;
}

int md_text_request_len(const md_text_request* req, size_t* len_out) {
    if (!req || !len_out) return MD_ERR_INVALID_ARG;
    *len_out = req->pos;
    return MD_OK;
}

int md_text_encoder(md_text_model* model, const uint32_t* ids, size_t n, uint16_t* out) {
    if (!model) return MD_ERR_INVALID_ARG;
    md_ctx* ctx = model->ctx;
    if (!ids || !out) return md_fail(ctx, MD_ERR_INVALID_ARG, "text_encoder: null pointer");
    const md_text_weights& w = model->w;
    if (n > w.max_seq) return md_fail(ctx, MD_ERR_SEQUENCE_TOO_LONG, "text_encoder: %zu ids > %zu", n, w.max_seq);
    std::vector<unsigned long long> wide(n);
    for (size_t i = 0; i < n; ++i) {
        if (ids[i] >= w.vocab) return md_fail(ctx, MD_ERR_INVALID_ARG, "text_encoder: token id %u out of bounds", ids[i]);
        wide[i] = ids[i];
    }
    if (n == 0) return MD_OK;
    void* scratch = nullptr;
    const size_t ids_bytes = (n * 8 + 255) & ~(size_t)255;
    MD_TRY(md_scratch(ctx, ids_bytes + n * w.dim * 2, &scratch));
    MD_CUDA(ctx, cudaMemcpyAsync(scratch, wide.data(), n * 8, cudaMemcpyHostToDevice, ctx->stream));
    __half* rows = reinterpret_cast<__half*>((char*)scratch + ids_bytes);
    const bool to_dev = md_is_device_ptr(out);
    __half* dst = to_dev ? H(out) : rows;
    embed_kernel<<<(unsigned)n, 256, 0, ctx->stream>>>(H(w.wte), (const unsigned long long*)scratch, dst, (int)w.dim,
                                                       (int)w.vocab);
    MD_LAUNCH_CHECK(ctx, "embed_kernel");
    if (!to_dev) MD_CUDA(ctx, cudaMemcpyAsync(out, rows, n * w.dim * 2, cudaMemcpyDeviceToHost, ctx->stream));
    MD_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // `wide` goes out of scope
    return MD_OK;
}

int md_text_forward(md_text_model* model, md_text_request* req, const uint16_t* embeds, size_t S,
                    uint16_t* hidden_out, uint16_t* logits_out, uint64_t* token_out) {
    if (!model || !req) return MD_ERR_INVALID_ARG;
    md_ctx* ctx = model->ctx;
    const md_text_weights& w = model->w;
    if (!embeds || S == 0) return md_fail(ctx, MD_ERR_INVALID_ARG, "text_forward: no input rows");
    if (req->pos + S > w.max_seq)
        return md_fail(ctx, MD_ERR_SEQUENCE_TOO_LONG, "text_forward: %zu cached + %zu new tokens exceed %zu", req->pos, S,
                       w.max_seq);
    MD_TRY(ensure_rows(req, S > 8 ? S : 8));
    const cudaMemcpyKind kind = md_is_device_ptr(embeds) ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    MD_CUDA(ctx, cudaMemcpyAsync(req->hidden.p, embeds, S * w.dim * 2, kind, ctx->stream));
    const LayerIO io = io_of(req);
    md_text_request* reqs[1] = {req};
    const size_t pos0 = req->pos;
    // S == 1 takes the decode kernels (text_model.zig:284-290 switches on seq_len == 1 as well)
    auto body = [&]() -> int {
        PdlScope pdl_scope(ctx);
        for (size_t l = 0; l < w.n_layers; ++l) MD_TRY(text_layer(model, l, io, S, S == 1, reqs, pos0));
        set_int_kernel<<<1, 1, 0, ctx->stream>>>(req->pos_dev, (int)(pos0 + S));
        MD_LAUNCH_CHECK(ctx, "set_int_kernel");
        return MD_OK;
    };
    if (S > 1 && req->prefill_graph && req->prefill_S == S && req->prefill_pos == pos0 &&
        req->prefill_graph_gen == ctx->generation) {
        MD_TRY(md_graph_launch(ctx, req->prefill_graph));
    } else {
        MD_TRY(body());
        if (S > 1 && !ctx->capturing && req->seen_S == S && req->seen_pos == pos0) {
            // second prefill of this shape: record it (the ~170 launches are host-bound when issued one by one)
            if (req->prefill_graph) { md_graph_destroy(ctx, req->prefill_graph); req->prefill_graph = nullptr; }
            MD_TRY(md_graph_begin(ctx));
            const int st = body();
            md_graph* g = nullptr;
            const int st2 = md_graph_end(ctx, &g);
            if (st == MD_OK && st2 == MD_OK) {
                req->prefill_graph = g;
                req->prefill_graph_gen = ctx->generation;
                req->prefill_S = S;
                req->prefill_pos = pos0;
            } else if (g) {
                md_graph_destroy(ctx, g);
            }
        }
        req->seen_S = S;
        req->seen_pos = pos0;
    }
    req->pos = pos0 + S;
    MD_TRY(copy_out(ctx, hidden_out, req->hidden.p, S * w.dim * 2));
    if (logits_out || token_out) {
        MD_TRY(text_lm_head(model, req->hidden.as<__half>() + (S - 1) * w.dim, 1, req->ln_last.as<__half>(),
                            req->logits.as<__half>(), req->sampled.as<unsigned long long>()));
        MD_TRY(copy_out(ctx, logits_out, req->logits.p, w.vocab * 2));
        MD_TRY(copy_out(ctx, token_out, req->sampled.p, sizeof(uint64_t)));
    }
    return md_check_flags(ctx);
}

// Enqueue one decode step for `batch` requests that share the activation buffers of reqs[0].
static int enqueue_decode_step(md_text_model* model, md_text_request* const* reqs, size_t batch, size_t n_steps,
                               bool forced, bool keep_logits) {
    md_ctx* ctx = model->ctx;
    const md_text_weights& w = model->w;
    md_text_request* r0 = reqs[0];
    // registered weights are never written on this stream: the GEMVs may overlap their predecessors' tails
    PdlScope pdl_scope(ctx);
    // hidden already holds the embeddings of the current tokens (generate_impl / the previous advance_kernel)
    const LayerIO io = io_of(r0);
    const bool ln_once = ctx->decode_split_ln > 0 && batch >= (size_t)ctx->decode_split_ln;
    // The automatic GEMV variant is tuned for isolated calls; inside the decode step, where two kernel chains share
    // the SMs, 8 warps with 8 loads in flight per lane measured best for every GEMV and every batch size
    // (742 -> 730 us per step at 1 row, 962 -> 942 at 4 rows, 1210 -> 1079 at 6 rows).
    GemvVariantScope gemv_scope(ctx, 3);
    for (size_t l = 0; l < w.n_layers; ++l) MD_TRY(text_layer(model, l, io, batch, true, reqs, 0));
    const bool fused_head = ctx->fused_decode && !ln_once && md_gemv_ln_dual_supported(batch, w.dim, w.vocab, 0);
    if (fused_head) {
        // final LayerNorm + lm_head + greedy argmax in one kernel (text_model.zig:325-345, sampling.zig:257-273)
        MD_TRY(md_launch_gemv_ln_dual(ctx, r0->hidden.as<__half>(), H(w.ln_out_w), H(w.ln_out_b), eps_of(w.eps_f16),
                                      H(w.lm_w), H(w.lm_b), r0->logits.as<__half>(), w.vocab, nullptr, nullptr, nullptr,
                                      0, batch, w.dim, r0->sampled.as<unsigned long long>()));
    } else {
        MD_TRY(text_lm_head(model, r0->hidden.as<__half>(), batch, r0->ln_last.as<__half>(), r0->logits.as<__half>(),
                            r0->sampled.as<unsigned long long>()));
    }
    if (keep_logits) {
        copy_logits_kernel<<<32, 256, 0, ctx->stream>>>(r0->logits.as<__half>(), r0->logits_all.as<__half>(),
                                                        (int)w.vocab, r0->step.as<int>());
        MD_LAUNCH_CHECK(ctx, "copy_logits_kernel");
    }
    advance_kernel<<<1, 256, 0, ctx->stream>>>(r0->cur_token.as<unsigned long long>(),
                                               r0->sampled.as<unsigned long long>(), fused_head ? 1 : 0, (int)batch,
                                               r0->tokens_out.as<unsigned int>(), (int)n_steps,
                                               forced ? r0->forced.as<unsigned int>() : nullptr, r0->step.as<int>(),
                                               r0->pos_ptrs.as<int*>(), H(w.wte), r0->hidden.as<__half>(), (int)w.dim,
                                               (int)w.vocab);
    MD_LAUNCH_CHECK(ctx, "advance_kernel");
    return MD_OK;
}

static int generate_impl(md_text_model* model, md_text_request* const* reqs, size_t batch, const uint32_t* first,
                         size_t n_steps, uint32_t* tokens_out, const uint32_t* forced, uint16_t* logits_out) {
    md_ctx* ctx = model->ctx;
    const md_text_weights& w = model->w;
    if (batch == 0 || batch > 8) return md_fail(ctx, MD_ERR_INVALID_ARG, "generate: batch must be 1..8");
    if (!first || !tokens_out) return md_fail(ctx, MD_ERR_INVALID_ARG, "generate: null pointer");
    if (n_steps == 0) return MD_OK;
    for (size_t b = 0; b < batch; ++b) {
        if (!reqs[b] || reqs[b]->model != model) return md_fail(ctx, MD_ERR_INVALID_ARG, "generate: foreign request");
        if (reqs[b]->pos + n_steps > w.max_seq)
            return md_fail(ctx, MD_ERR_SEQUENCE_TOO_LONG, "generate: request %zu holds %zu tokens, %zu more exceed %zu", b,
                           reqs[b]->pos, n_steps, w.max_seq);
        if (first[b] >= w.vocab) return md_fail(ctx, MD_ERR_INVALID_ARG, "generate: token id %u out of bounds", first[b]);
    }
    md_text_request* r0 = reqs[0];
    MD_TRY(ensure_rows(r0, 8));
    MD_TRY(r0->tokens_out.ensure(ctx, batch * n_steps * sizeof(unsigned int)));
    if (forced) MD_TRY(r0->forced.ensure(ctx, batch * n_steps * sizeof(unsigned int)));
    if (logits_out) MD_TRY(r0->logits_all.ensure(ctx, n_steps * w.vocab * 2));
    MD_TRY(r0->pos_ptrs.ensure(ctx, 8 * sizeof(int*)));
    // device-side state of the loop
    unsigned long long cur[8] = {0};
    int* pos_ptrs[8] = {nullptr};
    for (size_t b = 0; b < batch; ++b) {
        cur[b] = first[b];
        pos_ptrs[b] = reqs[b]->pos_dev;
    }
    MD_CUDA(ctx, cudaMemcpyAsync(r0->cur_token.p, cur, sizeof(cur), cudaMemcpyHostToDevice, ctx->stream));
    MD_CUDA(ctx, cudaMemcpyAsync(r0->pos_ptrs.p, pos_ptrs, sizeof(pos_ptrs), cudaMemcpyHostToDevice, ctx->stream));
    MD_CUDA(ctx, cudaMemsetAsync(r0->step.p, 0, sizeof(int), ctx->stream));
    MD_CUDA(ctx, cudaMemsetAsync(r0->sampled.p, 0, 8 * sizeof(unsigned long long), ctx->stream));
    embed_kernel<<<(unsigned)batch, 256, 0, ctx->stream>>>(H(w.wte), r0->cur_token.as<unsigned long long>(),
                                                           r0->hidden.as<__half>(), (int)w.dim, (int)w.vocab);
    MD_LAUNCH_CHECK(ctx, "embed_kernel");
    if (forced)
        MD_CUDA(ctx, cudaMemcpyAsync(r0->forced.p, forced, batch * n_steps * sizeof(unsigned int), cudaMemcpyHostToDevice,
                                     ctx->stream));
    MD_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // cur / pos_ptrs are stack arrays

    // The graph depends on the requests' buffers and on which optional outputs exist; a single
    // request keeps its graph across calls, a batch captures one per call.
    const bool reuse = batch == 1 && r0->graph && r0->graph_gen == ctx->generation && r0->graph_steps == n_steps &&
                       r0->graph_forced == (forced != nullptr) &&
                       r0->graph_logits == (logits_out != nullptr);
    md_graph* graph = reuse ? r0->graph : nullptr;
    size_t done = 0;
    if (!graph) {
        // first step eagerly (sets up scratch and kernel attributes), then capture
        MD_TRY(enqueue_decode_step(model, reqs, batch, n_steps, forced != nullptr, logits_out != nullptr));
        done = 1;
        if (n_steps > 1) {
            MD_TRY(md_graph_begin(ctx));
            int st = enqueue_decode_step(model, reqs, batch, n_steps, forced != nullptr, logits_out != nullptr);
            md_graph* g = nullptr;
            const int st2 = md_graph_end(ctx, &g);
            if (st != MD_OK) { if (g) md_graph_destroy(ctx, g); return st; }
            if (st2 != MD_OK) return st2;
            graph = g;
            if (batch == 1) {
                if (r0->graph) md_graph_destroy(ctx, r0->graph);
                r0->graph = g;
                r0->graph_gen = ctx->generation;
                r0->graph_steps = n_steps;
                r0->graph_forced = forced != nullptr;
                r0->graph_logits = logits_out != nullptr;
            }
        }
    }
    for (; done < n_steps; ++done) MD_TRY(md_graph_launch(ctx, graph));
    for (size_t b = 0; b < batch; ++b) reqs[b]->pos += n_steps;
    MD_CUDA(ctx, cudaMemcpyAsync(tokens_out, r0->tokens_out.p, batch * n_steps * sizeof(unsigned int),
                                 cudaMemcpyDeviceToHost, ctx->stream));
    if (logits_out)
        MD_CUDA(ctx, cudaMemcpyAsync(logits_out, r0->logits_all.p, n_steps * w.vocab * 2, cudaMemcpyDeviceToHost,
                                     ctx->stream));
    const int st = md_check_flags(ctx);
    if (graph && batch != 1) md_graph_destroy(ctx, graph);
    return st;
}

int md_text_generate(md_text_model* model, md_text_request* req, uint32_t first, size_t n_steps, uint32_t* tokens_out,
                     const uint32_t* forced, uint16_t* logits_out) {
    if (!model || !req) return MD_ERR_INVALID_ARG;
    md_text_request* reqs[1] = {req};
    return generate_impl(model, reqs, 1, &first, n_steps, tokens_out, forced, logits_out);
}

int md_text_generate_batch(md_text_model* model, md_text_request* const* reqs, size_t batch, const uint32_t* first,
                           size_t n_steps, uint32_t* tokens_out) {
    if (!model || !reqs) return MD_ERR_INVALID_ARG;
    return generate_impl(model, reqs, batch, first, n_steps, tokens_out, nullptr, nullptr);
}

int md_text_generate_batch_forced(md_text_model* model, md_text_request* const* reqs, size_t batch, const uint32_t* first,
                                  size_t n_steps, uint32_t* tokens_out, const uint32_t* forced) {
    if (!model || !reqs) return MD_ERR_INVALID_ARG;
    return generate_impl(model, reqs, batch, first, n_steps, tokens_out, forced, nullptr);
}

}  // extern "C"

// ------------------------------------------------------------------------------------ vision

struct md_vision_model {
    md_ctx* ctx;
    md_vision_weights w;
    std::vector<const uint16_t*> ln1_w, ln1_b, wqkv, bqkv, wout, bout, ln2_w, ln2_b, wfc1, bfc1, wfc2, bfc2;
    size_t max_crops = 0, patch_dim = 0, patch_dim_padded = 0;
    DevPtr patch_w_padded, img, patches, x, ln, qkv, att, fc1, cat, pfc1, out;
    md_graph* graph = nullptr;  // the whole encode for (graph_crops, graph_a, graph_b), captured on its second use
    uint64_t graph_gen = 0;     // md_ctx::generation the graph was captured under
    size_t graph_crops = 0, graph_a = 0, graph_b = 0, seen_crops = 0, seen_a = 0, seen_b = 0;
};

extern "C" {

int md_vision_model_create(md_ctx* ctx, const md_vision_weights* w, size_t max_crops, md_vision_model** out) {
    if (!ctx) return MD_ERR_INVALID_ARG;
    if (!w || !out || max_crops == 0) return md_fail(ctx, MD_ERR_INVALID_ARG, "md_vision_model_create: bad argument");
    if (w->dim != w->n_heads * w->head_dim) return md_fail(ctx, MD_ERR_UNSUPPORTED, "vision dim != n_heads * head_dim");
    if (w->img % w->patch || (w->img / w->patch) * (w->img / w->patch) != w->tokens)
        return md_fail(ctx, MD_ERR_INVALID_ARG, "vision: image %zu / patch %zu does not give %zu tokens", w->img, w->patch,
                       w->tokens);
    md_vision_model* m = new md_vision_model();
    m->ctx = ctx;
    m->w = *w;
    m->max_crops = max_crops;
    const size_t L = w->n_layers;
    m->ln1_w = copy_ptrs(w->ln1_w, L); m->ln1_b = copy_ptrs(w->ln1_b, L);
    m->wqkv = copy_ptrs(w->wqkv, L); m->bqkv = copy_ptrs(w->bqkv, L);
    m->wout = copy_ptrs(w->wout, L); m->bout = copy_ptrs(w->bout, L);
    m->ln2_w = copy_ptrs(w->ln2_w, L); m->ln2_b = copy_ptrs(w->ln2_b, L);
    m->wfc1 = copy_ptrs(w->wfc1, L); m->bfc1 = copy_ptrs(w->bfc1, L);
    m->wfc2 = copy_ptrs(w->wfc2, L); m->bfc2 = copy_ptrs(w->bfc2, L);
    m->patch_dim = 3 * w->patch * w->patch;
    // The 588-wide patch vectors have 1176-byte rows, which TMA cannot address: pad K to a multiple of 8
    // (592) with zero columns in the patches and zero rows in a private copy of the embedding weight.
    m->patch_dim_padded = (m->patch_dim + 7) & ~(size_t)7;
    const size_t R = max_crops * w->tokens, D = w->dim;
    int st = m->patch_w_padded.ensure(ctx, m->patch_dim_padded * D * 2);
    if (st == MD_OK) st = m->img.ensure(ctx, max_crops * w->img * w->img * 3);
    if (st == MD_OK) st = m->patches.ensure(ctx, R * m->patch_dim_padded * 2);
    if (st == MD_OK) st = m->x.ensure(ctx, R * D * 2);
    if (st == MD_OK) st = m->ln.ensure(ctx, R * D * 2);
    if (st == MD_OK) st = m->qkv.ensure(ctx, R * 3 * D * 2);
    if (st == MD_OK) st = m->att.ensure(ctx, R * D * 2);
    if (st == MD_OK) st = m->fc1.ensure(ctx, R * w->hidden * 2);
    if (st == MD_OK) st = m->cat.ensure(ctx, w->tokens * 2 * D * 2);
    if (st == MD_OK) st = m->pfc1.ensure(ctx, w->tokens * w->proj_hidden * 2);
    if (st == MD_OK) st = m->out.ensure(ctx, w->tokens * w->proj_out * 2);
    if (st != MD_OK) { delete m; return st; }
    cudaMemsetAsync(m->patch_w_padded.p, 0, m->patch_dim_padded * D * 2, ctx->stream);
    cudaMemcpyAsync(m->patch_w_padded.p, w->patch_w, m->patch_dim * D * 2, cudaMemcpyDeviceToDevice, ctx->stream);
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) {
        delete m;
        return md_fail(ctx, MD_ERR_CUDA, "vision: weight padding copy failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    *out = m;
    return MD_OK;
}

int md_vision_model_destroy(md_vision_model* model) {
    if (model) cudaStreamSynchronize(model->ctx->stream);
    if (model && model->graph) md_graph_destroy(model->ctx, model->graph);
    delete model;
    return MD_OK;
}

}  // extern "C"

// images == false: one image of `crops` crops, projection of concat(features[a], features[b]) -> outs[0].
// images == true : `crops` independent single-crop images in one pass (the GEMMs see crops * tokens rows); image i is
//                  projected from concat(features[i], features[i]) (the reference's two identical crops) -> outs[i].
static int vision_encode_impl(md_vision_model* m, const uint8_t* crops_u8, size_t crops, size_t crop_a, size_t crop_b,
                              bool images, uint16_t* features_out, uint16_t* const* outs) {
    md_ctx* ctx = m->ctx;
    const md_vision_weights& w = m->w;
    if (crops == 0 || crops > m->max_crops || crop_a >= crops || crop_b >= crops)
        return md_fail(ctx, MD_ERR_INVALID_ARG, "vision_encode: crops %zu (max %zu), a %zu, b %zu", crops, m->max_crops, crop_a,
                       crop_b);
    const size_t PR = images ? crops * w.tokens : w.tokens;   // rows of the projection
    if (m->graph && (m->cat.cap < PR * 2 * w.dim * 2 || m->pfc1.cap < PR * w.proj_hidden * 2 || m->out.cap < PR * w.proj_out * 2)) {
        md_graph_destroy(ctx, m->graph);   // the projection's buffers are about to move: the captured encode is stale
        m->graph = nullptr;
    }
    MD_TRY(m->cat.ensure(ctx, PR * 2 * w.dim * 2));
    MD_TRY(m->pfc1.ensure(ctx, PR * w.proj_hidden * 2));
    MD_TRY(m->out.ensure(ctx, PR * w.proj_out * 2));
    const size_t T = w.tokens, D = w.dim, F = w.hidden, R = crops * T;
    const float eps = eps_of(w.eps_f16);
    const cudaMemcpyKind in_kind = md_is_device_ptr(crops_u8) ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    MD_CUDA(ctx, cudaMemcpyAsync(m->img.p, crops_u8, crops * w.img * w.img * 3, in_kind, ctx->stream));
    const uint8_t* img = m->img.as<uint8_t>();
    __half* ln = m->ln.as<__half>();
    auto body = [&]() -> int {
    PdlScope pdl_scope(ctx);
    __half *x = m->x.as<__half>(), *qkv = m->qkv.as<__half>(), *att = m->att.as<__half>(),
           *fc1 = m->fc1.as<__half>();
    MD_TRY(md_launch_patchify(ctx, img, m->patches.as<__half>(), crops, w.img, w.img, w.patch, m->patch_dim_padded));
    // patch embedding + bias, then the position embedding broadcast over the crops (vision_model.zig:220-228)
    md_epilogue e_patch;
    e_patch.bias = H(w.patch_b);
    e_patch.residual = H(w.pos_emb);
    e_patch.residual_rows = (int)T;
    MD_TRY(md_gemm_dispatch(ctx, m->patches.as<__half>(), m->patch_w_padded.as<__half>(), x, R, D, m->patch_dim_padded, 0,
                            e_patch));
    for (size_t l = 0; l < w.n_layers; ++l) {
        MD_TRY(md_launch_layernorm(ctx, x, H(m->ln1_w[l]), H(m->ln1_b[l]), ln, R, D, eps));
        md_epilogue e_qkv;
        e_qkv.bias = H(m->bqkv[l]);
        MD_TRY(md_gemm_dispatch(ctx, ln, H(m->wqkv[l]), qkv, R, 3 * D, D, 0, e_qkv));
        MD_TRY(md_launch_sdpa(ctx, qkv, qkv + D, qkv + 2 * D, nullptr, att, w.n_heads, T, T, w.head_dim, 3 * D, w.head_dim,
                              3 * D, w.head_dim, D, w.head_dim, crops, T * 3 * D, T * 3 * D, T * D, -1));
        md_epilogue e_out;  // x += attn_out (vision_model.zig:239-240)
        e_out.bias = H(m->bout[l]);
        e_out.residual = x;
        MD_TRY(md_gemm_dispatch(ctx, att, H(m->wout[l]), x, R, D, D, 0, e_out));
        MD_TRY(md_launch_layernorm(ctx, x, H(m->ln2_w[l]), H(m->ln2_b[l]), ln, R, D, eps));
        md_epilogue e_fc1;
        e_fc1.bias = H(m->bfc1[l]);
        e_fc1.gelu = 1;
        MD_TRY(md_gemm_dispatch(ctx, ln, H(m->wfc1[l]), fc1, R, F, D, 0, e_fc1));
        md_epilogue e_fc2;  // x += mlp_out (vision_model.zig:261-262)
        e_fc2.bias = H(m->bfc2[l]);
        e_fc2.residual = x;
        MD_TRY(md_gemm_dispatch(ctx, fc1, H(m->wfc2[l]), x, R, D, F, 0, e_fc2));
    }
    MD_TRY(md_launch_layernorm(ctx, x, H(w.norm_w), H(w.norm_b), ln, R, D, eps));  // features, in ln
        return MD_OK;
    };
    auto proj = [&]() -> int {
        // concat(features[a], features[b]) on the feature dim (vision_model.zig:189-195); for independent images
        // every image's rows are paired with themselves
        __half* cat = m->cat.as<__half>();
        const size_t ra = images ? 0 : crop_a * T, rb = images ? 0 : crop_b * T;
        MD_CUDA(ctx, cudaMemcpy2DAsync(cat, 2 * D * 2, ln + ra * D, D * 2, D * 2, PR, cudaMemcpyDeviceToDevice, ctx->stream));
        MD_CUDA(ctx, cudaMemcpy2DAsync(cat + D, 2 * D * 2, ln + rb * D, D * 2, D * 2, PR, cudaMemcpyDeviceToDevice,
                                       ctx->stream));
        md_epilogue e_p1;
        e_p1.bias = H(w.proj_fc1_b);
        e_p1.gelu = 1;
        MD_TRY(md_gemm_dispatch(ctx, cat, H(w.proj_fc1_w), m->pfc1.as<__half>(), PR, w.proj_hidden, 2 * D, 0, e_p1));
        md_epilogue e_p2;
        e_p2.bias = H(w.proj_fc2_b);
        MD_TRY(md_gemm_dispatch(ctx, m->pfc1.as<__half>(), H(w.proj_fc2_w), m->out.as<__half>(), PR, w.proj_out,
                                w.proj_hidden, 0, e_p2));
        return MD_OK;
    };
    if (images) crop_a = crop_b = ~(size_t)0;   // the graph key of the independent-images form
    if (m->graph && m->graph_gen == ctx->generation && m->graph_crops == crops && m->graph_a == crop_a &&
        m->graph_b == crop_b) {
        MD_TRY(md_graph_launch(ctx, m->graph));
    } else {
        MD_TRY(body());
        MD_TRY(proj());
        if (!ctx->capturing && m->seen_crops == crops && m->seen_a == crop_a && m->seen_b == crop_b) {
            if (m->graph) { md_graph_destroy(ctx, m->graph); m->graph = nullptr; }
            MD_TRY(md_graph_begin(ctx));
            int st = body();
            if (st == MD_OK) st = proj();
            md_graph* g = nullptr;
            const int st2 = md_graph_end(ctx, &g);
            if (st == MD_OK && st2 == MD_OK) {
                m->graph = g;
                m->graph_gen = ctx->generation;
                m->graph_crops = crops; m->graph_a = crop_a; m->graph_b = crop_b;
            } else if (g) {
                md_graph_destroy(ctx, g);
            }
        }
        m->seen_crops = crops; m->seen_a = crop_a; m->seen_b = crop_b;
    }
    MD_TRY(copy_out(ctx, features_out, ln, R * D * 2));
    for (size_t i = 0; i < (images ? crops : 1); ++i)
        MD_TRY(copy_out(ctx, outs[i], m->out.as<__half>() + i * T * w.proj_out, T * w.proj_out * 2));
    return md_check_flags(ctx);
}

extern "C" {

int md_vision_encode(md_vision_model* m, const uint8_t* crops_u8, size_t crops, size_t crop_a, size_t crop_b,
                     uint16_t* features_out, uint16_t* out) {
    if (!m) return MD_ERR_INVALID_ARG;
    if (!crops_u8 || !out) return md_fail(m->ctx, MD_ERR_INVALID_ARG, "vision_encode: null pointer");
    uint16_t* outs[1] = {out};
    return vision_encode_impl(m, crops_u8, crops, crop_a, crop_b, false, features_out, outs);
}

int md_vision_encode_images(md_vision_model* m, const uint8_t* images_u8, size_t n_images, uint16_t* const* outs) {
    if (!m) return MD_ERR_INVALID_ARG;
    if (!images_u8 || !outs) return md_fail(m->ctx, MD_ERR_INVALID_ARG, "vision_encode_images: null pointer");
    for (size_t i = 0; i < n_images; ++i)
        if (!outs[i]) return md_fail(m->ctx, MD_ERR_INVALID_ARG, "vision_encode_images: null output %zu", i);
    return vision_encode_impl(m, images_u8, n_images, 0, 0, true, nullptr, outs);
}

}  // extern "C"
