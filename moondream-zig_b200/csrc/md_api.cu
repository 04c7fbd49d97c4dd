// C ABI of libmoondream_b200: context, memory, host-or-device argument staging and the
// entry points declared in include/moondream_b200.h.  Host code only; kernels live in the
// other translation units.
#include "md_internal.cuh"

#include <cmath>
#include <cstring>

static thread_local std::string g_init_error;

int md_fail(md_ctx* ctx, int status, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (ctx) ctx->last_error = buf;
    else g_init_error = buf;
    return status;
}

bool md_is_device_ptr(const void* p) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

static int stage_reserve(md_ctx* ctx, int slot, size_t bytes, void** out) {
    if ((size_t)slot >= ctx->stage.size()) ctx->stage.resize(slot + 1);
    auto& s = ctx->stage[slot];
    if (s.cap < bytes) {
        if (s.ptr) {
            MD_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            MD_CUDA(ctx, cudaFree(s.ptr));
            s.ptr = nullptr;
            s.cap = 0;
        }
        size_t cap = bytes + bytes / 4;
        cap = (cap + 255) & ~(size_t)255;
        MD_CUDA(ctx, cudaMalloc(&s.ptr, cap));
        s.cap = cap;
    }
    *out = s.ptr;
    return MD_OK;
}

// Copies a small operand out of pinned, mapped host memory (the SMs read it over the bus).
__global__ void stage_in_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n16) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n16) dst[i] = src[i];
}

int md_stage_in(md_ctx* ctx, int slot, const void* user, size_t bytes, md_arg* out) {
    out->user = user;
    out->bytes = bytes;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, user) != cudaSuccess) {
        cudaGetLastError();
        attr.type = cudaMemoryTypeUnregistered;
        attr.devicePointer = nullptr;
    }
    if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) {
        out->dev = const_cast<void*>(user);
        out->staged = false;
        return MD_OK;
    }
    if (ctx->capturing)
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "host pointers cannot be used while a graph is being captured");
    MD_TRY(stage_reserve(ctx, slot, bytes ? bytes : 1, &out->dev));
    out->staged = true;
    if (!bytes) return MD_OK;
    // A small operand in pinned, mapped memory (the activations of a GEMV) is fetched by a kernel instead of the copy
    // engine: the call then queues two kernels on one engine, without the copy's start-up and the hand-over between
    // the engines, which together cost more than the GEMV itself.
    if (bytes <= ((size_t)64 << 10) && (bytes % 16) == 0 && attr.type == cudaMemoryTypeHost && attr.devicePointer &&
        (reinterpret_cast<uintptr_t>(attr.devicePointer) % 16) == 0) {
        const size_t n16 = bytes / 16;
        stage_in_kernel<<<(unsigned)((n16 + 255) / 256), 256, 0, ctx->stream>>>(
            reinterpret_cast<const uint4*>(attr.devicePointer), reinterpret_cast<uint4*>(out->dev), n16);
        MD_LAUNCH_CHECK(ctx, "stage_in_kernel");
        return MD_OK;
    }
    MD_CUDA(ctx, cudaMemcpyAsync(out->dev, user, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return MD_OK;
}

// Output that plain stores of a kernel may write in place when the caller's buffer is pinned, mapped host memory
// and small (the GEMV results): no staging buffer and no device-to-host copy, the call ends with the stream
// synchronize alone.  Anything else goes through md_stage_out.
int md_stage_out_mapped(md_ctx* ctx, int slot, void* user, size_t bytes, md_arg* out) {
    cudaPointerAttributes attr;
    if (bytes > 0 && bytes <= ((size_t)1 << 20) && !ctx->capturing &&
        cudaPointerGetAttributes(&attr, user) == cudaSuccess && attr.type == cudaMemoryTypeHost && attr.devicePointer) {
        out->user = user;
        out->bytes = bytes;
        out->dev = attr.devicePointer;
        out->staged = false;
        out->mapped = true;
        return MD_OK;
    }
    cudaGetLastError();
    return md_stage_out(ctx, slot, user, bytes, out);
}

int md_stage_out(md_ctx* ctx, int slot, void* user, size_t bytes, md_arg* out) {
    out->user = user;
    out->bytes = bytes;
    if (md_is_device_ptr(user)) {
        out->dev = user;
        out->staged = false;
        return MD_OK;
    }
    if (ctx->capturing)
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "host pointers cannot be used while a graph is being captured");
    MD_TRY(stage_reserve(ctx, slot, bytes ? bytes : 1, &out->dev));
    out->staged = true;
    return MD_OK;
}

static int reset_flags(md_ctx* ctx) {
    md_devflags init;
    init.error = 0;
    init.where = 0;
    init.mirror = nullptr;
    *ctx->mirror_host = 0;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&init.mirror), ctx->mirror_host, 0) != cudaSuccess) {
        cudaGetLastError();
        init.mirror = nullptr;
    }
    MD_CUDA(ctx, cudaMemcpy(ctx->flags, &init, sizeof(init), cudaMemcpyHostToDevice));
    // a kernel that gave up may have left arrival counts behind (split-KV decode attention, split-K GEMM): the next
    // launch must find them at zero
    if (ctx->counters) MD_CUDA(ctx, cudaMemset(ctx->counters, 0, MD_COUNTER_WORDS * 4));
    for (auto& w : ctx->splitk)
        if (w.tickets) MD_CUDA(ctx, cudaMemset(w.tickets, 0, MD_SPLITK_TICKETS * sizeof(unsigned)));
    return MD_OK;
}

// Synchronises the stream and reports a device-side wait that gave up.  The common case costs no copy: the
// kernels raise a word in mapped host memory together with the device flag.
int md_check_flags(md_ctx* ctx) {
    MD_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (*reinterpret_cast<volatile unsigned int*>(ctx->mirror_host) == 0u) return MD_OK;
    MD_CUDA(ctx, cudaMemcpy(ctx->flags_host, ctx->flags, sizeof(md_devflags), cudaMemcpyDeviceToHost));
    const unsigned where = ctx->flags_host->where;
    MD_TRY(reset_flags(ctx));
    return md_fail(ctx, MD_ERR_TIMEOUT, "a device-side wait gave up (site %u); results are invalid", where);
}

int md_finish_out(md_ctx* ctx, md_arg* out) {
    if (out->mapped) return md_check_flags(ctx);  // the kernel wrote the caller's buffer: wait for it
    if (!out->staged) return MD_OK;
    if (out->bytes)
        MD_CUDA(ctx, cudaMemcpyAsync(const_cast<void*>(out->user), out->dev, out->bytes, cudaMemcpyDeviceToHost,
                                     ctx->stream));
    return md_check_flags(ctx);
}

int md_scratch(md_ctx* ctx, size_t bytes, void** out) {
    if (ctx->scratch_cap < bytes) {
        if (ctx->capturing)
            return md_fail(ctx, MD_ERR_UNSUPPORTED,
                           "scratch memory would have to grow during graph capture; run the call once before capturing");
        if (ctx->scratch) {
            MD_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            MD_CUDA(ctx, cudaFree(ctx->scratch));
            ctx->scratch = nullptr;
            ctx->scratch_cap = 0;
        }
        size_t cap = bytes < (1u << 20) ? (1u << 20) : bytes + bytes / 2;
        cap = (cap + 255) & ~(size_t)255;
        MD_CUDA(ctx, cudaMalloc(&ctx->scratch, cap));
        ctx->scratch_cap = cap;
        ctx->generation++;  // graphs that hold the old address are stale
    }
    *out = ctx->scratch;
    return MD_OK;
}

// Partial tiles and tickets of a split-K GEMM for the stream the context is on.
int md_splitk_workspace(md_ctx* ctx, size_t bytes, float** part, unsigned** tickets) {
    md_ctx::SplitK* ws = nullptr;
    for (auto& w : ctx->splitk)
        if (w.stream == ctx->stream) ws = &w;
    if (!ws || ws->cap < bytes) {
        if (ctx->capturing)
            return md_fail(ctx, MD_ERR_UNSUPPORTED,
                           "split-K workspace would have to grow during graph capture; run the call once before capturing");
        if (!ws) {
            ctx->splitk.emplace_back();
            ws = &ctx->splitk.back();
            ws->stream = ctx->stream;
            MD_CUDA(ctx, cudaMalloc((void**)&ws->tickets, MD_SPLITK_TICKETS * sizeof(unsigned)));
            MD_CUDA(ctx, cudaMemset(ws->tickets, 0, MD_SPLITK_TICKETS * sizeof(unsigned)));
        }
        if (ws->part) {
            MD_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            MD_CUDA(ctx, cudaFree(ws->part));
            ws->part = nullptr;
            ws->cap = 0;
        }
        const size_t cap = (bytes + bytes / 4 + 255) & ~(size_t)255;
        MD_CUDA(ctx, cudaMalloc((void**)&ws->part, cap));
        ws->cap = cap;
        ctx->generation++;  // graphs that hold the old address are stale
    }
    *part = ws->part;
    *tickets = ws->tickets;
    return MD_OK;
}

int md_rope_cached(md_ctx* ctx, size_t rot_dim, float theta, size_t rows, const float** out) {
    if (!ctx->rope_tab || ctx->rope_dim != rot_dim || ctx->rope_theta != theta || ctx->rope_rows < rows) {
        if (ctx->capturing)
            return md_fail(ctx, MD_ERR_UNSUPPORTED, "the rope table must exist before graph capture; run the call once first");
        if (rot_dim == 0 || (rot_dim & 1)) return md_fail(ctx, MD_ERR_INVALID_ROT_DIM, "rope: rot_dim %zu", rot_dim);
        if (ctx->rope_tab) {
            MD_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            MD_CUDA(ctx, cudaFree(ctx->rope_tab));
            ctx->rope_tab = nullptr;
        }
        MD_CUDA(ctx, cudaMalloc((void**)&ctx->rope_tab, rows * rot_dim * sizeof(float)));
        ctx->rope_rows = rows;
        ctx->rope_dim = rot_dim;
        ctx->rope_theta = theta;
        ctx->generation++;  // graphs that hold the old table are stale
        MD_TRY(md_launch_rope_table(ctx, ctx->rope_tab, rot_dim, rows, theta));
    }
    *out = ctx->rope_tab;
    return MD_OK;
}

#define MD_NEED_CTX(ctx) \
    do { if (!(ctx)) return MD_ERR_INVALID_ARG; } while (0)
#define MD_NEED(ctx, cond, what) \
    do { if (!(cond)) return md_fail((ctx), MD_ERR_INVALID_ARG, "%s", what); } while (0)

extern "C" {

int md_init(md_ctx** out, int device) {
    if (!out) return MD_ERR_INVALID_ARG;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return md_fail(nullptr, MD_ERR_NO_DEVICE, "no CUDA device: %s (this library has no CPU fallback)",
                       e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
    }
    if (device < 0 || device >= count)
        return md_fail(nullptr, MD_ERR_NO_DEVICE, "device %d out of range (%d devices)", device, count);
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess)
        return md_fail(nullptr, MD_ERR_CUDA, "cudaGetDeviceProperties failed");
    if (prop.major != 10)
        return md_fail(nullptr, MD_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                       prop.major, prop.minor);
    md_ctx* ctx = new md_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    auto bail = [&](const char* what) {
        std::string msg = std::string(what) + ": " + cudaGetErrorString(cudaGetLastError());
        delete ctx;
        return md_fail(nullptr, MD_ERR_CUDA, "%s", msg.c_str());
    };
    if (cudaSetDevice(device) != cudaSuccess) return bail("cudaSetDevice");
    if (cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking) != cudaSuccess) return bail("stream");
    ctx->stream = ctx->own_stream;
    if (cudaMalloc(&ctx->flags, sizeof(md_devflags)) != cudaSuccess) return bail("cudaMalloc flags");
    if (cudaMallocHost(&ctx->flags_host, sizeof(md_devflags)) != cudaSuccess) return bail("cudaMallocHost");
    if (cudaHostAlloc(reinterpret_cast<void**>(&ctx->mirror_host), sizeof(unsigned int), cudaHostAllocMapped) != cudaSuccess)
        return bail("cudaHostAlloc mirror");
    if (reset_flags(ctx) != MD_OK) return bail("flag initialisation");
    if (cudaMalloc(&ctx->counters, MD_COUNTER_WORDS * 4) != cudaSuccess) return bail("cudaMalloc counters");
    if (cudaMemset(ctx->counters, 0, MD_COUNTER_WORDS * 4) != cudaSuccess) return bail("cudaMemset counters");
    ctx->scratch_cap = (size_t)16 << 20;
    if (cudaMalloc(&ctx->scratch, ctx->scratch_cap) != cudaSuccess) return bail("cudaMalloc scratch");
    *out = ctx;
    return MD_OK;
}

int md_destroy(md_ctx* ctx) {
    MD_NEED_CTX(ctx);
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto& s : ctx->stage)
        if (s.ptr) cudaFree(s.ptr);
    if (ctx->scratch) cudaFree(ctx->scratch);
    for (auto& w : ctx->splitk) {
        if (w.part) cudaFree(w.part);
        if (w.tickets) cudaFree(w.tickets);
    }
    if (ctx->counters) cudaFree(ctx->counters);
    if (ctx->rope_tab) cudaFree(ctx->rope_tab);
    if (ctx->flags) cudaFree(ctx->flags);
    if (ctx->flags_host) cudaFreeHost(ctx->flags_host);
    if (ctx->mirror_host) cudaFreeHost(ctx->mirror_host);
    if (ctx->side_stream) cudaStreamDestroy(ctx->side_stream);
    for (auto st : ctx->mlp_stream)
        if (st) cudaStreamDestroy(st);
    for (auto ev : ctx->ev_mlp)
        if (ev) cudaEventDestroy(ev);
    if (ctx->ev_fork) cudaEventDestroy(ctx->ev_fork);
    if (ctx->ev_side) cudaEventDestroy(ctx->ev_side);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    delete ctx;
    return MD_OK;
}

const char* md_last_error(const md_ctx* ctx) { return ctx ? ctx->last_error.c_str() : g_init_error.c_str(); }

int md_sync(md_ctx* ctx) {
    MD_NEED_CTX(ctx);
    return md_check_flags(ctx);
}

int md_selftest_bounded_wait(md_ctx* ctx, unsigned limit_ms) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, limit_ms >= 1 && limit_ms <= 2000, "md_selftest_bounded_wait: limit_ms must be 1..2000");
    MD_NEED(ctx, !ctx->capturing, "md_selftest_bounded_wait: not while a graph is being captured");
    return md_launch_selftest_wait(ctx, limit_ms);
}

int md_set_stream(md_ctx* ctx, void* cuda_stream) {
    MD_NEED_CTX(ctx);
    ctx->stream = cuda_stream ? reinterpret_cast<cudaStream_t>(cuda_stream) : ctx->own_stream;
    return MD_OK;
}

int md_alloc(md_ctx* ctx, size_t bytes, void** dev_out) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, dev_out, "md_alloc: null output");
    MD_CUDA(ctx, cudaMalloc(dev_out, bytes ? bytes : 1));
    return MD_OK;
}

int md_free(md_ctx* ctx, void* dev) {
    MD_NEED_CTX(ctx);
    if (dev) MD_CUDA(ctx, cudaFree(dev));
    return MD_OK;
}

int md_upload(md_ctx* ctx, const void* host, size_t bytes, void** dev_out) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, host && dev_out, "md_upload: null pointer");
    MD_TRY(md_alloc(ctx, bytes, dev_out));
    MD_CUDA(ctx, cudaMemcpyAsync(*dev_out, host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    MD_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return MD_OK;
}

int md_memcpy_h2d(md_ctx* ctx, void* dev, const void* host, size_t bytes) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, dev && host, "md_memcpy_h2d: null pointer");
    MD_CUDA(ctx, cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    MD_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return MD_OK;
}

int md_memcpy_d2h(md_ctx* ctx, void* host, const void* dev, size_t bytes) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, dev && host, "md_memcpy_d2h: null pointer");
    MD_CUDA(ctx, cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    MD_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return MD_OK;
}

int md_launch_count(const md_ctx* ctx, uint64_t* count_out) {
    if (!ctx || !count_out) return MD_ERR_INVALID_ARG;
    *count_out = ctx->launches;
    return MD_OK;
}

int md_set_option(md_ctx* ctx, const char* key, long value) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, key, "md_set_option: null key");
    ctx->generation++;  // options select kernels: graphs captured under the old settings are captured again
    if (!strcmp(key, "gemv_variant")) { ctx->gemv_variant = (int)value; return MD_OK; }
    if (!strcmp(key, "gemv_ksplit")) {
        MD_NEED(ctx, value == 0 || value == 1 || value == 2 || value == 4 || value == 8, "gemv_ksplit must be 0, 1, 2, 4 or 8");
        ctx->gemv_ksplit = (int)value;
        return MD_OK;
    }
    if (!strcmp(key, "decode_cluster")) {
        ctx->decode_cluster_mode = value < 0 ? -1 : (value ? 1 : 0);
        ctx->decode_cluster_ok = -1;
        return MD_OK;
    }
    if (!strcmp(key, "dualk_variant")) { ctx->dualk_variant = (int)value; return MD_OK; }
    if (!strcmp(key, "decode_split_ln")) { ctx->decode_split_ln = (int)value; return MD_OK; }
    if (!strcmp(key, "fused_decode")) { ctx->fused_decode = value ? 1 : 0; return MD_OK; }
    if (!strcmp(key, "pdl")) { ctx->pdl = value ? 1 : 0; return MD_OK; }
    if (!strcmp(key, "prefill_fork")) { ctx->prefill_fork = value ? 1 : 0; return MD_OK; }
    if (!strcmp(key, "decode_fork")) { ctx->decode_fork = value ? 1 : 0; return MD_OK; }
    if (!strcmp(key, "push_tma")) { ctx->push_tma = value ? 1 : 0; return MD_OK; }
    if (!strcmp(key, "tc_splitk")) {
        if (value < -1 || value == 1 || value > 8) return md_fail(ctx, MD_ERR_INVALID_ARG, "tc_splitk must be -1, 0 or 2..8");
        ctx->tc_splitk = (int)value;
        return MD_OK;
    }
    if (!strcmp(key, "attn_ctas_per_sm")) {
        if (value < 0 || value > 2) return md_fail(ctx, MD_ERR_INVALID_ARG, "attn_ctas_per_sm must be 0, 1 or 2");
        ctx->attn_ctas_per_sm = (int)value;
        return MD_OK;
    }
    if (!strcmp(key, "decode_loop")) { ctx->decode_loop = (int)value; return MD_OK; }
    if (!strcmp(key, "decode_mlp_split")) {
        MD_NEED(ctx, value == 0 || value == 2 || value == 4, "decode_mlp_split must be 0, 2 or 4");
        ctx->decode_mlp_split = (int)value;
        return MD_OK;
    }
    if (!strcmp(key, "skinny")) { ctx->skinny = value ? 1 : 0; return MD_OK; }
    if (!strcmp(key, "skinny_splits")) {
        MD_NEED(ctx, value >= 0 && value <= 16, "skinny_splits must be 0 (automatic) or 1..16 (rounded down to 1, 2, 4 or 8)");
        ctx->skinny_splits = (int)value;
        return MD_OK;
    }
    if (!strcmp(key, "attn_tc")) { ctx->attn_tc = value < 0 ? -1 : value ? 1 : 0; return MD_OK; }
    if (!strcmp(key, "tc_pair")) { ctx->tc_pair = value < 0 ? -1 : (value ? 1 : 0); return MD_OK; }
    if (!strcmp(key, "tc_block_n")) {
        MD_NEED(ctx, value == 0 || value == 64 || value == 128 || value == 256 || value == 512,
                "tc_block_n must be 0, 64, 128, 256 or 512 (512 = the 256 x 256 tile)");
        ctx->tc_block_n = (int)value;
        return MD_OK;
    }
    return md_fail(ctx, MD_ERR_INVALID_ARG, "md_set_option: unknown key '%s'", key);
}

int md_get_option(md_ctx* ctx, const char* key, long* value_out) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, key && value_out, "md_get_option: null argument");
    if (!strcmp(key, "last_tc_tile")) { *value_out = ctx->last_tc_tile; return MD_OK; }
    if (!strcmp(key, "gemv_variant")) { *value_out = ctx->gemv_variant; return MD_OK; }
    if (!strcmp(key, "tc_block_n")) { *value_out = ctx->tc_block_n; return MD_OK; }
    if (!strcmp(key, "pdl")) { *value_out = ctx->pdl; return MD_OK; }
    if (!strcmp(key, "push_tma")) { *value_out = ctx->push_tma; return MD_OK; }
    return md_fail(ctx, MD_ERR_INVALID_ARG, "md_get_option: unknown key '%s'", key);
}

int md_graph_begin(md_ctx* ctx) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, !ctx->capturing, "md_graph_begin: a capture is already in progress");
    MD_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
    ctx->capturing = true;
    return MD_OK;
}

int md_graph_end(md_ctx* ctx, md_graph** out) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, out, "md_graph_end: null output");
    MD_NEED(ctx, ctx->capturing, "md_graph_end: no capture in progress");
    ctx->capturing = false;
    md_graph* g = new md_graph();
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &g->graph);
    if (e == cudaSuccess) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
    if (e != cudaSuccess) {
        if (g->graph) cudaGraphDestroy(g->graph);
        delete g;
        return md_fail(ctx, MD_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
    }
    *out = g;
    return MD_OK;
}

int md_graph_launch(md_ctx* ctx, md_graph* graph) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, graph && graph->exec, "md_graph_launch: null graph");
    MD_CUDA(ctx, cudaGraphLaunch(graph->exec, ctx->stream));
    return MD_OK;
}

int md_graph_destroy(md_ctx* ctx, md_graph* graph) {
    MD_NEED_CTX(ctx);
    if (graph) {
        if (graph->exec) cudaGraphExecDestroy(graph->exec);
        if (graph->graph) cudaGraphDestroy(graph->graph);
        delete graph;
    }
    return MD_OK;
}

int md_set_gemm_mode(md_ctx* ctx, int mode) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, mode >= 0 && mode <= 2, "md_set_gemm_mode: mode must be 0, 1 or 2");
    ctx->gemm_mode = mode;
    ctx->generation++;
    return MD_OK;
}

int md_check_matmul_shapes(const size_t* a_shape, size_t a_rank, const size_t* b_shape, size_t b_rank,
                           int b_transposed) {
    if (!a_shape || !b_shape) return MD_ERR_INVALID_ARG;
    if (a_rank != 2 || b_rank != 2) return MD_ERR_INVALID_DIMENSION;
    const size_t k_b = b_transposed ? b_shape[1] : b_shape[0];
    if (k_b != a_shape[1]) return MD_ERR_SHAPE;
    return MD_OK;
}

// device-pointer GEMM dispatch shared by every matmul entry point
int md_gemm_dispatch(md_ctx* ctx, const __half* a, const __half* b, __half* c, size_t M, size_t N, size_t K,
                         int b_layout, const md_epilogue& ep) {
    if (M == 0 || N == 0) return MD_OK;
    if (K == 0) {
        // empty inner dimension: the product is all zeros (then the fused glue)
        MD_CUDA(ctx, cudaMemsetAsync(c, 0, M * N * sizeof(__half), ctx->stream));
        if (ep.bias) MD_TRY(md_launch_bias_add(ctx, c, ep.bias, M, N));
        if (ep.gelu) MD_TRY(md_launch_gelu(ctx, c, M * N));
        if (ep.residual && ep.residual_rows == 0) MD_TRY(md_launch_add(ctx, c, ep.residual, M * N));
        if (ep.residual2) MD_TRY(md_launch_add(ctx, c, ep.residual2, M * N));
        return MD_OK;
    }
    const bool aligned16 = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0;
    if (ctx->gemm_mode != 1 && b_layout == 1 && M <= 8 && (K % 8) == 0 && aligned16 && ctx->gemm_mode != 2)
        return md_launch_gemv_nt(ctx, a, b, c, M, N, K, ep);
    if (ctx->gemm_mode == 0 && ctx->skinny && md_gemm_skinny_supported(a, b, c, M, N, K))
        return md_launch_gemm_skinny(ctx, a, b, c, M, N, K, b_layout, ep);
    const bool tc_ok = md_gemm_tc_supported(a, b, c, M, N, K, b_layout);
    if (ctx->gemm_mode == 2 && !tc_ok)
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "tcgen05 GEMM forced but the shape/alignment does not allow it");
    if (ctx->gemm_mode != 1 && tc_ok) return md_launch_gemm_tc(ctx, a, b, c, M, N, K, b_layout, ep);
    return md_launch_gemm_simt(ctx, a, b, c, M, N, K, b_layout, ep);
}

static int hgemm_entry(md_ctx* ctx, const uint16_t* a, const uint16_t* b, uint16_t* c, size_t M, size_t N, size_t K,
                       int b_layout) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, a && b && c, "hgemm: null tensor pointer");
    MD_CUDA(ctx, cudaSetDevice(ctx->device));
    md_arg A, B, Cc;
    MD_TRY(md_stage_in(ctx, 0, a, M * K * 2, &A));
    MD_TRY(md_stage_in(ctx, 1, b, N * K * 2, &B));
    // the GEMV kernel (same conditions as in md_gemm_dispatch) writes with plain stores, which may target
    // mapped host memory; the TMA-store epilogue of the tcgen05 GEMM always gets device memory
    const bool gemv = ctx->gemm_mode == 0 && b_layout == 1 && M >= 1 && M <= 8 && K > 0 && (K % 8) == 0 &&
                      ((reinterpret_cast<uintptr_t>(A.dev) | reinterpret_cast<uintptr_t>(B.dev)) & 15) == 0;
    if (gemv) MD_TRY(md_stage_out_mapped(ctx, 2, c, M * N * 2, &Cc));
    else MD_TRY(md_stage_out(ctx, 2, c, M * N * 2, &Cc));
    md_epilogue ep;
    MD_TRY(md_gemm_dispatch(ctx, (const __half*)A.dev, (const __half*)B.dev, (__half*)Cc.dev, M, N, K, b_layout, ep));
    return md_finish_out(ctx, &Cc);
}

int md_hgemm_nn(md_ctx* ctx, const uint16_t* a, const uint16_t* b, uint16_t* c, size_t M, size_t N, size_t K) {
    return hgemm_entry(ctx, a, b, c, M, N, K, 0);
}

int md_hgemm_nt(md_ctx* ctx, const uint16_t* a, const uint16_t* b_t, uint16_t* c, size_t M, size_t N, size_t K) {
    return hgemm_entry(ctx, a, b_t, c, M, N, K, 1);
}

int md_hgemm_fused(md_ctx* ctx, const uint16_t* a, const uint16_t* b, uint16_t* c, size_t M, size_t N, size_t K,
                   int b_layout, const uint16_t* bias, int gelu, const uint16_t* residual) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, a && b && c, "hgemm_fused: null tensor pointer");
    MD_NEED(ctx, b_layout == 0 || b_layout == 1, "hgemm_fused: b_layout must be 0 or 1");
    md_epilogue ep;
    ep.bias = (const __half*)bias;
    ep.residual = (const __half*)residual;
    ep.gelu = gelu;
    return md_gemm_dispatch(ctx, (const __half*)a, (const __half*)b, (__half*)c, M, N, K, b_layout, ep);
}

int md_hgemm_colsplit_push(md_ctx* ctx, const uint16_t* a, const uint16_t* b_slice, uint16_t* c_full, size_t M,
                           size_t N_local, size_t K, int b_layout, size_t N_total, size_t col_offset, size_t n_peers,
                           uint16_t* const* peer_c_full) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, a && b_slice && c_full, "colsplit_push: null tensor pointer");
    MD_NEED(ctx, b_layout == 0 || b_layout == 1, "colsplit_push: b_layout must be 0 or 1");
    MD_NEED(ctx, n_peers <= 7 && (n_peers == 0 || peer_c_full), "colsplit_push: at most 7 peers");
    if (col_offset + N_local > N_total) return md_fail(ctx, MD_ERR_SHAPE, "colsplit_push: column block outside C");
    if ((col_offset % 8) != 0 || (N_total % 8) != 0)
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "colsplit_push: column offset and N_total must be multiples of 8");
    md_push push;
    push.n = (int)n_peers;
    push.ld = (long long)N_total;
    for (size_t i = 0; i < n_peers; ++i) {
        MD_NEED(ctx, peer_c_full[i], "colsplit_push: null peer pointer");
        push.base[i] = reinterpret_cast<__half*>(peer_c_full[i]) + col_offset;
    }
    push.self = reinterpret_cast<const __half*>(c_full) + col_offset;
    push.tma = ctx->push_tma ? 1 : 0;
    md_epilogue ep;
    return md_launch_gemm_tc_ex(ctx, (const __half*)a, (const __half*)b_slice, (__half*)c_full + col_offset, M, N_local, K,
                                b_layout, ep, N_total, push);
}

int md_gather_colblocks(md_ctx* ctx, const uint16_t* gathered, uint16_t* c, size_t world, size_t M, size_t N_local) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, gathered && c, "gather_colblocks: null pointer");
    if (!world || !M || !N_local) return MD_OK;
    if ((N_local % 8) == 0 && ((reinterpret_cast<uintptr_t>(gathered) | reinterpret_cast<uintptr_t>(c)) & 15) == 0)
        return md_launch_gather_colblocks(ctx, gathered, c, world, M, N_local);  // one kernel, 16 bytes per thread
    // block g is a contiguous [M, N_local] matrix: one strided 2-D copy per block
    for (size_t g = 0; g < world; ++g)
        MD_CUDA(ctx, cudaMemcpy2DAsync(c + g * N_local, world * N_local * 2, gathered + g * M * N_local, N_local * 2,
                                       N_local * 2, M, cudaMemcpyDeviceToDevice, ctx->stream));
    return MD_OK;
}

int md_sdpa_maskless(md_ctx* ctx, const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* out,
                     size_t n_heads, size_t q_len, size_t kv_len, size_t d) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, q && k && v && out, "sdpa_maskless: null tensor pointer");
    MD_NEED(ctx, n_heads && q_len && kv_len && d, "sdpa_maskless: zero-sized dimension");
    md_arg Q, Kk, V, O;
    MD_TRY(md_stage_in(ctx, 0, q, n_heads * q_len * d * 2, &Q));
    MD_TRY(md_stage_in(ctx, 1, k, n_heads * kv_len * d * 2, &Kk));
    MD_TRY(md_stage_in(ctx, 2, v, n_heads * kv_len * d * 2, &V));
    MD_TRY(md_stage_out(ctx, 3, out, n_heads * q_len * d * 2, &O));
    MD_TRY(md_launch_sdpa(ctx, (const __half*)Q.dev, (const __half*)Kk.dev, (const __half*)V.dev, nullptr,
                          (__half*)O.dev, n_heads, q_len, kv_len, d, d, q_len * d, d, kv_len * d, d, q_len * d, 1, 0, 0,
                          0, -1));
    return md_finish_out(ctx, &O);
}

int md_create_attention_mask(md_ctx* ctx, uint8_t* mask, size_t pos, size_t seq_len) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, mask, "create_attention_mask: null pointer");
    md_arg Mk;
    MD_TRY(md_stage_out(ctx, 0, mask, seq_len * (pos + seq_len), &Mk));
    MD_TRY(md_launch_mask(ctx, (uint8_t*)Mk.dev, pos, seq_len));
    return md_finish_out(ctx, &Mk);
}

int md_sdpa_masked(md_ctx* ctx, const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint8_t* mask,
                   uint16_t* out, size_t n_heads, size_t q_len, size_t kv_len, size_t d) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, q && k && v && mask && out, "sdpa_masked: null tensor pointer");
    MD_NEED(ctx, n_heads && q_len && kv_len && d, "sdpa_masked: zero-sized dimension");
    md_arg Q, Kk, V, Mk, O;
    MD_TRY(md_stage_in(ctx, 0, q, n_heads * q_len * d * 2, &Q));
    MD_TRY(md_stage_in(ctx, 1, k, n_heads * kv_len * d * 2, &Kk));
    MD_TRY(md_stage_in(ctx, 2, v, n_heads * kv_len * d * 2, &V));
    MD_TRY(md_stage_in(ctx, 3, mask, q_len * kv_len, &Mk));
    MD_TRY(md_stage_out(ctx, 4, out, n_heads * q_len * d * 2, &O));
    MD_TRY(md_launch_sdpa(ctx, (const __half*)Q.dev, (const __half*)Kk.dev, (const __half*)V.dev,
                          (const uint8_t*)Mk.dev, (__half*)O.dev, n_heads, q_len, kv_len, d, d, q_len * d, d,
                          kv_len * d, d, q_len * d, 1, 0, 0, 0, -1));
    return md_finish_out(ctx, &O);
}

int md_sdpa_single(md_ctx* ctx, const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint8_t* mask,
                   uint16_t* out, size_t kv_len) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, q && k && v && mask && out, "sdpa_single: null tensor pointer");
    MD_NEED(ctx, kv_len > 0, "sdpa_single: kv_len is 0");
    if (kv_len > 2048) return md_fail(ctx, MD_ERR_SEQUENCE_TOO_LONG, "sdpa_single: kv_len %zu > 2048", kv_len);
    md_arg Q, Kk, V, Mk, O;
    MD_TRY(md_stage_in(ctx, 0, q, 32 * 64 * 2, &Q));
    MD_TRY(md_stage_in(ctx, 1, k, 32 * kv_len * 64 * 2, &Kk));
    MD_TRY(md_stage_in(ctx, 2, v, 32 * kv_len * 64 * 2, &V));
    MD_TRY(md_stage_in(ctx, 3, mask, kv_len, &Mk));
    MD_TRY(md_stage_out(ctx, 4, out, 32 * 64 * 2, &O));
    MD_TRY(md_launch_sdpa_single(ctx, (const __half*)Q.dev, (const __half*)Kk.dev, (const __half*)V.dev,
                                 (const uint8_t*)Mk.dev, (__half*)O.dev, kv_len));
    return md_finish_out(ctx, &O);
}

int md_sdpa_decode_fused(md_ctx* ctx, const uint16_t* qkv_row, uint16_t* key_cache, uint16_t* value_cache,
                         uint16_t* out, size_t n_heads, size_t head_dim, size_t max_seq, size_t pos, size_t rot_dim,
                         float theta) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, qkv_row && key_cache && value_cache && out, "sdpa_decode_fused: null tensor pointer");
    if (pos >= max_seq) return md_fail(ctx, MD_ERR_SEQUENCE_TOO_LONG, "decode: position %zu >= cache size %zu", pos, max_seq);
    if (rot_dim > head_dim || (rot_dim & 1)) return md_fail(ctx, MD_ERR_INVALID_ROT_DIM, "decode: rot_dim %zu", rot_dim);
    return md_launch_sdpa_decode_fused(ctx, (const __half*)qkv_row, (__half*)key_cache, (__half*)value_cache,
                                       (__half*)out, n_heads, head_dim, max_seq, pos, rot_dim, theta);
}

int md_sdpa_prefill_fused(md_ctx* ctx, const uint16_t* qkv, uint16_t* key_cache, uint16_t* value_cache, uint16_t* out,
                          size_t S, size_t n_heads, size_t head_dim, size_t max_seq, size_t pos, size_t rot_dim,
                          float theta) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, qkv && key_cache && value_cache && out, "sdpa_prefill_fused: null tensor pointer");
    MD_NEED(ctx, S > 0, "sdpa_prefill_fused: S is 0");
    if (pos + S > max_seq)
        return md_fail(ctx, MD_ERR_SEQUENCE_TOO_LONG, "prefill: %zu + %zu tokens exceed the cache (%zu)", pos, S, max_seq);
    if (rot_dim > head_dim || (rot_dim & 1)) return md_fail(ctx, MD_ERR_INVALID_ROT_DIM, "prefill: rot_dim %zu", rot_dim);
    const size_t hd = n_heads * head_dim;
    void* q_rot = nullptr;
    MD_TRY(md_scratch(ctx, S * hd * 2, &q_rot));
    MD_TRY(md_launch_rope_cache_write(ctx, (const __half*)qkv, (__half*)q_rot, (__half*)key_cache,
                                      (__half*)value_cache, S, n_heads, head_dim, max_seq, pos, rot_dim, theta));
    return md_launch_sdpa(ctx, (const __half*)q_rot, (const __half*)key_cache, (const __half*)value_cache, nullptr,
                          (__half*)out, n_heads, S, pos + S, head_dim, hd, head_dim, head_dim, max_seq * head_dim, hd,
                          head_dim, 1, 0, 0, 0, (int)pos);
}

int md_sdpa_vit_fused(md_ctx* ctx, const uint16_t* qkv, uint16_t* out, size_t crops, size_t tokens, size_t n_heads,
                      size_t head_dim) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, qkv && out, "sdpa_vit_fused: null tensor pointer");
    MD_NEED(ctx, crops && tokens && n_heads && head_dim, "sdpa_vit_fused: zero-sized dimension");
    const size_t hd = n_heads * head_dim;
    const __half* base = (const __half*)qkv;
    return md_launch_sdpa(ctx, base, base + hd, base + 2 * hd, nullptr, (__half*)out, n_heads, tokens, tokens, head_dim,
                          3 * hd, head_dim, 3 * hd, head_dim, hd, head_dim, crops, tokens * 3 * hd, tokens * 3 * hd,
                          tokens * hd, -1);
}

int md_rope_table(md_ctx* ctx, float* table, size_t dim, size_t end, float theta) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, table, "rope_table: null pointer");
    MD_NEED(ctx, dim > 0 && (dim % 2) == 0 && end > 0 && theta > 0.f, "rope_table: invalid dim/end/theta");
    md_arg T;
    MD_TRY(md_stage_out(ctx, 0, table, end * (dim / 2) * 2 * sizeof(float), &T));
    MD_TRY(md_launch_rope_table(ctx, (float*)T.dev, dim, end, theta));
    return md_finish_out(ctx, &T);
}

int md_rope_apply(md_ctx* ctx, const uint16_t* x, uint16_t* out, size_t n_heads, size_t seq_len, size_t head_dim,
                  const float* freqs_cis, size_t freqs_half, const uint64_t* position_ids, size_t rot_dim) {
    MD_NEED_CTX(ctx);
    if (!x || !out || !freqs_cis || !position_ids)
        return md_fail(ctx, MD_ERR_INVALID_DIMENSION, "rope_apply: null tensor pointer");
    if (rot_dim != freqs_half * 2 || rot_dim > head_dim)
        return md_fail(ctx, MD_ERR_INVALID_ROT_DIM, "rope_apply: rot_dim %zu does not match the table (%zu pairs)", rot_dim,
                       freqs_half);
    // the table must cover the largest position; host position ids are checked here
    md_arg X, F, P, O;
    const size_t n = n_heads * seq_len * head_dim * 2;
    size_t max_pos = 0;
    const bool pos_on_host = !md_is_device_ptr(position_ids);
    if (pos_on_host)
        for (size_t i = 0; i < seq_len; ++i) max_pos = position_ids[i] > max_pos ? (size_t)position_ids[i] : max_pos;
    MD_TRY(md_stage_in(ctx, 0, x, n, &X));
    // a host table is assumed to be the reference's [max_seq=2048 or more, half, 2]; copy what is needed
    const size_t table_rows = pos_on_host ? max_pos + 1 : 0;
    if (!md_is_device_ptr(freqs_cis) && !pos_on_host)
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "rope_apply: a host table needs host position ids");
    MD_TRY(md_stage_in(ctx, 1, freqs_cis, table_rows * freqs_half * 2 * sizeof(float), &F));
    MD_TRY(md_stage_in(ctx, 2, position_ids, seq_len * sizeof(uint64_t), &P));
    MD_TRY(md_stage_out(ctx, 3, out, n, &O));
    MD_TRY(md_launch_rope_apply(ctx, (const __half*)X.dev, (__half*)O.dev, n_heads, seq_len, head_dim,
                                (const float*)F.dev, (const unsigned long long*)P.dev, rot_dim));
    return md_finish_out(ctx, &O);
}

int md_kv_update(md_ctx* ctx, uint16_t* key_cache, uint16_t* value_cache, const uint16_t* k_new, const uint16_t* v_new,
                 size_t n_heads, size_t max_seq, size_t head_dim, size_t cur_len, size_t seq_len) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, key_cache && value_cache && k_new && v_new, "kv_update: null pointer");
    if (cur_len + seq_len > max_seq)
        return md_fail(ctx, MD_ERR_SEQUENCE_TOO_LONG, "kv_update: %zu + %zu > %zu", cur_len, seq_len, max_seq);
    MD_NEED(ctx, md_is_device_ptr(key_cache) && md_is_device_ptr(value_cache), "kv_update: the cache must be device memory");
    md_arg Kn, Vn;
    MD_TRY(md_stage_in(ctx, 0, k_new, n_heads * seq_len * head_dim * 2, &Kn));
    MD_TRY(md_stage_in(ctx, 1, v_new, n_heads * seq_len * head_dim * 2, &Vn));
    return md_launch_kv_update(ctx, (__half*)key_cache, (__half*)value_cache, (const __half*)Kn.dev,
                               (const __half*)Vn.dev, n_heads, max_seq, head_dim, cur_len, seq_len);
}

int md_kv_active(md_ctx* ctx, const uint16_t* key_cache, const uint16_t* value_cache, uint16_t* k_out, uint16_t* v_out,
                 size_t n_heads, size_t max_seq, size_t head_dim, size_t cur_len) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, key_cache && value_cache && k_out && v_out, "kv_active: null pointer");
    if (cur_len > max_seq) return md_fail(ctx, MD_ERR_SEQUENCE_TOO_LONG, "kv_active: %zu > %zu", cur_len, max_seq);
    MD_NEED(ctx, md_is_device_ptr(key_cache) && md_is_device_ptr(value_cache), "kv_active: the cache must be device memory");
    md_arg Ko, Vo;
    const size_t n = n_heads * cur_len * head_dim * 2;
    MD_TRY(md_stage_out(ctx, 0, k_out, n, &Ko));
    MD_TRY(md_stage_out(ctx, 1, v_out, n, &Vo));
    MD_TRY(md_launch_kv_active(ctx, (const __half*)key_cache, (const __half*)value_cache, (__half*)Ko.dev,
                               (__half*)Vo.dev, n_heads, max_seq, head_dim, cur_len));
    if (Ko.staged && n)
        MD_CUDA(ctx, cudaMemcpyAsync(k_out, Ko.dev, n, cudaMemcpyDeviceToHost, ctx->stream));
    Ko.staged = false;
    return md_finish_out(ctx, &Vo);
}

int md_layernorm(md_ctx* ctx, const uint16_t* x, const uint16_t* w, const uint16_t* b, uint16_t* y, size_t rows,
                 size_t cols, uint16_t eps_f16) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, x && w && b && y, "layernorm: null pointer");
    MD_NEED(ctx, cols > 0, "layernorm: empty rows");
    __half_raw raw;
    raw.x = eps_f16;
    const float eps = __half2float(__half(raw));
    MD_NEED(ctx, eps > 0.f, "layernorm: eps must be positive");
    md_arg X, W, B, Y;
    MD_TRY(md_stage_in(ctx, 0, x, rows * cols * 2, &X));
    MD_TRY(md_stage_in(ctx, 1, w, cols * 2, &W));
    MD_TRY(md_stage_in(ctx, 2, b, cols * 2, &B));
    MD_TRY(md_stage_out(ctx, 3, y, rows * cols * 2, &Y));
    MD_TRY(md_launch_layernorm(ctx, (const __half*)X.dev, (const __half*)W.dev, (const __half*)B.dev, (__half*)Y.dev,
                               rows, cols, eps));
    return md_finish_out(ctx, &Y);
}

// in-place ops: a host buffer is staged in, processed, and copied back
static int inplace_begin(md_ctx* ctx, void* a, size_t bytes, md_arg* A) {
    MD_TRY(md_stage_in(ctx, 0, a, bytes, A));
    return MD_OK;
}

int md_gelu(md_ctx* ctx, uint16_t* x, size_t n) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, x, "gelu: null pointer");
    md_arg X;
    MD_TRY(inplace_begin(ctx, x, n * 2, &X));
    MD_TRY(md_launch_gelu(ctx, (__half*)X.dev, n));
    return md_finish_out(ctx, &X);
}

int md_bias_add(md_ctx* ctx, uint16_t* a, const uint16_t* b, size_t rows, size_t cols) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, a && b, "bias_add: null pointer");
    md_arg A, B;
    MD_TRY(inplace_begin(ctx, a, rows * cols * 2, &A));
    MD_TRY(md_stage_in(ctx, 1, b, cols * 2, &B));
    MD_TRY(md_launch_bias_add(ctx, (__half*)A.dev, (const __half*)B.dev, rows, cols));
    return md_finish_out(ctx, &A);
}

int md_add(md_ctx* ctx, uint16_t* a, const uint16_t* b, size_t n) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, a && b, "add: null pointer");
    md_arg A, B;
    MD_TRY(inplace_begin(ctx, a, n * 2, &A));
    MD_TRY(md_stage_in(ctx, 1, b, n * 2, &B));
    MD_TRY(md_launch_add(ctx, (__half*)A.dev, (const __half*)B.dev, n));
    return md_finish_out(ctx, &A);
}

int md_argmax(md_ctx* ctx, const uint16_t* x, size_t n, uint64_t* idx_out) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, x && idx_out, "argmax: null pointer");
    MD_NEED(ctx, n > 0, "argmax: empty tensor");
    md_arg X, I;
    MD_TRY(md_stage_in(ctx, 0, x, n * 2, &X));
    MD_TRY(md_stage_out(ctx, 1, idx_out, sizeof(uint64_t), &I));
    MD_TRY(md_launch_argmax(ctx, (const __half*)X.dev, n, (unsigned long long*)I.dev));
    return md_finish_out(ctx, &I);
}

int md_preprocess_patchify(md_ctx* ctx, const uint8_t* img, uint16_t* out, size_t crops, size_t height, size_t width,
                           size_t patch, size_t out_stride) {
    MD_NEED_CTX(ctx);
    MD_NEED(ctx, img && out, "patchify: null pointer");
    MD_NEED(ctx, patch > 0 && height % patch == 0 && width % patch == 0, "patchify: image not divisible by the patch size");
    MD_NEED(ctx, out_stride >= 3 * patch * patch, "patchify: out_stride smaller than the patch vector");
    md_arg I, O;
    const size_t out_bytes = crops * (height / patch) * (width / patch) * out_stride * 2;
    MD_TRY(md_stage_in(ctx, 0, img, crops * height * width * 3, &I));
    MD_TRY(md_stage_out(ctx, 1, out, out_bytes, &O));
    MD_TRY(md_launch_patchify(ctx, (const uint8_t*)I.dev, (__half*)O.dev, crops, height, width, patch, out_stride));
    return md_finish_out(ctx, &O);
}

}  // extern "C"
