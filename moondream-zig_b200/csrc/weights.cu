// Reader of the moondream.bin weight file (the format weights.zig:61-207 reads and weights.py:82-246
// writes) and its upload into HBM.  Host code only: parsing runs without a device, the upload streams the
// mapped file through two pinned staging buffers so that the page-in of the next chunk overlaps the
// host-to-device copy of the previous one.
#include "md_internal.cuh"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <vector>

#include "../../include/moondream_b200_model.h"

namespace {

constexpr uint32_t WEIGHTS_MAGIC = 0x4D4F4F4E;  // "MOON", weights.zig:10
constexpr uint32_t WEIGHTS_VERSION = 2;         // weights.zig:11
constexpr size_t STAGE_CHUNK = size_t(64) << 20;

struct Expected {
    const char* name;
    std::vector<size_t> shape;
};

// calculateShapes (weights.zig:439-478), in the order weights.py writes the tensors.
std::vector<Expected> expected_shapes(const md_model_config& c) {
    const size_t qkv = c.n_heads * c.head_dim * 3, vqkv = c.n_vit_heads * c.vit_head_dim * 3;
    const size_t L = c.n_layers, V = c.n_vit_layers;
    return {
        {"word_token_embedding", {c.vocab, c.dim}},
        {"t_ln_w", {L, c.dim}},
        {"t_ln_b", {L, c.dim}},
        {"t_Wqkv_w", {L, qkv, c.dim}},
        {"t_Wqkv_b", {L, qkv}},
        {"t_out_proj_w", {L, c.dim, c.dim}},
        {"t_out_proj_bias", {L, c.dim}},
        {"t_fc1_w", {L, c.hidden_dim, c.dim}},
        {"t_fc1_b", {L, c.hidden_dim}},
        {"t_fc2_w", {L, c.dim, c.hidden_dim}},
        {"t_fc2_b", {L, c.dim}},
        {"t_linear_w", {c.vocab, c.dim}},
        {"t_linear_b", {c.vocab}},
        {"t_ln_out_w", {c.dim}},
        {"t_ln_out_b", {c.dim}},
        {"v_patch_embedding_linear_w", {c.patch_size * c.patch_size * c.img_channels, c.vit_dim}},
        {"v_patch_embedding_linear_b", {c.vit_dim}},
        {"v_pos_embedding", {1, c.num_patches, c.vit_dim}},
        {"v_Wqkv_w", {V, c.vit_dim, vqkv}},
        {"v_Wqkv_b", {V, vqkv}},
        {"v_out_proj_w", {V, c.vit_dim, c.vit_dim}},
        {"v_out_proj_b", {V, c.vit_dim}},
        {"v_fc1_w", {V, c.vit_dim, c.hidden_features}},
        {"v_fc1_b", {V, c.hidden_features}},
        {"v_fc2_w", {V, c.hidden_features, c.vit_dim}},
        {"v_fc2_b", {V, c.vit_dim}},
        {"v_norm1_w", {V, c.vit_dim}},
        {"v_norm1_b", {V, c.vit_dim}},
        {"v_norm2_w", {V, c.vit_dim}},
        {"v_norm2_b", {V, c.vit_dim}},
        {"v_norm_out_w", {c.vit_dim}},
        {"v_norm_out_b", {c.vit_dim}},
        // the reference sizes the projection input with the TEXT head count (weights.zig:470)
        {"v_proj_fc1_w", {c.vit_head_dim * c.n_heads, c.hidden_dim}},
        {"v_proj_fc1_b", {c.hidden_dim}},
        {"v_proj_fc2_w", {c.hidden_dim, c.dim}},
        {"v_proj_fc2_b", {c.dim}},
    };
}

std::string shape_str(const std::vector<size_t>& s) {
    std::string r = "[";
    for (size_t i = 0; i < s.size(); ++i) r += (i ? ", " : "") + std::to_string(s[i]);
    return r + "]";
}

uint32_t rd32(const uint8_t* p) {
    uint32_t v;
    memcpy(&v, p, 4);
    return v;  // the file and every supported host are little-endian
}
uint64_t rd64(const uint8_t* p) {
    uint64_t v;
    memcpy(&v, p, 8);
    return v;
}

}  // namespace

struct md_weight_file {
    md_model_config cfg;
    std::vector<Expected> expected;
    int fd = -1;
    const uint8_t* map = nullptr;
    size_t map_bytes = 0;
    struct Tensor {
        std::string name;
        std::vector<size_t> shape;
        size_t offset = 0, elems = 0;  // data position in the mapping, element count
        void* dev = nullptr;
    };
    std::vector<Tensor> tensors;          // file order
    md_ctx* ctx = nullptr;                // set by upload
    std::vector<std::vector<const uint16_t*>> layer_ptrs;  // per-layer pointer arrays handed out to the models

    const Tensor* find(const char* name) const {
        const Tensor* hit = nullptr;
        for (const Tensor& t : tensors)
            if (t.name == name) hit = &t;  // the last occurrence wins (weights.zig:240-322 overwrites the field)
        return hit;
    }
};

int md_model_config_default(md_model_config* c) {
    if (!c) return md_fail(nullptr, MD_ERR_INVALID_ARG, "md_model_config_default: null pointer");
    *c = md_model_config{};
    c->vocab = 51200, c->dim = 2048, c->hidden_dim = 8192, c->n_layers = 24, c->n_heads = 32, c->head_dim = 64;
    c->seq_len = 2048, c->rope_theta = 10000.f, c->partial_rotary_factor = 0.5f;
    c->img_channels = 3, c->img_dim = 378, c->patch_size = 14, c->num_patches = (378 / 14) * (378 / 14);
    c->vit_dim = 1152, c->n_vit_layers = 27, c->n_vit_heads = 16, c->vit_head_dim = 72, c->hidden_features = 4304;
    return MD_OK;
}

static int parse(md_weight_file* wf, const char* path) {
    const uint8_t* p = wf->map;
    const size_t n = wf->map_bytes;
    size_t pos = 0;
    if (n < 4) return md_fail(nullptr, MD_ERR_IO, "InvalidRead: %s ends inside the magic number", path);
    if (rd32(p) != WEIGHTS_MAGIC)
        return md_fail(nullptr, MD_ERR_FORMAT, "InvalidMagicNumber: %s starts with 0x%08X, expected 0x%08X", path,
                       rd32(p), WEIGHTS_MAGIC);
    if (n < 8) return md_fail(nullptr, MD_ERR_IO, "InvalidRead: %s ends inside the version", path);
    if (rd32(p + 4) != WEIGHTS_VERSION)
        return md_fail(nullptr, MD_ERR_FORMAT, "InvalidVersion: %s has version %u, expected %u", path, rd32(p + 4),
                       WEIGHTS_VERSION);
    pos = 8;
    while (pos < n) {
        if (n - pos < 12)
            return md_fail(nullptr, MD_ERR_FORMAT, "InvalidHeader: %zu trailing bytes at offset %zu of %s", n - pos, pos,
                           path);
        const uint32_t name_length = rd32(p + pos), shape_length = rd32(p + pos + 4);
        // the third word (element count) is written by weights.py:118-123 and never read by weights.zig:140-141
        if (name_length > 256)
            return md_fail(nullptr, MD_ERR_FORMAT, "InvalidNameLength: %u at offset %zu of %s", name_length, pos, path);
        if (shape_length > 4)
            return md_fail(nullptr, MD_ERR_FORMAT, "InvalidShapeLength: %u at offset %zu of %s", shape_length, pos, path);
        pos += 12;
        if (n - pos < name_length) return md_fail(nullptr, MD_ERR_IO, "InvalidRead: %s ends inside a tensor name", path);
        md_weight_file::Tensor t;
        t.name.assign(reinterpret_cast<const char*>(p + pos), name_length);
        pos += name_length;
        if (n - pos < size_t(8) * shape_length)
            return md_fail(nullptr, MD_ERR_IO, "InvalidRead: %s ends inside the shape of %s", path, t.name.c_str());
        for (uint32_t i = 0; i < shape_length; ++i) t.shape.push_back(size_t(rd64(p + pos + 8 * i)));
        pos += size_t(8) * shape_length;
        const Expected* want = nullptr;
        for (const Expected& e : wf->expected)
            if (t.name == e.name) want = &e;
        if (!want)
            return md_fail(nullptr, MD_ERR_FORMAT, "UnknownTensorName: '%s' at offset %zu of %s", t.name.c_str(), pos,
                           path);
        if (t.shape != want->shape)
            return md_fail(nullptr, MD_ERR_FORMAT, "ShapeMismatch: tensor '%s' has shape %s, expected %s",
                           t.name.c_str(), shape_str(t.shape).c_str(), shape_str(want->shape).c_str());
        t.elems = 1;
        for (size_t d : t.shape) t.elems *= d;
        if ((n - pos) / 2 < t.elems)
            return md_fail(nullptr, MD_ERR_IO, "InvalidRead: %s holds %zu of the %zu bytes of tensor '%s'", path, n - pos,
                           t.elems * 2, t.name.c_str());
        t.offset = pos;
        pos += t.elems * 2;
        wf->tensors.push_back(std::move(t));
    }
    return MD_OK;
}

int md_weight_file_open(const char* path, const md_model_config* cfg, md_weight_file** out) {
    if (!path || !out) return md_fail(nullptr, MD_ERR_INVALID_ARG, "md_weight_file_open: null pointer");
    *out = nullptr;
    md_weight_file* wf = new md_weight_file();
    if (cfg) wf->cfg = *cfg;
    else md_model_config_default(&wf->cfg);
    wf->expected = expected_shapes(wf->cfg);
    wf->fd = open(path, O_RDONLY);
    struct stat st;
    if (wf->fd < 0 || fstat(wf->fd, &st) != 0) {
        const int st_open = md_fail(nullptr, MD_ERR_IO, "FileNotFound: cannot open %s: %s", path, strerror(errno));
        md_weight_file_close(wf);
        return st_open;
    }
    wf->map_bytes = size_t(st.st_size);
    if (wf->map_bytes) {
        void* m = mmap(nullptr, wf->map_bytes, PROT_READ, MAP_PRIVATE, wf->fd, 0);
        if (m == MAP_FAILED) {
            const int st_map = md_fail(nullptr, MD_ERR_IO, "FileNotFound: cannot map %s: %s", path, strerror(errno));
            md_weight_file_close(wf);
            return st_map;
        }
        wf->map = static_cast<const uint8_t*>(m);
        madvise(m, wf->map_bytes, MADV_SEQUENTIAL);
    }
    const int status = parse(wf, path);
    if (status != MD_OK) {
        md_weight_file_close(wf);
        return status;
    }
    *out = wf;
    return MD_OK;
}

int md_weight_file_close(md_weight_file* wf) {
    if (!wf) return MD_OK;
    if (wf->ctx) {
        cudaSetDevice(wf->ctx->device);
        for (md_weight_file::Tensor& t : wf->tensors)
            if (t.dev) cudaFree(t.dev);
    }
    if (wf->map) munmap(const_cast<uint8_t*>(wf->map), wf->map_bytes);
    if (wf->fd >= 0) close(wf->fd);
    delete wf;
    return MD_OK;
}

int md_weight_file_count(const md_weight_file* wf, size_t* n_out) {
    if (!wf || !n_out) return md_fail(nullptr, MD_ERR_INVALID_ARG, "md_weight_file_count: null pointer");
    *n_out = wf->tensors.size();
    return MD_OK;
}

int md_weight_file_tensor(const md_weight_file* wf, size_t index, const char** name, size_t* rank, size_t shape[4],
                          const uint16_t** host_data) {
    if (!wf) return md_fail(nullptr, MD_ERR_INVALID_ARG, "md_weight_file_tensor: null pointer");
    if (index >= wf->tensors.size())
        return md_fail(nullptr, MD_ERR_INVALID_ARG, "md_weight_file_tensor: index %zu of %zu", index, wf->tensors.size());
    const md_weight_file::Tensor& t = wf->tensors[index];
    if (name) *name = t.name.c_str();
    if (rank) *rank = t.shape.size();
    if (shape)
        for (size_t i = 0; i < t.shape.size(); ++i) shape[i] = t.shape[i];
    if (host_data) *host_data = reinterpret_cast<const uint16_t*>(wf->map + t.offset);
    return MD_OK;
}

int md_weight_file_upload(md_weight_file* wf, md_ctx* ctx) {
    if (!wf || !ctx) return md_fail(ctx, MD_ERR_INVALID_ARG, "md_weight_file_upload: null pointer");
    if (wf->ctx) return md_fail(ctx, MD_ERR_INVALID_ARG, "md_weight_file_upload: the file is already resident");
    MD_CUDA(ctx, cudaSetDevice(ctx->device));
    wf->ctx = ctx;  // from here on md_weight_file_close frees what was allocated, also after a failure
    uint8_t* stage[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    auto release = [&]() {
        for (int i = 0; i < 2; ++i) {
            if (stage[i]) cudaFreeHost(stage[i]);
            if (done[i]) cudaEventDestroy(done[i]);
        }
    };
    int status = MD_OK;
    auto run = [&]() -> int {
        for (int i = 0; i < 2; ++i) {
            MD_CUDA(ctx, cudaMallocHost(reinterpret_cast<void**>(&stage[i]), STAGE_CHUNK));
            MD_CUDA(ctx, cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming));
        }
        size_t turn = 0;
        for (md_weight_file::Tensor& t : wf->tensors) {
            const size_t bytes = t.elems * 2;
            if (!bytes) continue;
            MD_CUDA(ctx, cudaMalloc(&t.dev, bytes));
            for (size_t off = 0; off < bytes; off += STAGE_CHUNK, ++turn) {
                const int b = int(turn & 1);
                const size_t len = std::min(STAGE_CHUNK, bytes - off);
                if (turn >= 2) MD_CUDA(ctx, cudaEventSynchronize(done[b]));  // the copy that last used this buffer
                memcpy(stage[b], wf->map + t.offset + off, len);             // pages the file in
                MD_CUDA(ctx, cudaMemcpyAsync(static_cast<uint8_t*>(t.dev) + off, stage[b], len, cudaMemcpyHostToDevice,
                                             ctx->stream));
                MD_CUDA(ctx, cudaEventRecord(done[b], ctx->stream));
            }
        }
        MD_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        return MD_OK;
    };
    status = run();
    if (status != MD_OK) cudaStreamSynchronize(ctx->stream);  // nothing may still read the staging buffers
    release();
    return status;
}

namespace {

// Device pointer of a tensor, or of each layer of a stacked tensor.
int need(md_weight_file* wf, const char* name, const md_weight_file::Tensor** out) {
    if (!wf->ctx) return md_fail(nullptr, MD_ERR_INVALID_ARG, "the weight file is not resident: call md_weight_file_upload first");
    const md_weight_file::Tensor* t = wf->find(name);
    if (!t) return md_fail(wf->ctx, MD_ERR_FORMAT, "MissingTensor: the weight file holds no '%s'", name);
    *out = t;
    return MD_OK;
}
int single(md_weight_file* wf, const char* name, const uint16_t** out) {
    const md_weight_file::Tensor* t;
    MD_TRY(need(wf, name, &t));
    *out = static_cast<const uint16_t*>(t->dev);
    return MD_OK;
}
int stacked(md_weight_file* wf, const char* name, const uint16_t* const** out) {
    const md_weight_file::Tensor* t;
    MD_TRY(need(wf, name, &t));
    const size_t layers = t->shape[0], stride = layers ? t->elems / layers : 0;
    wf->layer_ptrs.emplace_back();
    std::vector<const uint16_t*>& v = wf->layer_ptrs.back();
    for (size_t l = 0; l < layers; ++l) v.push_back(static_cast<const uint16_t*>(t->dev) + l * stride);
    *out = v.data();
    return MD_OK;
}
uint16_t eps_bits() { return 0x00A8; }  // f16(1e-5) = 1.0013580322265625e-05 (text_model.zig:28, vision_model.zig:35)

}  // namespace

int md_weight_file_text(md_weight_file* wf, md_text_weights* w) {
    if (!wf || !w) return md_fail(nullptr, MD_ERR_INVALID_ARG, "md_weight_file_text: null pointer");
    const md_model_config& c = wf->cfg;
    *w = md_text_weights{};
    w->n_layers = c.n_layers, w->dim = c.dim, w->hidden = c.hidden_dim, w->n_heads = c.n_heads, w->head_dim = c.head_dim;
    w->vocab = c.vocab, w->max_seq = c.seq_len;
    w->rot_dim = size_t(float(c.head_dim) * c.partial_rotary_factor);
    w->rope_theta = c.rope_theta, w->eps_f16 = eps_bits();
    MD_TRY(stacked(wf, "t_ln_w", &w->ln_w));
    MD_TRY(stacked(wf, "t_ln_b", &w->ln_b));
    MD_TRY(stacked(wf, "t_Wqkv_w", &w->wqkv));
    MD_TRY(stacked(wf, "t_Wqkv_b", &w->bqkv));
    MD_TRY(stacked(wf, "t_out_proj_w", &w->wout));
    MD_TRY(stacked(wf, "t_out_proj_bias", &w->bout));
    MD_TRY(stacked(wf, "t_fc1_w", &w->wfc1));
    MD_TRY(stacked(wf, "t_fc1_b", &w->bfc1));
    MD_TRY(stacked(wf, "t_fc2_w", &w->wfc2));
    MD_TRY(stacked(wf, "t_fc2_b", &w->bfc2));
    MD_TRY(single(wf, "t_ln_out_w", &w->ln_out_w));
    MD_TRY(single(wf, "t_ln_out_b", &w->ln_out_b));
    MD_TRY(single(wf, "t_linear_w", &w->lm_w));
    MD_TRY(single(wf, "t_linear_b", &w->lm_b));
    MD_TRY(single(wf, "word_token_embedding", &w->wte));
    return MD_OK;
}

int md_weight_file_vision(md_weight_file* wf, md_vision_weights* w) {
    if (!wf || !w) return md_fail(nullptr, MD_ERR_INVALID_ARG, "md_weight_file_vision: null pointer");
    const md_model_config& c = wf->cfg;
    *w = md_vision_weights{};
    w->n_layers = c.n_vit_layers, w->dim = c.vit_dim, w->n_heads = c.n_vit_heads, w->head_dim = c.vit_head_dim;
    w->hidden = c.hidden_features, w->tokens = c.num_patches, w->patch = c.patch_size, w->img = c.img_dim;
    w->proj_hidden = c.hidden_dim, w->proj_out = c.dim, w->eps_f16 = eps_bits();
    MD_TRY(single(wf, "v_patch_embedding_linear_w", &w->patch_w));
    MD_TRY(single(wf, "v_patch_embedding_linear_b", &w->patch_b));
    MD_TRY(single(wf, "v_pos_embedding", &w->pos_emb));
    MD_TRY(stacked(wf, "v_norm1_w", &w->ln1_w));
    MD_TRY(stacked(wf, "v_norm1_b", &w->ln1_b));
    MD_TRY(stacked(wf, "v_Wqkv_w", &w->wqkv));
    MD_TRY(stacked(wf, "v_Wqkv_b", &w->bqkv));
    MD_TRY(stacked(wf, "v_out_proj_w", &w->wout));
    MD_TRY(stacked(wf, "v_out_proj_b", &w->bout));
    MD_TRY(stacked(wf, "v_norm2_w", &w->ln2_w));
    MD_TRY(stacked(wf, "v_norm2_b", &w->ln2_b));
    MD_TRY(stacked(wf, "v_fc1_w", &w->wfc1));
    MD_TRY(stacked(wf, "v_fc1_b", &w->bfc1));
    MD_TRY(stacked(wf, "v_fc2_w", &w->wfc2));
    MD_TRY(stacked(wf, "v_fc2_b", &w->bfc2));
    MD_TRY(single(wf, "v_norm_out_w", &w->norm_w));
    MD_TRY(single(wf, "v_norm_out_b", &w->norm_b));
    MD_TRY(single(wf, "v_proj_fc1_w", &w->proj_fc1_w));
    MD_TRY(single(wf, "v_proj_fc1_b", &w->proj_fc1_b));
    MD_TRY(single(wf, "v_proj_fc2_w", &w->proj_fc2_w));
    MD_TRY(single(wf, "v_proj_fc2_b", &w->proj_fc2_b));
    return MD_OK;
}
