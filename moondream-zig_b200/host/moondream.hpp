// C++ host-side mirror of the reference's operator interface for the hot path.
//
// The reference is Zig; where no Zig toolchain exists this header plays the role of the
// Zig shim: the same function names, argument meaning and error behaviour as
// src/core/{hgemm,hgemm_trans,attention,rope}.zig, implemented as thin calls into the C ABI
// (include/moondream_b200.h).  Zig error unions become exceptions named after the Zig error.
//
//   Tensor<T>                     tensor.zig:12-14  (shape + contiguous row-major data, owned)
//   hgemm::matmul(a, b)           hgemm.zig:362
//   hgemm_trans::matmul(a, b_t)   hgemm_trans.zig:400
//   attention::multiMasklessSDPA  attention.zig:125
//   attention::createAttentionMask attention.zig:256
//   attention::multiMaskedSDPA    attention.zig:416
//   attention::singleMaskedSDPA   attention.zig:759
//   rope::precomputeFreqsCis      rope.zig:32
//   rope::applyRotEmb             rope.zig:130
//   Weights                       weights.zig:61-207 (init from a moondream.bin), 324-369 (deinit)
//
// The allocator parameter of the Zig functions has no counterpart: results are returned by value.
#pragma once

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/moondream_b200.h"
#include "../../include/moondream_b200_model.h"

namespace moondream {

typedef uint16_t f16;  // IEEE binary16 bits

struct ZigError : std::runtime_error {
    std::string name;  // e.g. "IncompatibleTensorShapes"
    ZigError(const std::string& n, const std::string& msg) : std::runtime_error("error." + n + ": " + msg), name(n) {}
};

template <class T> struct Tensor {
    std::vector<size_t> shape;
    std::vector<T> data;
    Tensor() {}
    explicit Tensor(std::vector<size_t> s) : shape(std::move(s)) {
        size_t n = 1;
        for (size_t d : shape) n *= d;
        data.assign(n, T());
    }
    size_t size() const { return data.size(); }
};

// One process-wide context, like the reference's process-wide thread pools.
class Backend {
public:
    static md_ctx* ctx() {
        static Backend b;
        return b.ctx_;
    }
    static void check(int status) {
        if (status == MD_OK) return;
        const std::string msg = md_last_error(ctx_or_null());
        switch (status) {
            case MD_ERR_INVALID_DIMENSION: throw ZigError("InvalidTensorDimension", msg);
            case MD_ERR_SHAPE: throw ZigError("IncompatibleTensorShapes", msg);
            case MD_ERR_SEQUENCE_TOO_LONG: throw ZigError("SequenceTooLong", msg);
            case MD_ERR_INVALID_ROT_DIM: throw ZigError("InvalidRotationDimension", msg);
            case MD_ERR_OOM: throw ZigError("OutOfMemory", msg);
            default: throw ZigError("CudaFailure", msg);
        }
    }

private:
    md_ctx* ctx_ = nullptr;
    static md_ctx*& ctx_or_null() {
        static md_ctx* p = nullptr;
        return p;
    }
    Backend() {
        const int st = md_init(&ctx_, 0);
        if (st != MD_OK) throw ZigError("CudaInitFailed", md_last_error(nullptr));
        ctx_or_null() = ctx_;
    }
    ~Backend() {
        if (ctx_) md_destroy(ctx_);
        ctx_or_null() = nullptr;
    }
};

namespace hgemm {
inline Tensor<f16> matmul(const Tensor<f16>& a, const Tensor<f16>& b) {
    Backend::check(md_check_matmul_shapes(a.shape.data(), a.shape.size(), b.shape.data(), b.shape.size(), 0));
    const size_t M = a.shape[0], K = a.shape[1], N = b.shape[1];
    Tensor<f16> c({M, N});
    Backend::check(md_hgemm_nn(Backend::ctx(), a.data.data(), b.data.data(), c.data.data(), M, N, K));
    return c;
}
}  // namespace hgemm

namespace hgemm_trans {
inline Tensor<f16> matmul(const Tensor<f16>& a, const Tensor<f16>& b_transposed) {
    Backend::check(md_check_matmul_shapes(a.shape.data(), a.shape.size(), b_transposed.shape.data(),
                                          b_transposed.shape.size(), 1));
    const size_t M = a.shape[0], K = a.shape[1], N = b_transposed.shape[0];
    Tensor<f16> c({M, N});
    Backend::check(md_hgemm_nt(Backend::ctx(), a.data.data(), b_transposed.data.data(), c.data.data(), M, N, K));
    return c;
}
}  // namespace hgemm_trans

namespace attention {
inline Tensor<f16> multiMasklessSDPA(size_t n_heads, size_t head_dim, const Tensor<f16>& query, const Tensor<f16>& key,
                                     const Tensor<f16>& value) {
    const size_t q_len = query.shape[1], kv_len = key.shape[1];
    Tensor<f16> out({n_heads, q_len, head_dim});
    Backend::check(md_sdpa_maskless(Backend::ctx(), query.data.data(), key.data.data(), value.data.data(),
                                    out.data.data(), n_heads, q_len, kv_len, head_dim));
    return out;
}

inline Tensor<uint8_t> createAttentionMask(size_t pos, size_t seq_len) {
    Tensor<uint8_t> mask({1, seq_len, pos + seq_len});
    Backend::check(md_create_attention_mask(Backend::ctx(), mask.data.data(), pos, seq_len));
    return mask;
}

inline Tensor<f16> multiMaskedSDPA(const Tensor<f16>& query, const Tensor<f16>& key, const Tensor<f16>& value,
                                   const Tensor<uint8_t>& mask, size_t n_heads, size_t head_dim) {
    const size_t q_len = query.shape[1], kv_len = key.shape[1];
    Tensor<f16> out({n_heads, q_len, head_dim});
    Backend::check(md_sdpa_masked(Backend::ctx(), query.data.data(), key.data.data(), value.data.data(),
                                  mask.data.data(), out.data.data(), n_heads, q_len, kv_len, head_dim));
    return out;
}

inline Tensor<f16> singleMaskedSDPA(const Tensor<f16>& query, const Tensor<f16>& key, const Tensor<f16>& value,
                                    const Tensor<uint8_t>& mask) {
    const size_t kv_len = key.shape[1];
    Tensor<f16> out({32, 1, 64});
    Backend::check(md_sdpa_single(Backend::ctx(), query.data.data(), key.data.data(), value.data.data(),
                                  mask.data.data(), out.data.data(), kv_len));
    return out;
}
}  // namespace attention

namespace rope {
inline Tensor<float> precomputeFreqsCis(size_t dim, size_t end, float theta) {
    if (dim == 0) throw ZigError("DimensionTooSmall", "dim is 0");
    if (dim % 2 != 0) throw ZigError("DimensionNotEven", "dim is odd");
    if (end == 0) throw ZigError("EndTooSmall", "end is 0");
    if (!(theta > 0.f)) throw ZigError("ThetaTooSmall", "theta <= 0");
    Tensor<float> t({end, dim / 2, 2});
    Backend::check(md_rope_table(Backend::ctx(), t.data.data(), dim, end, theta));
    return t;
}

inline Tensor<f16> applyRotEmb(const Tensor<f16>& x, size_t n_heads, size_t head_dim, const Tensor<float>& freqs_cis,
                               const Tensor<uint64_t>& position_ids, size_t rot_dim) {
    if (x.shape.size() != 3) throw ZigError("InvalidInputDimensions", "x must be rank 3");
    const size_t freqs_half = freqs_cis.shape[freqs_cis.shape.size() - 2];
    Tensor<f16> out(x.shape);
    Backend::check(md_rope_apply(Backend::ctx(), x.data.data(), out.data.data(), n_heads, x.shape[1], head_dim,
                                 freqs_cis.data.data(), freqs_half, position_ids.data.data(), rot_dim));
    return out;
}
}  // namespace rope

// Weights.init(config, filename, allocator): parse and validate the file, then make it resident on the
// backend's device.  The Zig error of a rejected file (InvalidMagicNumber, ShapeMismatch, ...) is the name of
// the exception.  text() / vision() give the device-pointer tables the model runners take.
class Weights {
public:
    explicit Weights(const std::string& filename, const md_model_config* config = nullptr) {
        fail_if(md_weight_file_open(filename.c_str(), config, &file_), nullptr);
        const int st = md_weight_file_upload(file_, Backend::ctx());
        if (st != MD_OK) {
            md_weight_file_close(file_);
            file_ = nullptr;
            Backend::check(st);
        }
    }
    ~Weights() { md_weight_file_close(file_); }
    Weights(const Weights&) = delete;
    Weights& operator=(const Weights&) = delete;

    md_text_weights text() {
        md_text_weights w;
        fail_if(md_weight_file_text(file_, &w), Backend::ctx());
        return w;
    }
    md_vision_weights vision() {
        md_vision_weights w;
        fail_if(md_weight_file_vision(file_, &w), Backend::ctx());
        return w;
    }

private:
    md_weight_file* file_ = nullptr;
    static void fail_if(int status, const md_ctx* ctx) {
        if (status == MD_OK) return;
        const std::string msg = md_last_error(ctx);
        if (status == MD_ERR_IO || status == MD_ERR_FORMAT) throw ZigError(msg.substr(0, msg.find(':')), msg);
        Backend::check(status);
    }
};

}  // namespace moondream
