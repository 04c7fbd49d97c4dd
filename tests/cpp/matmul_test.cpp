// The reference's hgemm tests (src/core/matmul_test.zig:154-367) restated against the C++ host
// mirror: same shapes, fill patterns, in-test naive product and comparison rule.  Prints one
// "ok <name>" line per test; exits non-zero on the first failure.
#include <cmath>
#include <cstdio>
#include <random>

#include <cuda_fp16.h>

#include "../../moondream-zig_b200/host/moondream.hpp"

using namespace moondream;

static float h2f(f16 h) { __half_raw r; r.x = h; return __half2float(__half(r)); }
static f16 f2h(float f) { __half_raw r = __float2half_rn(f); return r.x; }

enum Pattern { Identity, Sequential, Random };

// fillTestPattern, matmul_test.zig:40-66
static void fill(Tensor<f16>& t, Pattern p) {
    const size_t rows = t.shape[0], cols = t.shape[1];
    std::mt19937 rng(42);
    std::uniform_real_distribution<float> u(0.f, 1.f);
    for (size_t i = 0; i < rows; ++i)
        for (size_t j = 0; j < cols; ++j) {
            const size_t idx = i * cols + j;
            if (p == Identity) t.data[idx] = f2h(i == j ? 1.f : 0.f);
            else if (p == Sequential) t.data[idx] = f2h((float)idx * 0.01f);
            else t.data[idx] = f2h(u(rng) * 2.f - 1.f);
        }
}
static void scale(Tensor<f16>& t, float s) { for (auto& v : t.data) v = f2h(h2f(v) * s); }

// naiveMatMulF16, matmul_test.zig:83-106
static Tensor<f16> naive(const Tensor<f16>& A, const Tensor<f16>& B) {
    const size_t M = A.shape[0], K = A.shape[1], N = B.shape[1];
    Tensor<f16> C({M, N});
    for (size_t i = 0; i < M; ++i)
        for (size_t j = 0; j < N; ++j) {
            float sum = 0.f;
            for (size_t k = 0; k < K; ++k) sum += h2f(A.data[i * K + k]) * h2f(B.data[k * N + j]);
            C.data[i * N + j] = f2h(sum);
        }
    return C;
}

// compareResultsF16, matmul_test.zig:108-152
static bool compare(const Tensor<f16>& e, const Tensor<f16>& a, float eps) {
    if (e.shape != a.shape) return false;
    size_t bad = 0;
    for (size_t i = 0; i < e.size(); ++i) {
        const float ev = h2f(e.data[i]), av = h2f(a.data[i]), diff = std::fabs(ev - av);
        const bool big = std::fabs(ev) > 1.0f;
        if ((big ? diff / std::fabs(ev) : diff) > (big ? eps : eps * 0.1f)) ++bad;
    }
    return bad == 0;
}

#define CHECK(name, cond)                                   \
    do {                                                    \
        if (!(cond)) { std::printf("FAIL %s\n", name); return 1; } \
        std::printf("ok %s\n", name);                       \
    } while (0)

int main() {
    {   // "HGEMM MatMul - Basic functionality"
        Tensor<f16> A({4, 3}), B({3, 4});
        fill(A, Sequential); fill(B, Sequential);
        CHECK("basic", compare(naive(A, B), hgemm::matmul(A, B), 0.005f));
    }
    {   // "HGEMM MatMul - Large matrices"
        Tensor<f16> A({2000, 180}), B({180, 1600});
        fill(A, Random); fill(B, Random); scale(A, 0.01f); scale(B, 0.01f);
        CHECK("large", compare(naive(A, B), hgemm::matmul(A, B), 0.05f));
    }
    {   // "HGEMM MatMul - Non-square matrices"
        const size_t shapes[3][3] = {{50, 30, 70}, {25, 80, 35}, {100, 20, 100}};
        for (auto& s : shapes) {
            Tensor<f16> A({s[0], s[1]}), B({s[1], s[2]});
            fill(A, Random); fill(B, Random); scale(A, 0.01f); scale(B, 0.01f);
            CHECK("non-square", compare(naive(A, B), hgemm::matmul(A, B), 0.05f));
        }
    }
    {   // "HGEMM MatMul - Identity matrix"
        Tensor<f16> A({32, 32}), I({32, 32});
        fill(A, Random); fill(I, Identity); scale(A, 0.01f);
        CHECK("identity", compare(A, hgemm::matmul(A, I), 0.005f));
    }
    {   // "HGEMM MatMul - Error cases"
        Tensor<f16> A({3, 4}), B({5, 6});
        bool thrown = false;
        try { hgemm::matmul(A, B); } catch (const ZigError& e) { thrown = e.name == "IncompatibleTensorShapes"; }
        CHECK("error-case", thrown);
        thrown = false;
        try { hgemm_trans::matmul(A, B); } catch (const ZigError& e) { thrown = e.name == "IncompatibleTensorShapes"; }
        CHECK("error-case-trans", thrown);
    }
    {   // "HGEMM MatMul - Tile boundary cases"
        for (size_t size : {158, 159, 160, 161, 162}) {
            Tensor<f16> A({size, size}), B({size, size});
            fill(A, Random); fill(B, Random); scale(A, 0.01f); scale(B, 0.01f);
            CHECK("tile-boundary", compare(naive(A, B), hgemm::matmul(A, B), 0.05f));
        }
    }
    {   // "HGEMM MatMul - Numerical stability"
        for (float v : {1e-2f, 1.0f}) {
            Tensor<f16> A({32, 32}), B({32, 32});
            for (auto& x : A.data) x = f2h(v);
            for (auto& x : B.data) x = f2h(v);
            CHECK("constant", compare(naive(A, B), hgemm::matmul(A, B), 0.01f));
        }
    }
    {   // hgemm_trans against hgemm on the transposed weight, incl. the M == 1 vector path
        for (size_t M : {1, 8, 64}) {
            Tensor<f16> A({M, 256}), B({256, 96}), Bt({96, 256});
            fill(A, Random); fill(B, Random); scale(B, 0.05f);
            for (size_t k = 0; k < 256; ++k) for (size_t n = 0; n < 96; ++n) Bt.data[n * 256 + k] = B.data[k * 96 + n];
            CHECK("trans-vs-nn", compare(naive(A, B), hgemm_trans::matmul(A, Bt), 0.05f));
        }
    }
    {   // attention + rope smoke through the mirror: mask shape and error behaviour
        auto m = attention::createAttentionMask(3, 2);
        CHECK("mask", m.shape.size() == 3 && m.shape[2] == 5 && m.data[0 * 5 + 3] == 1 && m.data[0 * 5 + 4] == 0 &&
                          m.data[1 * 5 + 4] == 1);
        Tensor<f16> q({32, 1, 64}), k({32, 2049, 64});
        Tensor<uint8_t> mk({1, 1, 2049});
        bool thrown = false;
        try { attention::singleMaskedSDPA(q, k, k, mk); } catch (const ZigError& e) { thrown = e.name == "SequenceTooLong"; }
        CHECK("sequence-too-long", thrown);
        auto t = rope::precomputeFreqsCis(32, 2048, 10000.f);
        CHECK("rope-table", t.shape[0] == 2048 && t.shape[1] == 16 && std::fabs(t.data[0] - 1.f) < 1e-6f);
        Tensor<f16> x({32, 2, 64});
        Tensor<uint64_t> pos({2});
        thrown = false;
        try { rope::applyRotEmb(x, 32, 64, t, pos, 30); } catch (const ZigError& e) { thrown = e.name == "InvalidRotationDimension"; }
        CHECK("rope-rot-dim", thrown);
    }
    std::printf("all ok\n");
    return 0;
}
