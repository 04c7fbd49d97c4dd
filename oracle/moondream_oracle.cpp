// CPU oracle for the moondream-zig FP16 matmul + attention hot path.
//
// TEST INFRASTRUCTURE ONLY — see moondream_oracle.h for the parity status of
// every function (which rows are pinned by the reference's own tests and which
// are unpinned).  Each function names the reference file:line it restates.
//
// The arithmetic mirrors the reference: f16 storage, widening to f32, 8-lane
// f32 FMA vectors (the reference's @Vector(8,f32) + @mulAdd), round-to-nearest-
// even f32->f16 exactly where the reference rounds.  Threading mirrors it too:
// worker threads are spawned and joined inside every matmul call and pull work
// items from one atomic counter (hgemm.zig:100-143,419-423).
//
// Build: g++ -O3 -std=c++17 -mavx2 -mfma -mf16c -shared -fPIC -pthread

#include "moondream_oracle.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

namespace {

typedef _Float16 f16;
typedef float v8f __attribute__((vector_size(32)));

inline float h2f(uint16_t h) { f16 x; std::memcpy(&x, &h, 2); return (float)x; }
inline uint16_t f2h(float f) { f16 x = (f16)f; uint16_t h; std::memcpy(&h, &x, 2); return h; }
inline const f16* H(const uint16_t* p) { return reinterpret_cast<const f16*>(p); }
inline f16* H(uint16_t* p) { return reinterpret_cast<f16*>(p); }

std::atomic<int> g_threads{0};

int worker_count() {
    int n = g_threads.load();
    if (n <= 0) n = (int)std::thread::hardware_concurrency();
    return n > 0 ? n : 1;
}

// Spawn n threads running fn(thread_index) and join them: the reference creates
// and joins its workers inside every call (hgemm.zig:419-423).
template <class F> void spawn_join(int n, F fn) {
    if (n <= 1) { fn(0); return; }
    std::vector<std::thread> pool;
    pool.reserve(n);
    for (int t = 0; t < n; ++t) pool.emplace_back(fn, t);
    for (auto& th : pool) th.join();
}

constexpr size_t TILE = 168;  // hgemm.zig:34-38, hgemm_trans.zig:19

struct TileBuf {
    alignas(32) float a[TILE][TILE];
    alignas(32) float b[TILE][TILE];
    alignas(32) float c[TILE][TILE];
};

// hgemm.zig:231-347 / hgemm_trans.zig:293-356 — 8x8 register-blocked outer
// products over k, scalar FMA tails for the N%8 columns and the M%8 rows.
void tile_fma(TileBuf& t, size_t i_size, size_t j_size, size_t k_size) {
    size_t i = 0;
    for (; i + 8 <= i_size; i += 8) {
        size_t j = 0;
        for (; j + 8 <= j_size; j += 8) {
            v8f acc[8];
            for (int r = 0; r < 8; ++r) acc[r] = v8f{0, 0, 0, 0, 0, 0, 0, 0};
            for (size_t k = 0; k < k_size; ++k) {
                v8f bv;
                std::memcpy(&bv, &t.b[k][j], 32);
                for (int r = 0; r < 8; ++r) {
                    float s = t.a[i + r][k];
                    v8f av = v8f{s, s, s, s, s, s, s, s};
                    acc[r] = av * bv + acc[r];
                }
            }
            for (int r = 0; r < 8; ++r)
                for (int cidx = 0; cidx < 8; ++cidx) t.c[i + r][j + cidx] += acc[r][cidx];
        }
        for (; j < j_size; ++j) {
            for (int r = 0; r < 8; ++r) {
                float sum = 0.f;
                for (size_t k = 0; k < k_size; ++k) sum = std::fma(t.a[i + r][k], t.b[k][j], sum);
                t.c[i + r][j] += sum;
            }
        }
    }
    for (; i < i_size; ++i) {
        for (size_t j = 0; j < j_size; ++j) {
            float sum = 0.f;
            for (size_t k = 0; k < k_size; ++k) sum = std::fma(t.a[i][k], t.b[k][j], sum);
            t.c[i][j] += sum;
        }
    }
}

// Tiled GEMM shared by the NN (hgemm.zig:100-143) and NT (hgemm_trans.zig:359-398)
// entry points; they differ only in how the B sub-tile is widened into b[k][j].
template <bool B_TRANSPOSED>
void hgemm_tiled(const f16* A, const f16* B, f16* C, size_t M, size_t N, size_t K) {
    const size_t tiles_m = (M + TILE - 1) / TILE, tiles_n = (N + TILE - 1) / TILE;
    const size_t total = tiles_m * tiles_n;
    std::atomic<size_t> next{0};
    spawn_join(worker_count(), [&](int) {
        std::vector<TileBuf> holder(1);
        TileBuf& t = holder[0];
        for (;;) {
            size_t idx = next.fetch_add(1);
            if (idx >= total) break;
            const size_t i0 = (idx / tiles_n) * TILE, j0 = (idx % tiles_n) * TILE;
            const size_t i1 = std::min(i0 + TILE, M), j1 = std::min(j0 + TILE, N);
            const size_t isz = i1 - i0, jsz = j1 - j0;
            for (size_t r = 0; r < TILE; ++r) std::memset(t.c[r], 0, sizeof(t.c[r]));
            for (size_t k0 = 0; k0 < K; k0 += TILE) {
                const size_t ksz = std::min(k0 + TILE, K) - k0;
                for (size_t i = 0; i < isz; ++i) {
                    const f16* src = A + (i0 + i) * K + k0;
                    for (size_t k = 0; k < ksz; ++k) t.a[i][k] = (float)src[k];
                }
                if (B_TRANSPOSED) {
                    for (size_t j = 0; j < jsz; ++j) {
                        const f16* src = B + (j0 + j) * K + k0;
                        for (size_t k = 0; k < ksz; ++k) t.b[k][j] = (float)src[k];
                    }
                } else {
                    for (size_t k = 0; k < ksz; ++k) {
                        const f16* src = B + (k0 + k) * N + j0;
                        for (size_t j = 0; j < jsz; ++j) t.b[k][j] = (float)src[j];
                    }
                }
                tile_fma(t, isz, jsz, ksz);
            }
            for (size_t i = 0; i < isz; ++i) {
                f16* dst = C + (i0 + i) * N + j0;
                for (size_t j = 0; j < jsz; ++j) dst[j] = (f16)t.c[i][j];
            }
        }
    });
}

inline v8f load8_f16(const f16* p) {
    v8f r;
    for (int i = 0; i < 8; ++i) r[i] = (float)p[i];
    return r;
}

inline float hsum(v8f v) {
    float s = 0.f;
    for (int i = 0; i < 8; ++i) s += v[i];
    return s;
}

// hgemm_trans.zig:55-118 — one output element: four independent 8-lane FMA
// accumulators over k in steps of 32, a scalar tail, then one horizontal add.
inline f16 gemv_row(const f16* a, const f16* row, size_t K) {
    v8f acc0 = {0, 0, 0, 0, 0, 0, 0, 0}, acc1 = acc0, acc2 = acc0, acc3 = acc0;
    const size_t k_aligned = K - (K % 32);
    size_t k = 0;
    for (; k < k_aligned; k += 32) {
        acc0 = load8_f16(a + k) * load8_f16(row + k) + acc0;
        acc1 = load8_f16(a + k + 8) * load8_f16(row + k + 8) + acc1;
        acc2 = load8_f16(a + k + 16) * load8_f16(row + k + 16) + acc2;
        acc3 = load8_f16(a + k + 24) * load8_f16(row + k + 24) + acc3;
    }
    float tail = 0.f;
    for (; k < K; ++k) tail += (float)a[k] * (float)row[k];
    return (f16)(hsum(acc0 + acc1 + acc2 + acc3) + tail);
}

// sgemm_inplace.zig:92-322 — f32 tiled GEMM with the same 8x8 micro-kernel.
void sgemm_tiled(const float* A, const float* B, float* C, size_t M, size_t N, size_t K, int threads) {
    std::memset(C, 0, M * N * sizeof(float));
    constexpr size_t T = 168;  // sgemm_inplace.zig:15-18
    const size_t tiles_m = (M + T - 1) / T, tiles_n = (N + T - 1) / T, total = tiles_m * tiles_n;
    std::atomic<size_t> next{0};
    spawn_join(threads, [&](int) {
        std::vector<float> accbuf(T * T);
        for (;;) {
            size_t idx = next.fetch_add(1);
            if (idx >= total) break;
            const size_t i0 = (idx / tiles_n) * T, j0 = (idx % tiles_n) * T;
            const size_t isz = std::min(i0 + T, M) - i0, jsz = std::min(j0 + T, N) - j0;
            std::fill(accbuf.begin(), accbuf.end(), 0.f);
            for (size_t k0 = 0; k0 < K; k0 += T) {
                const size_t ksz = std::min(k0 + T, K) - k0;
                for (size_t i = 0; i < isz; ++i) {
                    const float* arow = A + (i0 + i) * K + k0;
                    float* crow = accbuf.data() + i * T;
                    for (size_t k = 0; k < ksz; ++k) {
                        const float s = arow[k];
                        const float* brow = B + (k0 + k) * N + j0;
                        for (size_t j = 0; j < jsz; ++j) crow[j] = std::fma(s, brow[j], crow[j]);
                    }
                }
            }
            for (size_t i = 0; i < isz; ++i)
                for (size_t j = 0; j < jsz; ++j) C[(i0 + i) * N + j0 + j] = accbuf[i * T + j];
        }
    });
}

void softmax_rows(float* data, size_t rows, size_t cols) {
    std::vector<float> e(cols);
    for (size_t r = 0; r < rows; ++r) {
        float* row = data + r * cols;
        float mx = row[0];
        for (size_t i = 1; i < cols; ++i)
            if (row[i] > mx) mx = row[i];
        float sum = 0.f;
        for (size_t i = 0; i < cols; ++i) {
            const float v = row[i] - mx;
            e[i] = (v > -88.0f) ? std::exp(v) : 0.f;
            sum += e[i];
        }
        if (sum > 0.f) {
            const float inv = 1.0f / sum;
            for (size_t i = 0; i < cols; ++i) row[i] = e[i] * inv;
        }
    }
}

// attention.zig:125-234 (mask == nullptr) and :416-541 (mask given): whole
// q,k,v widened to f32, K transposed to [h,d,kv], per head two f32 GEMMs around
// a scaled (then masked) row softmax, f16 rounding of the output only.
void sdpa_multi(const f16* q, const f16* k, const f16* v, const uint8_t* mask, f16* out, size_t n_heads,
                size_t q_len, size_t kv_len, size_t d) {
    const float scale = 1.0f / std::sqrt((float)d);
    const int cpus = worker_count();
    int head_threads = (int)std::min<size_t>(std::max<size_t>(n_heads / 2, 1), std::max(cpus / 2, 1));
    const int inner = std::max(1, cpus / head_threads);
    std::atomic<size_t> next{0};
    spawn_join(head_threads, [&](int) {
        std::vector<float> qh(q_len * d), kt(d * kv_len), vh(kv_len * d), w(q_len * kv_len), oh(q_len * d);
        for (;;) {
            const size_t h = next.fetch_add(1);
            if (h >= n_heads) break;
            const f16* qs = q + h * q_len * d;
            const f16* ks = k + h * kv_len * d;
            const f16* vs = v + h * kv_len * d;
            for (size_t i = 0; i < q_len * d; ++i) qh[i] = (float)qs[i];
            for (size_t i = 0; i < kv_len * d; ++i) vh[i] = (float)vs[i];
            for (size_t t = 0; t < kv_len; ++t)
                for (size_t c = 0; c < d; ++c) kt[c * kv_len + t] = (float)ks[t * d + c];
            sgemm_tiled(qh.data(), kt.data(), w.data(), q_len, kv_len, d, inner);
            for (auto& x : w) x *= scale;
            if (mask) {
                for (size_t i = 0; i < q_len; ++i)
                    for (size_t j = 0; j < kv_len; ++j)
                        if (!mask[i * kv_len + j]) w[i * kv_len + j] = -std::numeric_limits<float>::infinity();
            }
            softmax_rows(w.data(), q_len, kv_len);
            sgemm_tiled(w.data(), vh.data(), oh.data(), q_len, d, kv_len, inner);
            f16* os = out + h * q_len * d;
            for (size_t i = 0; i < q_len * d; ++i) os[i] = (f16)oh[i];
        }
    });
}

constexpr size_t SINGLE_HEADS = 32, SINGLE_DIM = 64, SINGLE_MAX_KV = 2048;  // attention.zig:248-253

void layernorm_rows(const f16* x, const f16* w, const f16* b, f16* y, size_t rows, size_t cols, float eps) {
    // ops.zig:1152-1419.  The reference keeps 64 lane-parallel Welford states seeded with
    // 100000 "fake zeros" (so the running reciprocal can be refined by Newton steps), merges
    // them pairwise and subtracts the fake zeros at the end.  Here each of the 64 lanes runs a
    // plain Welford update and the lanes are merged pairwise with the same merge formula; the
    // mean and biased variance agree to f32 rounding.
    constexpr int LANES = 64;
    for (size_t r = 0; r < rows; ++r) {
        const f16* xr = x + r * cols;
        float cnt[LANES], mean[LANES], m2[LANES];
        for (int l = 0; l < LANES; ++l) cnt[l] = mean[l] = m2[l] = 0.f;
        for (size_t i = 0; i < cols; ++i) {
            const int l = (int)(i % LANES);
            const float v = (float)xr[i];
            cnt[l] += 1.f;
            const float delta = v - mean[l];
            mean[l] += delta / cnt[l];
            m2[l] += delta * (v - mean[l]);
        }
        for (int step = 1; step < LANES; step *= 2) {
            for (int l = 0; l + step < LANES; l += 2 * step) {
                const float na = cnt[l], nb = cnt[l + step], n = na + nb;
                if (n == 0.f) continue;
                const float delta = mean[l + step] - mean[l];
                mean[l] += delta * (nb / n);
                m2[l] += m2[l + step] + delta * delta * (na * nb / n);
                cnt[l] = n;
            }
        }
        const float variance = m2[0] / cnt[0];
        const float rstd = 1.0f / std::sqrt(variance + eps);
        const float mean_rstd = mean[0] * rstd;
        f16* yr = y + r * cols;
        for (size_t i = 0; i < cols; ++i) {
            const float n = (float)xr[i] * rstd - mean_rstd;
            yr[i] = (f16)(n * (float)w[i] + (float)b[i]);
        }
    }
}

void gelu_inplace(f16* x, size_t n) {
    // ops.zig:1641-1642: both constants are f16 values in the reference.
    auto r16 = [](float v) { return (float)(f16)v; };
    const float c = r16(std::sqrt(r16(2.0f / r16(3.14159265358979323846f))));
    const float a = r16(0.044715f);
    auto body = [&](size_t lo, size_t hi) {
        for (size_t i = lo; i < hi; ++i) {
            const float v = (float)x[i];
            const float inner = c * (v + a * (v * v * v));
            x[i] = (f16)(0.5f * v * (1.0f + std::tanh(inner)));
        }
    };
    if (n < (1u << 16)) { body(0, n); return; }
    const int nt = worker_count();
    const size_t chunk = (n + nt - 1) / nt;
    spawn_join(nt, [&](int t) { body(std::min(n, t * chunk), std::min(n, (t + 1) * chunk)); });
}

void bias_add(f16* a, const f16* b, size_t rows, size_t cols) {
    for (size_t r = 0; r < rows; ++r) {
        f16* ar = a + r * cols;
        for (size_t j = 0; j < cols; ++j) ar[j] = (f16)((float)ar[j] + (float)b[j]);
    }
}

void add_inplace(f16* a, const f16* b, size_t n) {
    for (size_t i = 0; i < n; ++i) a[i] = (f16)((float)a[i] + (float)b[i]);
}

void rope_table(float* table, size_t dim, size_t end, float theta) {
    const size_t half = dim / 2;
    std::vector<float> freqs(half);
    for (size_t i = 0; i < half; ++i) freqs[i] = 1.0f / std::pow(theta, (float)(2 * i) / (float)dim);
    for (size_t p = 0; p < end; ++p)
        for (size_t j = 0; j < half; ++j) {
            const float ang = (float)p * freqs[j];
            table[(p * half + j) * 2] = std::cos(ang);
            table[(p * half + j) * 2 + 1] = std::sin(ang);
        }
}

void rope_apply(const f16* x, f16* out, size_t n_heads, size_t seq_len, size_t head_dim, const float* freqs,
                const size_t* pos, size_t rot_dim) {
    const size_t half = rot_dim / 2;
    for (size_t h = 0; h < n_heads; ++h)
        for (size_t s = 0; s < seq_len; ++s) {
            const size_t base = (h * seq_len + s) * head_dim;
            const float* f = freqs + pos[s] * half * 2;
            for (size_t j = 0; j < half; ++j) {
                const float xr = (float)x[base + j], xi = (float)x[base + half + j];
                const float c = f[2 * j], sn = f[2 * j + 1];
                out[base + j] = (f16)(xr * c - xi * sn);
                out[base + half + j] = (f16)(xr * sn + xi * c);
            }
            for (size_t j = rot_dim; j < head_dim; ++j) out[base + j] = x[base + j];
        }
}

// [S, n_heads*d] (one chunk of a [S, row_stride] matrix at column col0) -> [n_heads, S, d]
void split_heads(const f16* src, size_t row_stride, size_t col0, f16* dst, size_t S, size_t n_heads, size_t d) {
    for (size_t s = 0; s < S; ++s)
        for (size_t h = 0; h < n_heads; ++h)
            std::memcpy(dst + (h * S + s) * d, src + s * row_stride + col0 + h * d, d * sizeof(f16));
}

// [n_heads, S, d] -> [S, n_heads*d]
void merge_heads(const f16* src, f16* dst, size_t S, size_t n_heads, size_t d) {
    for (size_t s = 0; s < S; ++s)
        for (size_t h = 0; h < n_heads; ++h)
            std::memcpy(dst + s * n_heads * d + h * d, src + (h * S + s) * d, d * sizeof(f16));
}

}  // namespace

extern "C" {

void orc_set_threads(int n) { g_threads.store(n); }
int orc_get_threads(void) { return worker_count(); }

int orc_hgemm_nn(const uint16_t* a, const uint16_t* b, uint16_t* c, size_t M, size_t N, size_t K) {
    if (!a || !b || !c) return ORC_ERR_INVALID_ARG;
    hgemm_tiled<false>(H(a), H(b), H(c), M, N, K);
    return ORC_OK;
}

int orc_hgemm_nt(const uint16_t* a, const uint16_t* b_t, uint16_t* c, size_t M, size_t N, size_t K) {
    if (!a || !b_t || !c) return ORC_ERR_INVALID_ARG;
    if (M == 1) {
        // hgemm_trans.zig:430-455 — work items of 32 consecutive outputs.
        const f16 *A = H(a), *B = H(b_t);
        f16* C = H(c);
        const size_t chunk = 32, total = (N + chunk - 1) / chunk;
        std::atomic<size_t> next{0};
        spawn_join(worker_count(), [&](int) {
            for (;;) {
                const size_t ci = next.fetch_add(1);
                if (ci >= total) break;
                const size_t n1 = std::min(ci * chunk + chunk, N);
                for (size_t n = ci * chunk; n < n1; ++n) C[n] = gemv_row(A, B + n * K, K);
            }
        });
        return ORC_OK;
    }
    hgemm_tiled<true>(H(a), H(b_t), H(c), M, N, K);
    return ORC_OK;
}

int orc_naive_matmul_f16(const uint16_t* a, const uint16_t* b, uint16_t* c, size_t M, size_t N, size_t K) {
    const f16 *A = H(a), *B = H(b);
    f16* C = H(c);
    for (size_t i = 0; i < M; ++i)
        for (size_t j = 0; j < N; ++j) {
            volatile float sum = 0.f;  // volatile: keep mul and add separately rounded, in k order
            for (size_t k = 0; k < K; ++k) {
                volatile float p = (float)A[i * K + k] * (float)B[k * N + j];
                sum = sum + p;
            }
            C[i * N + j] = (f16)sum;
        }
    return ORC_OK;
}

int orc_sgemm(const float* a, const float* b, float* c, size_t M, size_t N, size_t K) {
    if (!a || !b || !c) return ORC_ERR_INVALID_ARG;
    sgemm_tiled(a, b, c, M, N, K, worker_count());
    return ORC_OK;
}

int orc_softmax_rows(float* data, size_t rows, size_t cols) {
    if (!data || cols == 0) return ORC_ERR_INVALID_ARG;
    softmax_rows(data, rows, cols);
    return ORC_OK;
}

int orc_sdpa_maskless(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* out, size_t n_heads,
                      size_t q_len, size_t kv_len, size_t head_dim) {
    if (!q || !k || !v || !out || !n_heads || !q_len || !kv_len || !head_dim) return ORC_ERR_INVALID_ARG;
    sdpa_multi(H(q), H(k), H(v), nullptr, H(out), n_heads, q_len, kv_len, head_dim);
    return ORC_OK;
}

int orc_create_attention_mask(uint8_t* mask, size_t pos, size_t seq_len) {
    if (!mask) return ORC_ERR_INVALID_ARG;
    const size_t w = pos + seq_len;
    for (size_t i = 0; i < seq_len; ++i) {
        for (size_t j = 0; j < pos; ++j) mask[i * w + j] = 1;
        for (size_t j = 0; j < seq_len; ++j) mask[i * w + pos + j] = (j <= i) ? 1 : 0;
    }
    return ORC_OK;
}

int orc_sdpa_masked(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint8_t* mask, uint16_t* out,
                    size_t n_heads, size_t q_len, size_t kv_len, size_t head_dim) {
    if (!q || !k || !v || !mask || !out || !n_heads || !q_len || !kv_len || !head_dim) return ORC_ERR_INVALID_ARG;
    sdpa_multi(H(q), H(k), H(v), mask, H(out), n_heads, q_len, kv_len, head_dim);
    return ORC_OK;
}

int orc_sdpa_single(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint8_t* mask, uint16_t* out,
                    size_t kv_len) {
    if (!q || !k || !v || !mask || !out || kv_len == 0) return ORC_ERR_INVALID_ARG;
    if (kv_len > SINGLE_MAX_KV) return ORC_ERR_SEQUENCE_TOO_LONG;
    const f16 *Q = H(q), *Kp = H(k), *V = H(v);
    f16* O = H(out);
    const float scale = 1.0f / std::sqrt((float)SINGLE_DIM);
    const int nt = (int)std::min<size_t>(SINGLE_HEADS, (size_t)worker_count());
    std::atomic<size_t> next{0};
    spawn_join(nt, [&](int) {
        std::vector<float> scores(SINGLE_MAX_KV);
        alignas(32) float acc[SINGLE_DIM];
        for (;;) {
            const size_t h = next.fetch_add(1);
            if (h >= SINGLE_HEADS) break;
            const f16* qh = Q + h * SINGLE_DIM;
            const f16* kh = Kp + h * kv_len * SINGLE_DIM;
            const f16* vh = V + h * kv_len * SINGLE_DIM;
            for (size_t j = 0; j < kv_len; ++j) {
                float sum = 0.f;
                for (size_t c = 0; c < SINGLE_DIM; c += 8) sum += hsum(load8_f16(qh + c) * load8_f16(kh + j * SINGLE_DIM + c));
                scores[j] = mask[j] ? sum * scale : -std::numeric_limits<float>::infinity();
            }
            float mx = scores[0];
            for (size_t j = 1; j < kv_len; ++j) mx = std::max(mx, scores[j]);
            float sum = 0.f;
            for (size_t j = 0; j < kv_len; ++j) {
                scores[j] = std::exp(scores[j] - mx);
                sum += scores[j];
            }
            const float inv = 1.0f / sum;
            for (size_t j = 0; j < kv_len; ++j) scores[j] *= inv;
            for (size_t c = 0; c < SINGLE_DIM; ++c) acc[c] = 0.f;
            for (size_t j = 0; j < kv_len; ++j) {
                const float wgt = scores[j];
                for (size_t c = 0; c < SINGLE_DIM; ++c) acc[c] += (float)vh[j * SINGLE_DIM + c] * wgt;
            }
            for (size_t c = 0; c < SINGLE_DIM; ++c) O[h * SINGLE_DIM + c] = (f16)acc[c];
        }
    });
    return ORC_OK;
}

int orc_rope_table(float* table, size_t dim, size_t end, float theta) {
    if (!table || dim == 0 || (dim & 1) || end == 0 || !(theta > 0.f)) return ORC_ERR_INVALID_ARG;
    rope_table(table, dim, end, theta);
    return ORC_OK;
}

int orc_rope_apply(const uint16_t* x, uint16_t* out, size_t n_heads, size_t seq_len, size_t head_dim,
                   const float* freqs_cis, size_t freqs_half, const size_t* position_ids, size_t rot_dim) {
    if (!x || !out || !freqs_cis || !position_ids) return ORC_ERR_INVALID_DIMENSION;
    if (rot_dim != freqs_half * 2 || rot_dim > head_dim) return ORC_ERR_INVALID_ROT_DIM;
    rope_apply(H(x), H(out), n_heads, seq_len, head_dim, freqs_cis, position_ids, rot_dim);
    return ORC_OK;
}

int orc_layernorm(const uint16_t* x, const uint16_t* w, const uint16_t* b, uint16_t* y, size_t rows, size_t cols,
                  uint16_t eps_f16) {
    if (!x || !w || !b || !y || cols == 0) return ORC_ERR_INVALID_ARG;
    const float eps = h2f(eps_f16);
    if (!(eps > 0.f)) return ORC_ERR_INVALID_ARG;
    layernorm_rows(H(x), H(w), H(b), H(y), rows, cols, eps);
    return ORC_OK;
}

int orc_gelu(uint16_t* x, size_t n) {
    if (!x) return ORC_ERR_INVALID_ARG;
    gelu_inplace(H(x), n);
    return ORC_OK;
}

int orc_bias_add(uint16_t* a, const uint16_t* b, size_t rows, size_t cols) {
    if (!a || !b) return ORC_ERR_INVALID_ARG;
    bias_add(H(a), H(b), rows, cols);
    return ORC_OK;
}

int orc_add(uint16_t* a, const uint16_t* b, size_t n) {
    if (!a || !b) return ORC_ERR_INVALID_ARG;
    add_inplace(H(a), H(b), n);
    return ORC_OK;
}

int orc_argmax_f16(const uint16_t* x, size_t n, size_t* idx_out) {
    if (!x || !idx_out || n == 0) return ORC_ERR_INVALID_ARG;
    size_t best = 0;
    float bv = h2f(x[0]);
    for (size_t i = 0; i < n; ++i) {
        const float v = h2f(x[i]);
        if (v > bv) { bv = v; best = i; }
    }
    *idx_out = best;
    return ORC_OK;
}

int orc_kv_update(uint16_t* key_cache, uint16_t* value_cache, const uint16_t* k_new, const uint16_t* v_new,
                  size_t n_heads, size_t max_seq, size_t head_dim, size_t cur_len, size_t seq_len) {
    if (!key_cache || !value_cache || !k_new || !v_new) return ORC_ERR_INVALID_ARG;
    if (cur_len + seq_len > max_seq) return ORC_ERR_SEQUENCE_TOO_LONG;
    for (size_t h = 0; h < n_heads; ++h) {
        const size_t dst = (h * max_seq + cur_len) * head_dim, src = h * seq_len * head_dim;
        std::memcpy(key_cache + dst, k_new + src, seq_len * head_dim * 2);
        std::memcpy(value_cache + dst, v_new + src, seq_len * head_dim * 2);
    }
    return ORC_OK;
}

int orc_kv_active(const uint16_t* key_cache, const uint16_t* value_cache, uint16_t* k_out, uint16_t* v_out,
                  size_t n_heads, size_t max_seq, size_t head_dim, size_t cur_len) {
    if (!key_cache || !value_cache || !k_out || !v_out) return ORC_ERR_INVALID_ARG;
    if (cur_len > max_seq) return ORC_ERR_SEQUENCE_TOO_LONG;
    for (size_t h = 0; h < n_heads; ++h) {
        std::memcpy(k_out + h * cur_len * head_dim, key_cache + h * max_seq * head_dim, cur_len * head_dim * 2);
        std::memcpy(v_out + h * cur_len * head_dim, value_cache + h * max_seq * head_dim, cur_len * head_dim * 2);
    }
    return ORC_OK;
}

int orc_preprocess_patchify(const uint8_t* img, uint16_t* out, size_t crops, size_t height, size_t width,
                            size_t patch) {
    if (!img || !out || patch == 0 || height % patch || width % patch) return ORC_ERR_INVALID_ARG;
    const size_t hp = height / patch, wp = width / patch, pd = 3 * patch * patch;
    f16* O = H(out);
    const f16 k255 = (f16)255.0f, half = (f16)0.5f;
    for (size_t b = 0; b < crops; ++b)
        for (size_t y = 0; y < height; ++y)
            for (size_t x = 0; x < width; ++x)
                for (size_t c = 0; c < 3; ++c) {
                    f16 v = (f16)(float)img[((b * height + y) * width + x) * 3 + c];
                    v = (f16)((float)v / (float)k255);             // vision_model.zig:167-169, f16 divide
                    v = (f16)(((float)v - (float)half));           // reshape_handler.zig:89 (v - mean) ...
                    v = (f16)((float)v / (float)half);             // ... / std, each f16 op rounds
                    const size_t pidx = (y / patch) * wp + (x / patch);
                    const size_t e = (c * patch + (y % patch)) * patch + (x % patch);
                    O[(b * hp * wp + pidx) * pd + e] = v;
                }
    return ORC_OK;
}

int orc_text_decoder(const orc_text_weights* w, uint16_t* hidden_io, size_t S, uint16_t* const* key_cache,
                     uint16_t* const* value_cache, size_t cur_len) {
    if (!w || !hidden_io || !key_cache || !value_cache || S == 0) return ORC_ERR_INVALID_ARG;
    const size_t D = w->dim, Hh = w->n_heads, d = w->head_dim, F = w->hidden, rot = d / 2;
    if (cur_len + S > w->max_seq) return ORC_ERR_SEQUENCE_TOO_LONG;
    const uint16_t eps = f2h(1e-5f);  // text_model.zig:28
    std::vector<float> freqs(w->max_seq * (rot / 2) * 2);
    rope_table(freqs.data(), rot, w->max_seq, 10000.0f);  // text_model.zig:88
    std::vector<size_t> pos(S);
    for (size_t i = 0; i < S; ++i) pos[i] = cur_len + i;
    const size_t kv_len = cur_len + S;
    std::vector<uint16_t> ln(S * D), qkv(S * 3 * D), q(S * D), k(S * D), v(S * D), qr(S * D), kr(S * D),
        ka(Hh * kv_len * d), va(Hh * kv_len * d), att(S * D), attm(S * D), attn_out(S * D), fc1(S * F), mlp_out(S * D);
    std::vector<uint8_t> mask(S * kv_len);
    for (size_t l = 0; l < w->n_layers; ++l) {
        orc_layernorm(hidden_io, w->ln_w[l], w->ln_b[l], ln.data(), S, D, eps);
        // attention_block, text_model.zig:182-301
        orc_hgemm_nt(ln.data(), w->wqkv[l], qkv.data(), S, 3 * D, D);
        orc_bias_add(qkv.data(), w->bqkv[l], S, 3 * D);
        split_heads(H(qkv.data()), 3 * D, 0, H(q.data()), S, Hh, d);
        split_heads(H(qkv.data()), 3 * D, D, H(k.data()), S, Hh, d);
        split_heads(H(qkv.data()), 3 * D, 2 * D, H(v.data()), S, Hh, d);
        rope_apply(H(q.data()), H(qr.data()), Hh, S, d, freqs.data(), pos.data(), rot);
        rope_apply(H(k.data()), H(kr.data()), Hh, S, d, freqs.data(), pos.data(), rot);
        orc_kv_update(key_cache[l], value_cache[l], kr.data(), v.data(), Hh, w->max_seq, d, cur_len, S);
        orc_kv_active(key_cache[l], value_cache[l], ka.data(), va.data(), Hh, w->max_seq, d, kv_len);
        orc_create_attention_mask(mask.data(), cur_len, S);
        int rc;
        if (S == 1) rc = orc_sdpa_single(qr.data(), ka.data(), va.data(), mask.data(), att.data(), kv_len);
        else rc = orc_sdpa_masked(qr.data(), ka.data(), va.data(), mask.data(), att.data(), Hh, S, kv_len, d);
        if (rc) return rc;
        merge_heads(H(att.data()), H(attm.data()), S, Hh, d);
        orc_hgemm_nt(attm.data(), w->wout[l], attn_out.data(), S, D, D);
        orc_bias_add(attn_out.data(), w->bout[l], S, D);
        // mlp on the same LayerNorm output, text_model.zig:304-323
        orc_hgemm_nt(ln.data(), w->wfc1[l], fc1.data(), S, F, D);
        orc_bias_add(fc1.data(), w->bfc1[l], S, F);
        orc_gelu(fc1.data(), S * F);
        orc_hgemm_nt(fc1.data(), w->wfc2[l], mlp_out.data(), S, D, F);
        orc_bias_add(mlp_out.data(), w->bfc2[l], S, D);
        orc_add(attn_out.data(), mlp_out.data(), S * D);  // text_model.zig:170-171
        orc_add(hidden_io, attn_out.data(), S * D);
    }
    return ORC_OK;
}

int orc_lm_head(const orc_text_weights* w, const uint16_t* hidden, size_t S, uint16_t* logits) {
    if (!w || !hidden || !logits || S == 0) return ORC_ERR_INVALID_ARG;
    std::vector<uint16_t> ln(w->dim);
    orc_layernorm(hidden + (S - 1) * w->dim, w->ln_out_w, w->ln_out_b, ln.data(), 1, w->dim, f2h(1e-5f));
    orc_hgemm_nt(ln.data(), w->lm_w, logits, 1, w->vocab, w->dim);
    orc_bias_add(logits, w->lm_b, 1, w->vocab);
    return ORC_OK;
}

int orc_vision_encoder(const orc_vision_weights* w, const uint16_t* patches, size_t crops, int joint_attention,
                       uint16_t* features) {
    if (!w || !patches || !features || crops == 0) return ORC_ERR_INVALID_ARG;
    const size_t T = w->tokens, D = w->dim, Hh = w->n_heads, d = w->head_dim, F = w->hidden, R = crops * T;
    const uint16_t eps = f2h(1e-5f);  // vision_model.zig:35
    std::vector<uint16_t> x(R * D), ln(R * D), qkv(R * 3 * D), q(R * D), k(R * D), v(R * D), att(R * D), attm(R * D),
        proj(R * D), fc1(R * F), fc2(R * D);
    orc_hgemm_nn(patches, w->patch_w, x.data(), R, D, w->patch_dim);
    orc_bias_add(x.data(), w->patch_b, R, D);
    for (size_t c = 0; c < crops; ++c)  // pos_emb [1,T,D] broadcast over the crops, vision_model.zig:228
        for (size_t t = 0; t < T; ++t) orc_bias_add(x.data() + (c * T + t) * D, w->pos_emb + t * D, 1, D);
    for (size_t l = 0; l < w->n_layers; ++l) {
        orc_layernorm(x.data(), w->ln1_w[l], w->ln1_b[l], ln.data(), R, D, eps);
        orc_hgemm_nn(ln.data(), w->wqkv[l], qkv.data(), R, 3 * D, D);
        orc_bias_add(qkv.data(), w->bqkv[l], R, 3 * D);
        const size_t groups = joint_attention ? 1 : crops, L = joint_attention ? R : T;
        for (size_t g = 0; g < groups; ++g) {
            const f16* base = H(qkv.data()) + g * L * 3 * D;
            split_heads(base, 3 * D, 0, H(q.data()), L, Hh, d);
            split_heads(base, 3 * D, D, H(k.data()), L, Hh, d);
            split_heads(base, 3 * D, 2 * D, H(v.data()), L, Hh, d);
            orc_sdpa_maskless(q.data(), k.data(), v.data(), att.data(), Hh, L, L, d);
            merge_heads(H(att.data()), H(attm.data()) + g * L * D, L, Hh, d);
        }
        orc_hgemm_nn(attm.data(), w->wout[l], proj.data(), R, D, D);
        orc_bias_add(proj.data(), w->bout[l], R, D);
        orc_add(x.data(), proj.data(), R * D);
        orc_layernorm(x.data(), w->ln2_w[l], w->ln2_b[l], ln.data(), R, D, eps);
        orc_hgemm_nn(ln.data(), w->wfc1[l], fc1.data(), R, F, D);
        orc_bias_add(fc1.data(), w->bfc1[l], R, F);
        orc_gelu(fc1.data(), R * F);
        orc_hgemm_nn(fc1.data(), w->wfc2[l], fc2.data(), R, D, F);
        orc_bias_add(fc2.data(), w->bfc2[l], R, D);
        orc_add(x.data(), fc2.data(), R * D);
    }
    orc_layernorm(x.data(), w->norm_w, w->norm_b, features, R, D, eps);
    return ORC_OK;
}

int orc_vision_projection(const orc_vision_weights* w, const uint16_t* feat_a, const uint16_t* feat_b,
                          uint16_t* out) {
    if (!w || !feat_a || !feat_b || !out) return ORC_ERR_INVALID_ARG;
    const size_t T = w->tokens, D = w->dim;
    std::vector<uint16_t> cat(T * 2 * D), fc1(T * w->proj_hidden);
    for (size_t t = 0; t < T; ++t) {
        std::memcpy(cat.data() + t * 2 * D, feat_a + t * D, D * 2);
        std::memcpy(cat.data() + t * 2 * D + D, feat_b + t * D, D * 2);
    }
    orc_hgemm_nn(cat.data(), w->proj_fc1_w, fc1.data(), T, w->proj_hidden, 2 * D);
    orc_bias_add(fc1.data(), w->proj_fc1_b, T, w->proj_hidden);
    orc_gelu(fc1.data(), T * w->proj_hidden);
    orc_hgemm_nn(fc1.data(), w->proj_fc2_w, out, T, w->proj_out, w->proj_hidden);
    orc_bias_add(out, w->proj_fc2_b, T, w->proj_out);
    return ORC_OK;
}

}  // extern "C"
