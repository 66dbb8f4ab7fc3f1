// loom_oracle.cpp -- CPU restatement of Loom's BitNet ternary x int8 linear path.
//
// TEST INFRASTRUCTURE ONLY: the checker for the CUDA path (see loom_oracle.h).
// Build with -ffp-contract=off so that no multiply-add is fused: the reference is
// Go on amd64, which never fuses.  Reference citations are in loom_oracle.h.

#include "loom_oracle.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

#if defined(__x86_64__)
#include <immintrin.h>
#endif
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>

namespace {

// Minimal persistent worker pool (the goroutine fan-out stand-in).  parallel_chunks(n, workers, f)
// runs f(i) for i in [0,n) on up to `workers` threads (the caller is one of them) and returns when
// all are done.  Work items are handed out dynamically; callers that need the reference's static
// row partition encode it in what item i means.
class Pool {
  public:
    static Pool& get() {
        static Pool p;
        return p;
    }
    void run(int n, int workers, const std::function<void(int)>& f) {
        if (n <= 0) return;
        if (workers <= 1 || n == 1) {
            for (int i = 0; i < n; ++i) f(i);
            return;
        }
        std::unique_lock<std::mutex> outer(run_mu_);  // one parallel region at a time
        ensure(workers - 1);
        {
            std::lock_guard<std::mutex> lk(mu_);
            fn_ = &f;
            total_ = n;
            next_ = 0;
            done_ = 0;
            active_limit_ = workers - 1;
            ++epoch_;
        }
        cv_.notify_all();
        work();
        std::unique_lock<std::mutex> lk(mu_);
        done_cv_.wait(lk, [&] { return done_ == total_; });
        fn_ = nullptr;
    }

  private:
    Pool() = default;
    ~Pool() {
        {
            std::lock_guard<std::mutex> lk(mu_);
            stop_ = true;
        }
        cv_.notify_all();
        for (auto& t : threads_) t.join();
    }
    void ensure(int n) {
        while ((int)threads_.size() < n) {
            int id = (int)threads_.size();
            threads_.emplace_back([this, id] { loop(id); });
        }
    }
    void work() {
        for (;;) {
            int i;
            const std::function<void(int)>* f;
            {
                std::lock_guard<std::mutex> lk(mu_);
                if (!fn_ || next_ >= total_) return;
                i = next_++;
                f = fn_;
            }
            (*f)(i);
            {
                std::lock_guard<std::mutex> lk(mu_);
                if (++done_ == total_) done_cv_.notify_all();
            }
        }
    }
    void loop(int id) {
        unsigned long seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return stop_ || epoch_ != seen; });
                if (stop_) return;
                seen = epoch_;
                if (id >= active_limit_) continue;
            }
            work();
        }
    }
    std::mutex run_mu_, mu_;
    std::condition_variable cv_, done_cv_;
    std::vector<std::thread> threads_;
    const std::function<void(int)>* fn_ = nullptr;
    int total_ = 0, next_ = 0, done_ = 0, active_limit_ = 0;
    unsigned long epoch_ = 0;
    bool stop_ = false;
};

// Row fan-out rule of the reference: single thread below 262144 multiply-adds or
// fewer than 4 rows, otherwise contiguous chunks of ceil(rows/workers) rows.
template <class F>
void run_rows(int rows, int cols, int threads, F&& body) {
    long long work = (long long)rows * (long long)cols;
    int workers = threads;
    if (workers > rows) workers = rows;
    if (work < 262144 || rows < 4 || workers <= 1) {
        body(0, rows);
        return;
    }
    int chunk = (rows + workers - 1) / workers;
    int nchunks = (rows + chunk - 1) / chunk;
    Pool::get().run(nchunks, workers, [&](int c) {
        int s = c * chunk;
        int e = std::min(rows, s + chunk);
        body(s, e);
    });
}

inline uint32_t code_of(int q) { return q < 0 ? 0u : (q > 0 ? 2u : 1u); }

inline bool near_ternary(float v) {
    return std::fabs((double)v) < 1e-6 || std::fabs((double)(v - 1.0f)) < 1e-6 ||
           std::fabs((double)(v + 1.0f)) < 1e-6;
}

double now_s() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

}  // namespace

struct orc_matrix {
    int rows = 0, cols = 0, row_words = 0;
    float scale = 1.0f;
    std::vector<uint32_t> words;
    // byte-code cache for the AVX2 MAD path (one unsigned code per weight, rows padded to 32)
    std::vector<uint8_t> codes;
    int row_stride = 0;
};

extern "C" {

float orc_ternary_scale(const float* w, size_t n) {
    if (n == 0) return 1.0f;
    double sum = 0.0;
    for (size_t i = 0; i < n; ++i) sum += std::fabs((double)w[i]);
    float s = (float)(sum / (double)n);
    return s == 0.0f ? 1.0f : s;
}

int orc_quant_value(float v, float scale) {
    if (scale == 0.0f) scale = 1.0f;
    float ratio = v / scale;  // float32 division, as in the reference
    long q = (long)std::round((double)ratio);
    if (q > 1) q = 1;
    if (q < -1) q = -1;
    return (int)q;
}

int orc_row_words(int cols) { return (cols + 15) / 16; }

int orc_pack_native(const int8_t* q, int rows, int cols, uint32_t* words) {
    if (rows <= 0 || cols <= 0) return -1;
    int rw = orc_row_words(cols);
    std::memset(words, 0, sizeof(uint32_t) * (size_t)rows * rw);
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c)
            words[(size_t)r * rw + c / 16] |= code_of(q[(size_t)r * cols + c]) << (2 * (c % 16));
    return 0;
}

int orc_pack_f32(const float* w, int rows, int cols, uint32_t* words, float* scale_out) {
    if (rows <= 0 || cols <= 0) return -1;
    size_t total = (size_t)rows * cols;
    float scale = orc_ternary_scale(w, total);
    std::vector<int8_t> q(total);
    bool already = true;
    for (size_t i = 0; i < total; ++i) {
        if (!near_ternary(w[i])) already = false;
        q[i] = (int8_t)orc_quant_value(w[i], scale);
    }
    if (already) {
        scale = 1.0f;
        for (size_t i = 0; i < total; ++i) q[i] = (int8_t)orc_quant_value(w[i], 1.0f);
    }
    orc_pack_native(q.data(), rows, cols, words);
    if (scale_out) *scale_out = scale;
    return 0;
}

float orc_morph_ternary(const float* w, size_t n, int8_t* q) {
    float scale = orc_ternary_scale(w, n);
    for (size_t i = 0; i < n; ++i) q[i] = (int8_t)orc_quant_value(w[i], scale);
    return scale;
}

static void ms_scatter(uint8_t b, int pr, int c, int packed_rows, int rw, uint32_t* words) {
    for (int lane = 0; lane < 4; ++lane) {
        uint32_t code = (b >> (2 * lane)) & 3u;
        if (code > 2) code = 1;
        int row = lane * packed_rows + pr;
        words[(size_t)row * rw + c / 16] |= code << (2 * (c % 16));
    }
}

int orc_pack_microsoft_u8(const uint8_t* packed, int rows, int cols, uint32_t* words) {
    if (rows <= 0 || cols <= 0 || rows % 4 != 0) return -1;
    int rw = orc_row_words(cols), pr_n = rows / 4;
    std::memset(words, 0, sizeof(uint32_t) * (size_t)rows * rw);
    for (int pr = 0; pr < pr_n; ++pr)
        for (int c = 0; c < cols; ++c) ms_scatter(packed[(size_t)pr * cols + c], pr, c, pr_n, rw, words);
    return 0;
}

int orc_pack_microsoft_f32slots(const float* packed, int rows, int cols, uint32_t* words) {
    if (rows <= 0 || cols <= 0 || rows % 4 != 0) return -1;
    int rw = orc_row_words(cols), pr_n = rows / 4;
    std::memset(words, 0, sizeof(uint32_t) * (size_t)rows * rw);
    for (int pr = 0; pr < pr_n; ++pr)
        for (int c = 0; c < cols; ++c)
            ms_scatter((uint8_t)packed[(size_t)pr * cols + c], pr, c, pr_n, rw, words);
    return 0;
}

static inline int8_t quant_one(double v, double s) {
    double r = std::round(v * s);
    long q = (long)r;
    if (q < -128) q = -128;
    if (q > 127) q = 127;
    return (int8_t)q;
}

float orc_quantize_f32(const float* x, int n, int8_t* q) {
    float amax = 0.0f;
    for (int i = 0; i < n; ++i) {
        float a = (float)std::fabs((double)x[i]);
        if (a > amax) amax = a;
    }
    if (amax < 1e-5f) amax = 1e-5f;
    double s = 127.0 / (double)amax;
    for (int i = 0; i < n; ++i) q[i] = quant_one((double)x[i], s);
    return amax;
}

float orc_quantize_f64(const double* x, int n, int8_t* q) {
    float amax = 0.0f;
    for (int i = 0; i < n; ++i) {
        float a = (float)std::fabs(x[i]);
        if (a > amax) amax = a;
    }
    if (amax < 1e-5f) amax = 1e-5f;
    double s = 127.0 / (double)amax;
    for (int i = 0; i < n; ++i) q[i] = quant_one(x[i], s);
    return amax;
}

static inline int32_t row_dot_words(const uint32_t* row, int cols, const int8_t* xq) {
    int full = cols / 16, tail = cols % 16;
    int32_t sum = 0;
    const int8_t* x = xq;
    for (int w = 0; w < full; ++w, x += 16) {
        uint32_t word = row[w];
        for (int i = 0; i < 16; ++i) sum += (int32_t)x[i] * ((int32_t)((word >> (2 * i)) & 3u) - 1);
    }
    if (tail > 0) {
        uint32_t word = row[full];
        for (int i = 0; i < tail; ++i) sum += (int32_t)x[i] * ((int32_t)((word >> (2 * i)) & 3u) - 1);
    }
    return sum;
}

void orc_matvec_i32(const uint32_t* words, int rows, int cols, const int8_t* xq, int32_t* acc) {
    int rw = orc_row_words(cols);
    for (int r = 0; r < rows; ++r) acc[r] = row_dot_words(words + (size_t)r * rw, cols, xq);
}

int32_t orc_code_row_dot_scalar(const uint8_t* codes, const int8_t* acts, int nbytes) {
    int32_t s = 0;
    for (int i = 0; i < nbytes; ++i) s += (int32_t)codes[i] * (int32_t)acts[i];
    return s;
}

int orc_has_avx2(void) {
#if defined(__x86_64__)
    return __builtin_cpu_supports("avx2") ? 1 : 0;
#else
    return 0;
#endif
}

#if defined(__x86_64__)
__attribute__((target("avx2"))) static int32_t code_row_dot_avx2_impl(const uint8_t* codes, const int8_t* acts,
                                                                        int nbytes) {
    __m256i acc = _mm256_setzero_si256();
    const __m256i ones = _mm256_set1_epi16(1);
    for (int i = 0; i + 32 <= nbytes; i += 32) {
        __m256i c = _mm256_loadu_si256((const __m256i*)(codes + i));
        __m256i a = _mm256_loadu_si256((const __m256i*)(acts + i));
        __m256i p16 = _mm256_maddubs_epi16(c, a);  // u8*s8 pair sums; |.| <= 2*2*128, never saturates
        acc = _mm256_add_epi32(acc, _mm256_madd_epi16(p16, ones));
    }
    __m128i lo = _mm256_castsi256_si128(acc), hi = _mm256_extracti128_si256(acc, 1);
    __m128i s = _mm_add_epi32(lo, hi);
    s = _mm_hadd_epi32(s, s);
    s = _mm_hadd_epi32(s, s);
    return _mm_cvtsi128_si32(s);
}
#endif

int32_t orc_code_row_dot_avx2(const uint8_t* codes, const int8_t* acts, int nbytes) {
#if defined(__x86_64__)
    if (orc_has_avx2()) return code_row_dot_avx2_impl(codes, acts, nbytes);
#endif
    return orc_code_row_dot_scalar(codes, acts, nbytes);
}

double orc_gate_product(double g, double u, int activation) {
    if (activation == ORC_ACT_RELU2) {
        if (g < 0) g = 0;
        return (g * g) * u;
    }
    double sig = 1.0 / (1.0 + std::exp(-g));
    return (g * sig) * u;
}

float orc_activate_f32(float v, int act) {
    switch (act) {
        case ORC_ACT_RELU: return v < 0 ? 0.0f : v;
        case ORC_ACT_SILU: return v * (float)(1.0 / (1.0 + std::exp(-(double)v)));
        case ORC_ACT_GELU: {
            double x = (double)v;
            return (float)(0.5 * x * (1.0 + std::tanh(std::sqrt(2.0 / M_PI) * (x + 0.044715 * std::pow(x, 3)))));
        }
        case ORC_ACT_TANH: return (float)std::tanh((double)v);
        case ORC_ACT_SIGMOID: return (float)(1.0 / (1.0 + std::exp(-(double)v)));
        case ORC_ACT_LEAKY_RELU: return v < 0 ? (float)((double)v * 0.01) : v;
        case ORC_ACT_RELU2: return v < 0 ? 0.0f : v * v;
        default: return v;
    }
}

void orc_inner_rmsnorm_f32(float* data, int n, const float* weight, int wlen, double eps) {
    if (n <= 0) return;
    if (eps <= 0) eps = 1e-5;
    double ss = 0.0;
    for (int i = 0; i < n; ++i) {
        double f = (double)data[i];
        ss += f * f;
    }
    double sc = 1.0 / std::sqrt(ss / (double)n + eps);
    for (int i = 0; i < n; ++i) {
        double w = (weight && i < wlen) ? (double)weight[i] : 1.0;
        data[i] = (float)((double)data[i] * sc * w);
    }
}

void orc_inner_rmsnorm_f64(double* data, int n, const float* weight, int wlen, double eps) {
    if (n <= 0) return;
    if (eps <= 0) eps = 1e-5;
    double ss = 0.0;
    for (int i = 0; i < n; ++i) ss += data[i] * data[i];
    double sc = 1.0 / std::sqrt(ss / (double)n + eps);
    for (int i = 0; i < n; ++i) {
        double w = (weight && i < wlen) ? (double)weight[i] : 1.0;
        data[i] *= sc * w;  // data * (sc*w), the grouping of Go's `data[i] *= scale * w`
    }
}

void orc_block_rmsnorm(const float* in, int rows, int n, const float* gain, double eps, float* out, float* rms_out) {
    if (eps <= 0) eps = 1e-6;
    for (int b = 0; b < rows; ++b) {
        const float* x = in + (size_t)b * n;
        double ss = 0.0;
        for (int i = 0; i < n; ++i) {
            double v = (double)x[i];
            ss += v * v;
        }
        double rms = std::sqrt(ss / (double)n + eps);
        if (rms_out) rms_out[b] = (float)rms;
        for (int i = 0; i < n; ++i) {
            double normed = (double)x[i] / rms;
            double g = gain ? (double)gain[i] : 1.0;
            out[(size_t)b * n + i] = (float)(normed * g);
        }
    }
}

// ---- matrix object ---------------------------------------------------------------

orc_matrix* orc_matrix_from_words(const uint32_t* words, int rows, int cols, float scale) {
    if (rows <= 0 || cols <= 0) return nullptr;
    auto* m = new orc_matrix();
    m->rows = rows;
    m->cols = cols;
    m->row_words = orc_row_words(cols);
    m->scale = scale == 0.0f ? 1.0f : scale;
    m->words.assign(words, words + (size_t)rows * m->row_words);
    return m;
}

orc_matrix* orc_matrix_from_f32(const float* w, int rows, int cols) {
    if (rows <= 0 || cols <= 0) return nullptr;
    auto* m = new orc_matrix();
    m->rows = rows;
    m->cols = cols;
    m->row_words = orc_row_words(cols);
    m->words.resize((size_t)rows * m->row_words);
    orc_pack_f32(w, rows, cols, m->words.data(), &m->scale);
    return m;
}

void orc_matrix_free(orc_matrix* m) { delete m; }
int orc_matrix_rows(const orc_matrix* m) { return m->rows; }
int orc_matrix_cols(const orc_matrix* m) { return m->cols; }
int orc_matrix_row_words(const orc_matrix* m) { return m->row_words; }
float orc_matrix_scale(const orc_matrix* m) { return m->scale; }
void orc_matrix_set_scale(orc_matrix* m, float scale) { m->scale = scale == 0.0f ? 1.0f : scale; }
const uint32_t* orc_matrix_words(const orc_matrix* m) { return m->words.data(); }

static void ensure_codes(orc_matrix* m) {
    if (!m->codes.empty() && m->row_stride >= m->cols) return;
    int stride = ((m->cols + 31) / 32) * 32;
    m->codes.assign((size_t)m->rows * stride, 0);
    for (int r = 0; r < m->rows; ++r)
        for (int c = 0; c < m->cols; ++c)
            m->codes[(size_t)r * stride + c] =
                (uint8_t)((m->words[(size_t)r * m->row_words + c / 16] >> (2 * (c % 16))) & 3u);
    m->row_stride = stride;
}

int orc_matrix_matvec(orc_matrix* m, const int8_t* xq, float amax, double* out, int simd, int threads) {
    if (!m || !xq || !out) return -1;
    double os = (double)m->scale * (double)amax / 127.0;
    if (os == 0.0) os = 1.0;
    if (simd) {
        ensure_codes(m);
        int stride = m->row_stride;
        std::vector<int8_t> acts((size_t)stride, 0);
        std::memcpy(acts.data(), xq, (size_t)m->cols);
        int32_t act_sum = 0;
        for (int i = 0; i < m->cols; ++i) act_sum += (int32_t)xq[i];
        const uint8_t* codes = m->codes.data();
        const int8_t* a = acts.data();
        run_rows(m->rows, m->cols, threads, [&](int s, int e) {
            for (int r = s; r < e; ++r) {
                int32_t raw = orc_code_row_dot_avx2(codes + (size_t)r * stride, a, stride);
                out[r] = (double)(raw - act_sum) * os;
            }
        });
    } else {
        const uint32_t* w = m->words.data();
        int rw = m->row_words, cols = m->cols;
        run_rows(m->rows, m->cols, threads, [&](int s, int e) {
            for (int r = s; r < e; ++r) out[r] = (double)row_dot_words(w + (size_t)r * rw, cols, xq) * os;
        });
    }
    return 0;
}

// ---- layers ---------------------------------------------------------------------

int orc_dense_forward(orc_matrix* w, int activation, const float* in, int batch, float* pre, float* post, int simd,
                      int threads) {
    if (!w || !in) return -1;
    int K = w->cols, N = w->rows;
    std::vector<double> tmp(N);
    std::vector<int8_t> xq(K);
    for (int b = 0; b < batch; ++b) {
        float amax = orc_quantize_f32(in + (size_t)b * K, K, xq.data());
        orc_matrix_matvec(w, xq.data(), amax, tmp.data(), simd, threads);
        for (int o = 0; o < N; ++o) {
            float v = (float)tmp[o];
            if (pre) pre[(size_t)b * N + o] = v;
            if (post) post[(size_t)b * N + o] = orc_activate_f32(v, activation);
        }
    }
    return 0;
}

int orc_swiglu_forward(orc_matrix* gate, orc_matrix* up, orc_matrix* down, const float* bg, const float* bu,
                       const float* bd, const float* inner_w, int inner_w_len, double rms_eps, int activation,
                       const float* in, int seq, float* pre, float* post, int8_t* q_in, float* amax_in,
                       float* raw_prod, int8_t* q_pre, float* amax_pre, int simd, int threads) {
    if (!gate || !up || !down || !in) return -1;
    int H = gate->cols, I = gate->rows;
    if (up->cols != H || up->rows != I || down->cols != I || down->rows != H) return -2;
    std::vector<double> g(I), u(I), d(H);
    std::vector<int8_t> xq(H), pq(I);
    std::vector<float> row(I);
    for (int s = 0; s < seq; ++s) {
        float amax = orc_quantize_f32(in + (size_t)s * H, H, xq.data());
        if (q_in) std::memcpy(q_in + (size_t)s * H, xq.data(), H);
        if (amax_in) amax_in[s] = amax;
        orc_matrix_matvec(gate, xq.data(), amax, g.data(), simd, threads);
        orc_matrix_matvec(up, xq.data(), amax, u.data(), simd, threads);
        for (int o = 0; o < I; ++o) {
            double gv = g[o] + (bg ? (double)bg[o] : 0.0);
            double uv = u[o] + (bu ? (double)bu[o] : 0.0);
            row[o] = (float)orc_gate_product(gv, uv, activation);
        }
        if (raw_prod) std::memcpy(raw_prod + (size_t)s * I, row.data(), sizeof(float) * I);
        orc_inner_rmsnorm_f32(row.data(), I, inner_w, inner_w_len, rms_eps);
        if (pre) std::memcpy(pre + (size_t)s * I, row.data(), sizeof(float) * I);
        float amax2 = orc_quantize_f32(row.data(), I, pq.data());
        if (q_pre) std::memcpy(q_pre + (size_t)s * I, pq.data(), I);
        if (amax_pre) amax_pre[s] = amax2;
        orc_matrix_matvec(down, pq.data(), amax2, d.data(), simd, threads);
        if (post)
            for (int i = 0; i < H; ++i) post[(size_t)s * H + i] = (float)(d[i] + (bd ? (double)bd[i] : 0.0));
    }
    return 0;
}

}  // extern "C"

struct orc_mha {
    int d_model, heads, kv_heads, head_dim, q_dim, kv_dim, msl;
    double theta, rms_eps;
    orc_matrix *wq, *wk, *wv, *wo;
    std::vector<float> bq, bk, bv, bo, qn, kn, inner;
    std::vector<float> cache_k, cache_v;  // [msl, kv_dim]
    bool cache_live = false;
    int kv_offset = 0;
};

namespace {

void per_head_norm_f64(double* data, const std::vector<float>& gamma, int heads, int hd, double eps) {
    if (eps <= 0) eps = 1e-6;
    for (int h = 0; h < heads; ++h) {
        double* p = data + (size_t)h * hd;
        double ss = 0.0;
        for (int i = 0; i < hd; ++i) ss += p[i] * p[i];
        double rms = std::sqrt(ss / (double)hd + eps);
        if (rms == 0.0) continue;
        double inv = 1.0 / rms;
        for (int d = 0; d < hd; ++d) {
            double sc = 1.0;
            if ((int)gamma.size() == hd) sc = (double)gamma[d];
            else if ((int)gamma.size() == heads * hd) sc = (double)gamma[(size_t)h * hd + d];
            p[d] = p[d] * inv * sc;
        }
    }
}

void per_head_norm_f32(float* data, const std::vector<float>& gamma, int heads, int hd, double eps) {
    if (eps <= 0) eps = 1e-6;
    for (int h = 0; h < heads; ++h) {
        float* p = data + (size_t)h * hd;
        double ss = 0.0;
        for (int i = 0; i < hd; ++i) {
            double v = (double)p[i];
            ss += v * v;
        }
        double rms = std::sqrt(ss / (double)hd + eps);
        if (rms == 0.0) continue;
        double inv = 1.0 / rms;
        for (int d = 0; d < hd; ++d) {
            double sc = 1.0;
            if ((int)gamma.size() == hd) sc = (double)gamma[d];
            else if ((int)gamma.size() == heads * hd) sc = (double)gamma[(size_t)h * hd + d];
            p[d] = (float)((double)p[d] * inv * sc);
        }
    }
}

void copy_opt(std::vector<float>& dst, const float* src, int n) {
    dst.clear();
    if (src && n > 0) dst.assign(src, src + n);
}

}  // namespace

extern "C" {

orc_mha* orc_mha_create(int d_model, int num_heads, int num_kv_heads, int head_dim, int max_seq_len,
                        double rope_theta, double rms_eps, orc_matrix* wq, orc_matrix* wk, orc_matrix* wv,
                        orc_matrix* wo, const float* bq, const float* bk, const float* bv, const float* bo,
                        const float* q_norm_w, int q_norm_len, const float* k_norm_w, int k_norm_len,
                        const float* inner_w, int inner_w_len) {
    if (!wq || !wk || !wv || !wo) return nullptr;
    auto* l = new orc_mha();
    l->d_model = d_model;
    l->heads = num_heads;
    l->kv_heads = num_kv_heads == 0 ? num_heads : num_kv_heads;
    l->head_dim = head_dim;
    l->q_dim = num_heads * head_dim;
    l->kv_dim = l->kv_heads * head_dim;
    l->msl = max_seq_len == 0 ? 512 : max_seq_len;
    l->theta = rope_theta > 0 ? rope_theta : 10000.0;
    l->rms_eps = rms_eps;
    l->wq = wq;
    l->wk = wk;
    l->wv = wv;
    l->wo = wo;
    copy_opt(l->bq, bq, l->q_dim);
    copy_opt(l->bk, bk, l->kv_dim);
    copy_opt(l->bv, bv, l->kv_dim);
    copy_opt(l->bo, bo, d_model);
    copy_opt(l->qn, q_norm_w, q_norm_len);
    copy_opt(l->kn, k_norm_w, k_norm_len);
    copy_opt(l->inner, inner_w, inner_w_len);
    return l;
}

void orc_mha_free(orc_mha* l) { delete l; }
void orc_mha_reset(orc_mha* l) { l->kv_offset = 0; }
int orc_mha_kv_offset(const orc_mha* l) { return l->kv_offset; }
int orc_mha_set_state(orc_mha* l, int kv_offset, const float* k, const float* v) {
    if (!l || kv_offset < 0 || kv_offset > l->msl || !k || !v) return -1;
    size_t n = (size_t)l->msl * l->kv_dim;
    l->cache_k.assign(k, k + n);
    l->cache_v.assign(v, v + n);
    l->cache_live = true;
    l->kv_offset = kv_offset;
    return 0;
}
const float* orc_mha_cache_k(const orc_mha* l) { return l->cache_k.data(); }
const float* orc_mha_cache_v(const orc_mha* l) { return l->cache_v.data(); }

int orc_mha_forward(orc_mha* l, const float* in, int batch, int seq, float* pre, float* post, double* q_tap,
                    double* attn_tap, int simd, int threads, int attn_threads) {
    if (!l || !in || batch <= 0 || seq <= 0) return -1;
    const int dm = l->d_model, H = l->heads, KVH = l->kv_heads, hd = l->head_dim;
    const int qd = l->q_dim, kvd = l->kv_dim, msl = l->msl, half = hd / 2;

    // Cache keeps its contents only for an incremental step (one token, warm cache).
    bool incremental = batch == 1 && seq == 1 && l->cache_live && l->kv_offset > 0;
    if (!incremental) {
        l->cache_k.assign((size_t)msl * kvd, 0.0f);
        l->cache_v.assign((size_t)msl * kvd, 0.0f);
        l->cache_live = true;
        l->kv_offset = 0;
    }
    const double qk_eps = l->rms_eps > 0 ? l->rms_eps : 1e-6;
    const int kv_start = l->kv_offset;

    std::vector<double> Q((size_t)seq * qd), tq(qd), tk(kvd), tv(kvd), attn((size_t)seq * qd), to(dm);
    std::vector<int8_t> xq(dm), aq(qd);
    std::vector<double> freq_div(half);
    for (int d = 0; d < half; ++d) freq_div[d] = std::pow(l->theta, (double)(2 * d) / (double)hd);

    for (int b = 0; b < batch; ++b) {
        const size_t base = (size_t)b * seq * dm;
        const int seq_base = kv_start + b * seq;
        for (int s = 0; s < seq; ++s) {
            const int pos = seq_base + s;
            float* krow = l->cache_k.data() + (size_t)(pos % msl) * kvd;
            float* vrow = l->cache_v.data() + (size_t)(pos % msl) * kvd;
            float amax = orc_quantize_f32(in + base + (size_t)s * dm, dm, xq.data());
            double* q = Q.data() + (size_t)s * qd;
            orc_matrix_matvec(l->wq, xq.data(), amax, tq.data(), simd, threads);
            for (int i = 0; i < qd; ++i) q[i] = tq[i] + (l->bq.empty() ? 0.0 : (double)l->bq[i]);
            orc_matrix_matvec(l->wk, xq.data(), amax, tk.data(), simd, threads);
            orc_matrix_matvec(l->wv, xq.data(), amax, tv.data(), simd, threads);
            for (int i = 0; i < kvd; ++i) {
                krow[i] = (float)(tk[i] + (l->bk.empty() ? 0.0 : (double)l->bk[i]));
                vrow[i] = (float)(tv[i] + (l->bv.empty() ? 0.0 : (double)l->bv[i]));
            }
            if (!l->qn.empty()) per_head_norm_f64(q, l->qn, H, hd, qk_eps);
            if (!l->kn.empty()) per_head_norm_f32(krow, l->kn, KVH, hd, qk_eps);
            for (int h = 0; h < H; ++h)
                for (int d = 0; d < half; ++d) {
                    double angle = (double)pos / freq_div[d];
                    double c = std::cos(angle), sn = std::sin(angle);
                    double v0 = q[h * hd + d], v1 = q[h * hd + d + half];
                    q[h * hd + d] = v0 * c - v1 * sn;
                    q[h * hd + d + half] = v0 * sn + v1 * c;
                }
            for (int h = 0; h < KVH; ++h)
                for (int d = 0; d < half; ++d) {
                    double angle = (double)pos / freq_div[d];
                    double c = std::cos(angle), sn = std::sin(angle);
                    double v0 = (double)krow[h * hd + d], v1 = (double)krow[h * hd + d + half];
                    krow[h * hd + d] = (float)(v0 * c - v1 * sn);
                    krow[h * hd + d + half] = (float)(v0 * sn + v1 * c);
                }
        }
        if (q_tap) std::memcpy(q_tap + (size_t)b * seq * qd, Q.data(), sizeof(double) * (size_t)seq * qd);

        const int per_kv = H / KVH;
        const double scale = 1.0 / std::sqrt((double)hd);
        const float* ck = l->cache_k.data();
        const float* cv = l->cache_v.data();
        const long long pairs = (long long)seq * H;
        int at = attn_threads > 1 ? attn_threads : 1;
        Pool::get().run((int)pairs, at, [&](int p) {
            int s = p / H, h = p % H;
            int last = seq_base + s, kvh = h / per_kv;
            std::vector<double> sc((size_t)last + 1);
            double mx = -1e9;
            const double* q = Q.data() + (size_t)s * qd + (size_t)h * hd;
            for (int kp = 0; kp <= last; ++kp) {
                const float* kr = ck + (size_t)(kp % msl) * kvd + (size_t)kvh * hd;
                double dot = 0.0;
                for (int d = 0; d < hd; ++d) dot += q[d] * (double)kr[d];
                double v = dot * scale;
                sc[kp] = v;
                if (v > mx) mx = v;
            }
            double den = 0.0;
            for (int kp = 0; kp <= last; ++kp) {
                sc[kp] = std::exp(sc[kp] - mx);
                den += sc[kp];
            }
            double* o = attn.data() + (size_t)s * qd + (size_t)h * hd;
            for (int d = 0; d < hd; ++d) {
                double sum = 0.0;
                for (int kp = 0; kp <= last; ++kp)
                    sum += sc[kp] * (double)cv[(size_t)(kp % msl) * kvd + (size_t)kvh * hd + d];
                o[d] = sum / den;
            }
        });
        if (attn_tap) std::memcpy(attn_tap + (size_t)b * seq * qd, attn.data(), sizeof(double) * (size_t)seq * qd);

        for (int s = 0; s < seq; ++s) {
            double* row = attn.data() + (size_t)s * qd;
            orc_inner_rmsnorm_f64(row, qd, l->inner.empty() ? nullptr : l->inner.data(), (int)l->inner.size(),
                                  l->rms_eps);
            float amax = orc_quantize_f64(row, qd, aq.data());
            orc_matrix_matvec(l->wo, aq.data(), amax, to.data(), simd, threads);
            for (int i = 0; i < dm; ++i) {
                if (pre) pre[base + (size_t)s * dm + i] = (float)row[i];
                if (post)
                    post[base + (size_t)s * dm + i] = (float)(to[i] + (l->bo.empty() ? 0.0 : (double)l->bo[i]));
            }
        }
    }
    l->kv_offset = kv_start + batch * seq;
    return 0;
}

int orc_argmax(const float* logits, int n) {
    int idx = 0;
    float best = logits[0];
    for (int i = 0; i < n; ++i)
        if (logits[i] > best) {
            best = logits[i];
            idx = i;
        }
    return idx;
}

void orc_lm_head(const float* hidden, const float* head, int vocab, int hs, float* logits, int threads) {
    auto body = [&](int s, int e) {
        for (int v = s; v < e; ++v) {
            const float* w = head + (size_t)v * hs;
            double sum = 0.0;
            for (int d = 0; d < hs; ++d) sum += (double)hidden[d] * (double)w[d];
            logits[v] = (float)sum;
        }
    };
    // same fan-out rule as the matvec: ApplyLMHead splits vocab rows across GOMAXPROCS
    run_rows(vocab, hs, threads, body);
}

}  // extern "C"

// ---- decoder ----------------------------------------------------------------------

struct orc_block {
    std::vector<float> g1, g2;
    orc_matrix* m[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};  // q k v o gate up down
    orc_mha* mha = nullptr;
};

struct orc_decoder {
    int layers, hidden, heads, kv_heads, head_dim, inter, vocab, act, msl;
    double eps, theta;
    std::vector<orc_block> blocks;
    const float* emb = nullptr;
    std::vector<float> final_gain;
    orc_matrix* head_tern = nullptr;  // untied LM head as a packed ternary matrix (borrowed), or null = tied fp32 head
};

namespace {

void free_block(orc_block& b) {
    if (b.mha) orc_mha_free(b.mha);
    b.mha = nullptr;
    for (auto*& m : b.m) {
        if (m) orc_matrix_free(m);
        m = nullptr;
    }
}

void finish_block(orc_decoder* d, orc_block& b, const float* g1, const float* g2) {
    b.g1.assign(d->hidden, 1.0f);
    b.g2.assign(d->hidden, 1.0f);
    if (g1) b.g1.assign(g1, g1 + d->hidden);
    if (g2) b.g2.assign(g2, g2 + d->hidden);
    b.mha = orc_mha_create(d->hidden, d->heads, d->kv_heads, d->head_dim, d->msl, d->theta, d->eps, b.m[0], b.m[1],
                           b.m[2], b.m[3], nullptr, nullptr, nullptr, nullptr, nullptr, 0, nullptr, 0, nullptr, 0);
}

}  // namespace

extern "C" {

orc_decoder* orc_decoder_create(int num_layers, int hidden, int num_heads, int num_kv_heads, int head_dim,
                                int intermediate, int vocab, double rms_eps, double rope_theta, int activation,
                                int max_seq_len) {
    auto* d = new orc_decoder();
    d->layers = num_layers;
    d->hidden = hidden;
    d->heads = num_heads;
    d->kv_heads = num_kv_heads;
    d->head_dim = head_dim;
    d->inter = intermediate;
    d->vocab = vocab;
    d->eps = rms_eps;
    d->theta = rope_theta;
    d->act = activation;
    d->msl = max_seq_len > 0 ? max_seq_len : 2048;  // NewTransformer default
    d->blocks.resize(num_layers);
    return d;
}

void orc_decoder_free(orc_decoder* d) {
    if (!d) return;
    for (auto& b : d->blocks) free_block(b);
    delete d;
}

int orc_decoder_set_block(orc_decoder* d, int block, const float* g1, const float* wq, const float* wk,
                          const float* wv, const float* wo, const float* g2, const float* wg, const float* wu,
                          const float* wd) {
    if (!d || block < 0 || block >= d->layers) return -1;
    orc_block& b = d->blocks[block];
    free_block(b);
    int qd = d->heads * d->head_dim, kvd = d->kv_heads * d->head_dim, H = d->hidden, I = d->inter;
    b.m[0] = orc_matrix_from_f32(wq, qd, H);
    b.m[1] = orc_matrix_from_f32(wk, kvd, H);
    b.m[2] = orc_matrix_from_f32(wv, kvd, H);
    b.m[3] = orc_matrix_from_f32(wo, H, qd);
    b.m[4] = orc_matrix_from_f32(wg, I, H);
    b.m[5] = orc_matrix_from_f32(wu, I, H);
    b.m[6] = orc_matrix_from_f32(wd, H, I);
    finish_block(d, b, g1, g2);
    return 0;
}

int orc_decoder_set_block_packed(orc_decoder* d, int block, const float* g1, const float* g2,
                                 const uint32_t* const* words7, const float* scales7) {
    if (!d || block < 0 || block >= d->layers) return -1;
    orc_block& b = d->blocks[block];
    free_block(b);
    int qd = d->heads * d->head_dim, kvd = d->kv_heads * d->head_dim, H = d->hidden, I = d->inter;
    int rows[7] = {qd, kvd, kvd, H, I, I, H};
    int cols[7] = {H, H, H, qd, H, H, I};
    for (int i = 0; i < 7; ++i) b.m[i] = orc_matrix_from_words(words7[i], rows[i], cols[i], scales7[i]);
    finish_block(d, b, g1, g2);
    return 0;
}

int orc_decoder_set_embeddings(orc_decoder* d, const float* emb, const float* final_gain) {
    if (!d || !emb) return -1;
    d->emb = emb;
    d->final_gain.assign(d->hidden, 1.0f);
    if (final_gain) d->final_gain.assign(final_gain, final_gain + d->hidden);
    return 0;
}

int orc_decoder_set_lm_head_ternary(orc_decoder* d, orc_matrix* head) {
    if (!d || (head && (orc_matrix_rows(head) != d->vocab || orc_matrix_cols(head) != d->hidden))) return -1;
    d->head_tern = head;
    return 0;
}

int orc_decoder_set_kv(orc_decoder* d, int block, int kv_offset, const float* k, const float* v) {
    if (!d || block < 0 || block >= d->layers || !d->blocks[block].mha) return -1;
    return orc_mha_set_state(d->blocks[block].mha, kv_offset, k, v);
}

void orc_decoder_reset(orc_decoder* d) {
    for (auto& b : d->blocks)
        if (b.mha) orc_mha_reset(b.mha);
}

int orc_decoder_forward(orc_decoder* d, const int32_t* tokens, int n, float* hidden_out, float* logits_out,
                        int simd, int threads, int attn_threads) {
    return orc_decoder_forward_taps(d, tokens, n, hidden_out, logits_out, nullptr, simd, threads, attn_threads);
}

int orc_decoder_forward_taps(orc_decoder* d, const int32_t* tokens, int n, float* hidden_out, float* logits_out,
                             float* block_out, int simd, int threads, int attn_threads) {
    if (!d || !d->emb || n <= 0) return -1;
    const int H = d->hidden;
    std::vector<float> x((size_t)n * H), resid, normed((size_t)n * H), sub((size_t)n * H);
    for (int i = 0; i < n; ++i) {
        long long off = (long long)tokens[i] * H;
        if (tokens[i] >= 0 && tokens[i] < d->vocab)
            std::memcpy(&x[(size_t)i * H], d->emb + off, sizeof(float) * H);
        else
            std::fill(x.begin() + (size_t)i * H, x.begin() + (size_t)(i + 1) * H, 0.0f);
    }
    for (auto& b : d->blocks) {
        if (!b.mha) return -2;
        resid = x;
        orc_block_rmsnorm(x.data(), n, H, b.g1.data(), d->eps, normed.data(), nullptr);
        orc_mha_forward(b.mha, normed.data(), 1, n, nullptr, sub.data(), nullptr, nullptr, simd, threads, attn_threads);
        for (size_t i = 0; i < x.size(); ++i) x[i] = sub[i] + resid[i];
        resid = x;
        orc_block_rmsnorm(x.data(), n, H, b.g2.data(), d->eps, normed.data(), nullptr);
        // the SwiGLU layer's own RMSNormEps is never set by the decoder builder: inner norm eps defaults to 1e-5
        orc_swiglu_forward(b.m[4], b.m[5], b.m[6], nullptr, nullptr, nullptr, nullptr, 0, 0.0, d->act, normed.data(), n,
                           nullptr, sub.data(), nullptr, nullptr, nullptr, nullptr, nullptr, simd, threads);
        for (size_t i = 0; i < x.size(); ++i) x[i] = sub[i] + resid[i];
        if (block_out) {  // the residual stream after this block, [n, H]
            std::memcpy(block_out, x.data(), sizeof(float) * x.size());
            block_out += x.size();
        }
    }
    orc_block_rmsnorm(x.data(), n, H, d->final_gain.data(), d->eps, normed.data(), nullptr);
    if (hidden_out) std::memcpy(hidden_out, normed.data(), sizeof(float) * (size_t)n * H);
    if (logits_out) {
        if (d->head_tern) {
            // applyPackedTernaryLMHead, poly/transformer.go:736-755: quantize the normalised row, packed matvec, float32(logit)
            std::vector<int8_t> xq((size_t)H);
            const float amax = orc_quantize_f32(&normed[(size_t)(n - 1) * H], H, xq.data());
            std::vector<double> l64((size_t)d->vocab);
            if (orc_matrix_matvec(d->head_tern, xq.data(), amax, l64.data(), simd, threads)) return -3;
            for (int v = 0; v < d->vocab; ++v) logits_out[v] = (float)l64[v];
        } else {
            orc_lm_head(&normed[(size_t)(n - 1) * H], d->emb, d->vocab, H, logits_out, threads);
        }
    }
    return 0;
}

int orc_decoder_generate(orc_decoder* d, const int32_t* prompt, int n_prompt, int max_new, int32_t* out_tokens,
                         double* prefill_seconds, double* decode_seconds, int simd, int threads, int attn_threads) {
    if (!d || n_prompt <= 0 || max_new < 0) return -1;
    std::vector<float> logits(d->vocab);
    orc_decoder_reset(d);
    double t0 = now_s();
    int rc = orc_decoder_forward(d, prompt, n_prompt, nullptr, logits.data(), simd, threads, attn_threads);
    if (rc) return rc;
    double t1 = now_s();
    for (int i = 0; i < max_new; ++i) {
        int32_t next = orc_argmax(logits.data(), d->vocab);
        out_tokens[i] = next;
        // Generate forwards after every sampled token, the last one included (its logits go unused)
        rc = orc_decoder_forward(d, &next, 1, nullptr, logits.data(), simd, threads, attn_threads);
        if (rc) return rc;
    }
    double t2 = now_s();
    if (prefill_seconds) *prefill_seconds = t1 - t0;
    if (decode_seconds) *decode_seconds = t2 - t1;
    return 0;
}

}  // extern "C"
