// Timed CPU baseline (test infrastructure, never shipped): a SIMD restatement of the reference's
// fastest applicable CPU arms for the benchmarked products -- Q4_K, Q5_K and TQ2_0 weights x Q8_K
// activations, Q8_0 weights x Q8_0 activations (scalar definitions: src/backend/quant/q4_k.zig:895-913,
// q5_k.zig:1093-1111, ternary.zig:377-386, q8_0.zig:1074-1089; the reference dispatches AVX2 / AVX-512
// forms of the same block dots at run time, q8_0.zig:1572-1635, q5_k.zig:1031-1152, ternary.zig:284-402).
// Integer block dots are exact in any order and the f32 epilogue keeps the scalar oracle's
// association, so the results equal oracle.cpp's bit for bit; tests/test_oracle_golden.py checks that.
// Formats without a SIMD arm here (folded TQ2_0, Q2_0) run the scalar oracle code.
//
// Threading follows QuantizedRhsParallel (src/backend/vector/matmul_quant.zig:522-616): products of
// fewer than 32 activation rows split the output columns into min(workers, n / 64) contiguous ranges
// once m*n*k >= 2^20, larger ones split the rows; results do not depend on the split. The worker count
// is set explicitly (cpuk_set_threads), never taken from the environment.
#include <immintrin.h>
#include <omp.h>

#include "oracle.cpp"  // structures, activation quantisers and the scalar block dots

namespace {

int g_threads = 0;  // 0: all logical CPUs the process may use

int workers() {
    int t = g_threads > 0 ? g_threads : omp_get_num_procs();
    if (t > 64) t = 64;  // the reference's -Dmax-threads ceiling (src/parallel.zig:19-25)
    return t < 1 ? 1 : t;
}

__attribute__((target("avx2"))) inline int32_t hsum_i32(__m256i v) {
    __m128i s = _mm_add_epi32(_mm256_castsi256_si128(v), _mm256_extracti128_si256(v, 1));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x4e));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0xb1));
    return _mm_cvtsi128_si32(s);
}

// One 256-weight block: 4 x 32 payload bytes, low nibbles = even sub-block, high nibbles = odd.
__attribute__((target("avx2"))) inline float dot_q4_k_q8_k_avx2(const BlockQ4_K* w, const BlockQ8_K* a) {
    const __m256i low_mask = _mm256_set1_epi8(0x0f);
    __m256i acc = _mm256_setzero_si256();  // eight int32 lanes of sum(scale * pair products)
    int32_t imin = 0;
    for (int pp = 0; pp < 4; ++pp) {
        uint8_t sc0, mn0, sc1, mn1;
        get_scale_min_k4(w->scales, 2 * pp, &sc0, &mn0);
        get_scale_min_k4(w->scales, 2 * pp + 1, &sc1, &mn1);
        const __m256i q = _mm256_loadu_si256((const __m256i*)(w->qs + pp * 32));
        const __m256i lo = _mm256_and_si256(q, low_mask);
        const __m256i hi = _mm256_and_si256(_mm256_srli_epi16(q, 4), low_mask);
        const __m256i a_lo = _mm256_loadu_si256((const __m256i*)(a->qs + pp * 64));
        const __m256i a_hi = _mm256_loadu_si256((const __m256i*)(a->qs + pp * 64 + 32));
        // unsigned levels (<= 15) times signed activations: pair sums fit int16 (2 * 15 * 127)
        const __m256i p_lo = _mm256_maddubs_epi16(lo, a_lo);
        const __m256i p_hi = _mm256_maddubs_epi16(hi, a_hi);
        acc = _mm256_add_epi32(acc, _mm256_madd_epi16(p_lo, _mm256_set1_epi16((short)sc0)));
        acc = _mm256_add_epi32(acc, _mm256_madd_epi16(p_hi, _mm256_set1_epi16((short)sc1)));
        imin += (int32_t)mn0 * ((int32_t)a->bsums[4 * pp] + (int32_t)a->bsums[4 * pp + 1]);
        imin += (int32_t)mn1 * ((int32_t)a->bsums[4 * pp + 2] + (int32_t)a->bsums[4 * pp + 3]);
    }
    const int32_t iscale = hsum_i32(acc);
    const float d = h2f(w->dm[0]) * a->d;
    const float dmin = h2f(w->dm[1]) * a->d;
    return d * (float)iscale - dmin * (float)imin;
}

// Q5_K: the same walk with bit s of qh[i] as the fifth bit of sub-block s (levels <= 31: pair sums fit int16).
__attribute__((target("avx2"))) inline float dot_q5_k_q8_k_avx2(const BlockQ5_K* w, const BlockQ8_K* a) {
    const __m256i low_mask = _mm256_set1_epi8(0x0f), one = _mm256_set1_epi8(1);
    const __m256i qh = _mm256_loadu_si256((const __m256i*)w->qh);
    __m256i acc = _mm256_setzero_si256();
    int32_t imin = 0;
    for (int pp = 0; pp < 4; ++pp) {
        uint8_t sc0, mn0, sc1, mn1;
        get_scale_min_k4(w->scales, 2 * pp, &sc0, &mn0);
        get_scale_min_k4(w->scales, 2 * pp + 1, &sc1, &mn1);
        const __m256i q = _mm256_loadu_si256((const __m256i*)(w->qs + pp * 32));
        // (qh >> s) & 1 per byte: the 16-bit shift drags bits across bytes, the mask keeps bit 0 of each byte
        const __m256i h_lo = _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(qh, 2 * pp), one), 4);
        const __m256i h_hi = _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(qh, 2 * pp + 1), one), 4);
        const __m256i lo = _mm256_or_si256(_mm256_and_si256(q, low_mask), h_lo);
        const __m256i hi = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(q, 4), low_mask), h_hi);
        const __m256i a_lo = _mm256_loadu_si256((const __m256i*)(a->qs + pp * 64));
        const __m256i a_hi = _mm256_loadu_si256((const __m256i*)(a->qs + pp * 64 + 32));
        const __m256i p_lo = _mm256_maddubs_epi16(lo, a_lo);
        const __m256i p_hi = _mm256_maddubs_epi16(hi, a_hi);
        acc = _mm256_add_epi32(acc, _mm256_madd_epi16(p_lo, _mm256_set1_epi16((short)sc0)));
        acc = _mm256_add_epi32(acc, _mm256_madd_epi16(p_hi, _mm256_set1_epi16((short)sc1)));
        imin += (int32_t)mn0 * ((int32_t)a->bsums[4 * pp] + (int32_t)a->bsums[4 * pp + 1]);
        imin += (int32_t)mn1 * ((int32_t)a->bsums[4 * pp + 2] + (int32_t)a->bsums[4 * pp + 3]);
    }
    const int32_t iscale = hsum_i32(acc);
    const float d = h2f(w->dm[0]) * a->d;
    const float dmin = h2f(w->dm[1]) * a->d;
    return d * (float)iscale - dmin * (float)imin;
}

// Q8_0 x Q8_0: |w| as the unsigned operand, sign(w) moved onto the activation (pair sums <= 2 * 127 * 127).
__attribute__((target("avx2"))) inline float dot_q8_0_q8_0_avx2(const BlockQ8_0* a, const BlockQ8_0* w) {
    const __m256i wq = _mm256_loadu_si256((const __m256i*)w->qs), aq = _mm256_loadu_si256((const __m256i*)a->qs);
    const __m256i p = _mm256_maddubs_epi16(_mm256_sign_epi8(wq, wq), _mm256_sign_epi8(aq, wq));
    const int32_t dot = hsum_i32(_mm256_madd_epi16(p, _mm256_set1_epi16(1)));
    const float d = h2f(a->d) * h2f(w->d);
    return (float)dot * d;
}

// TQ2_0: byte hg*32 + m carries elements hg*128 + n*32 + m in crumb n (codes 0..2, or 3 in a malformed block);
// sum(code * a) - sum(a), then h2f(d_w) * d_a * f32(isum) left to right.
__attribute__((target("avx2"))) inline float dot_tq2_0_q8_k_avx2(const BlockTQ2_0* w, const BlockQ8_K* a) {
    const __m256i three = _mm256_set1_epi8(3);
    __m256i acc16 = _mm256_setzero_si256();  // sixteen int16 lanes: 8 terms of at most 2 * 3 * 127 each
    for (int hg = 0; hg < 2; ++hg) {
        const __m256i q = _mm256_loadu_si256((const __m256i*)(w->qs + hg * 32));
        for (int n = 0; n < 4; ++n) {
            const __m256i code = _mm256_and_si256(_mm256_srli_epi16(q, 2 * n), three);
            const __m256i av = _mm256_loadu_si256((const __m256i*)(a->qs + hg * 128 + n * 32));
            acc16 = _mm256_add_epi16(acc16, _mm256_maddubs_epi16(code, av));
        }
    }
    const int32_t dots = hsum_i32(_mm256_madd_epi16(acc16, _mm256_set1_epi16(1)));
    const int32_t isum = dots - bsum_total(a);
    return h2f(w->d) * a->d * (float)isum;
}

bool simd_for(int fmt) {
    static const bool avx2 = __builtin_cpu_supports("avx2");
    return avx2 && (fmt == Q4_K || fmt == Q5_K || fmt == Q8_0 || fmt == TQ2_0);
}

// One output element, blocks ascending (row_dot of the scalar oracle with the SIMD block dots).
__attribute__((target("avx2"))) float row_dot_fast(int fmt, const uint8_t* wrow, const void* arow, size_t k) {
    float acc = 0;
    switch (fmt) {
        case Q4_K: {
            const BlockQ4_K* w = (const BlockQ4_K*)wrow;
            const BlockQ8_K* a = (const BlockQ8_K*)arow;
            for (size_t b = 0; b < k / 256; ++b) acc += dot_q4_k_q8_k_avx2(&w[b], &a[b]);
            return acc;
        }
        case Q5_K: {
            const BlockQ5_K* w = (const BlockQ5_K*)wrow;
            const BlockQ8_K* a = (const BlockQ8_K*)arow;
            for (size_t b = 0; b < k / 256; ++b) acc += dot_q5_k_q8_k_avx2(&w[b], &a[b]);
            return acc;
        }
        case Q8_0: {
            const BlockQ8_0* w = (const BlockQ8_0*)wrow;
            const BlockQ8_0* a = (const BlockQ8_0*)arow;
            for (size_t b = 0; b < k / 32; ++b) acc += dot_q8_0_q8_0_avx2(&a[b], &w[b]);
            return acc;
        }
        case TQ2_0: {
            const BlockTQ2_0* w = (const BlockTQ2_0*)wrow;
            const BlockQ8_K* a = (const BlockQ8_K*)arow;
            for (size_t b = 0; b < k / 256; ++b) acc += dot_tq2_0_q8_k_avx2(&w[b], &a[b]);
            return acc;
        }
    }
    return row_dot(fmt, wrow, arow, k);
}

inline float any_row_dot(bool simd, int fmt, const uint8_t* wrow, const void* arow, size_t k) {
    return simd ? row_dot_fast(fmt, wrow, arow, k) : row_dot(fmt, wrow, arow, k);
}

}  // namespace

extern "C" {

// 1 when a SIMD arm runs on this host for this format, 0 when the scalar oracle code is timed instead.
int cpuk_has_simd(int fmt) { return simd_for(fmt) ? 1 : 0; }

// Worker threads of the calls below: n > 0 sets it, 0 restores "all logical CPUs". Returns the count in use.
int cpuk_set_threads(int n) {
    g_threads = n > 0 ? n : 0;
    omp_set_num_threads(workers());  // also the default of parallel regions without a clause (the scalar oracle's encoders)
    return workers();
}
int cpuk_threads(void) { return workers(); }

// c[m, n] = a[m, k] . dequant(w)^T with the CPU kernels' arithmetic.
int cpuk_matmul(int fmt, const void* w, size_t nb01, const float* a, float* c, size_t m, size_t n, size_t k) {
    if (row_bytes(fmt, k) == 0 || nb01 < row_bytes(fmt, k)) return 1;
    const bool simd = simd_for(fmt);
    size_t astride = 0;
    std::vector<uint8_t> qa = quantize_acts(fmt, a, m, k, &astride);
    const uint8_t* wb = (const uint8_t*)w;
    const int T = workers();
    const unsigned __int128 work = (unsigned __int128)m * n * k;
    if (m < 32) {
        // column arm: contiguous column ranges, one per task
        long long tasks = work >= ((unsigned __int128)1 << 20) ? (long long)(n / 64) : 1;
        if (tasks > T) tasks = T;
        if (tasks < 1) tasks = 1;
#pragma omp parallel for schedule(static, 1) num_threads((int)tasks)
        for (long long t = 0; t < tasks; ++t) {
            const long long j0 = (long long)n * t / tasks, j1 = (long long)n * (t + 1) / tasks;
            for (long long j = j0; j < j1; ++j) {
                if (j + 1 < j1) _mm_prefetch((const char*)(wb + (size_t)(j + 1) * nb01), _MM_HINT_T0);
                for (size_t i = 0; i < m; ++i)
                    c[i * n + (size_t)j] = any_row_dot(simd, fmt, wb + (size_t)j * nb01, qa.data() + i * astride, k);
            }
        }
        return 0;
    }
    // row arm: activation rows over the tasks, every task walks all columns
#pragma omp parallel for schedule(static) num_threads(T)
    for (long long i = 0; i < (long long)m; ++i)
        for (size_t j = 0; j < n; ++j)
            c[(size_t)i * n + j] = any_row_dot(simd, fmt, wb + j * nb01, qa.data() + (size_t)i * astride, k);
    return 0;
}

// The expert layer with the same block dots (orc_moe_ffn's structure, exec/moe.zig:890-920, :1287-1292):
// pairs over the worker threads, per pair quantise the token row, gate/up dots, swiglu, requantise, down dots;
// then the slot-ordered weighted sum.
int cpuk_moe_ffn(int fmt, const void* gate, const void* up, const void* down, const float* x, size_t seq, size_t hidden,
                 size_t out_pe, size_t n_expert, size_t top_k, const int64_t* selected, const float* weights, float* out) {
    const size_t rb_in = row_bytes(fmt, hidden), rb_g = row_bytes(fmt, out_pe);
    if (rb_in == 0 || rb_g == 0) return 1;
    for (size_t p = 0; p < seq * top_k; ++p)
        if (selected[p] < 0 || (size_t)selected[p] >= n_expert) return 1;
    const bool simd = simd_for(fmt);
    std::vector<float> pair_out(seq * top_k * hidden);
#pragma omp parallel num_threads(workers())
    {
        std::vector<float> gate_v(out_pe), up_v(out_pe), g(out_pe);
#pragma omp for schedule(dynamic, 1)
        for (long long p = 0; p < (long long)(seq * top_k); ++p) {
            const size_t t = (size_t)p / top_k;
            const size_t e = (size_t)selected[p];
            size_t s_in = 0, s_g = 0;
            std::vector<uint8_t> qx = quantize_acts(fmt, x + t * hidden, 1, hidden, &s_in);
            const uint8_t* wg = (const uint8_t*)gate + e * out_pe * rb_in;
            const uint8_t* wu = (const uint8_t*)up + e * out_pe * rb_in;
            const uint8_t* wd = (const uint8_t*)down + e * hidden * rb_g;
            for (size_t j = 0; j < out_pe; ++j) {
                gate_v[j] = any_row_dot(simd, fmt, wg + j * rb_in, qx.data(), hidden);
                up_v[j] = any_row_dot(simd, fmt, wu + j * rb_in, qx.data(), hidden);
            }
            for (size_t j = 0; j < out_pe; ++j) g[j] = swiglu_pair(gate_v[j], up_v[j]);
            std::vector<uint8_t> qg = quantize_acts(fmt, g.data(), 1, out_pe, &s_g);
            float* po = pair_out.data() + (size_t)p * hidden;
            for (size_t j = 0; j < hidden; ++j) po[j] = any_row_dot(simd, fmt, wd + j * rb_g, qg.data(), out_pe);
        }
    }
    for (size_t t = 0; t < seq; ++t)
        for (size_t kk = 0; kk < top_k; ++kk) {
            const size_t p = t * top_k + kk;
            const float w = weights[p];
            const float* src = pair_out.data() + p * hidden;
            float* dst = out + t * hidden;
            if (kk == 0)
                for (size_t j = 0; j < hidden; ++j) dst[j] = w * src[j];
            else
                for (size_t j = 0; j < hidden; ++j) dst[j] += w * src[j];
        }
    return 0;
}

}  // extern "C"
