// Timed CPU baseline (test infrastructure, never shipped): a SIMD restatement of the reference's
// fastest CPU arm for the benchmarked product, Q4_K weights x Q8_K activations
// (src/backend/quant/q4_k.zig:895-913 is the scalar definition; the reference dispatches AVX2 /
// AVX-512 forms of the same block dot at run time). Integer block dots are exact in any order and the
// f32 epilogue keeps the scalar oracle's association, so the results equal oracle.cpp's bit for bit;
// tests/test_oracle_golden.py checks that. Formats without a SIMD arm here fall back to the scalar
// oracle code.
#include <immintrin.h>
#include <omp.h>

#include "oracle.cpp"  // structures, activation quantisers and the scalar block dots

namespace {

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
    __m128i s = _mm_add_epi32(_mm256_castsi256_si128(acc), _mm256_extracti128_si256(acc, 1));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x4e));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0xb1));
    const int32_t iscale = _mm_cvtsi128_si32(s);
    const float d = h2f(w->dm[0]) * a->d;
    const float dmin = h2f(w->dm[1]) * a->d;
    return d * (float)iscale - dmin * (float)imin;
}

__attribute__((target("avx2"))) void rows_q4_k_avx2(const uint8_t* w, size_t nb01, const uint8_t* qa, size_t astride, float* c, size_t m,
                                                    size_t n, size_t k, long long j0, long long j1) {
    const size_t nblk = k / 256;
    for (long long j = j0; j < j1; ++j) {
        const BlockQ4_K* wr = (const BlockQ4_K*)(w + (size_t)j * nb01);
        if (j + 1 < j1) _mm_prefetch((const char*)(w + (size_t)(j + 1) * nb01), _MM_HINT_T0);
        for (size_t i = 0; i < m; ++i) {
            const BlockQ8_K* ar = (const BlockQ8_K*)(qa + i * astride);
            float acc = 0.0f;
            for (size_t b = 0; b < nblk; ++b) acc += dot_q4_k_q8_k_avx2(&wr[b], &ar[b]);
            c[i * n + (size_t)j] = acc;
        }
    }
}

}  // namespace

extern "C" {

// 1 when the SIMD arm runs on this host for this format, 0 when cpuk_matmul falls back to the scalar code.
int cpuk_has_simd(int fmt) { return fmt == Q4_K && __builtin_cpu_supports("avx2") ? 1 : 0; }

// c[m, n] = a[m, k] . dequant(w)^T with the CPU kernels' arithmetic; rows split over the OpenMP threads.
int cpuk_matmul(int fmt, const void* w, size_t nb01, const float* a, float* c, size_t m, size_t n, size_t k) {
    if (!cpuk_has_simd(fmt)) return orc_matmul(fmt, w, nb01, a, c, m, n, k);
    size_t astride = 0;
    std::vector<uint8_t> qa = quantize_acts(fmt, a, m, k, &astride);
#pragma omp parallel
    {
        const long long nt = omp_get_num_threads(), t = omp_get_thread_num();
        const long long j0 = (long long)n * t / nt, j1 = (long long)n * (t + 1) / nt;
        rows_q4_k_avx2((const uint8_t*)w, nb01, qa.data(), astride, c, m, n, k, j0, j1);
    }
    return 0;
}

}  // extern "C"
