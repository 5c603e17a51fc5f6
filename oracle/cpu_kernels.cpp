// Timed CPU baseline (test infrastructure, never shipped): a SIMD restatement of the reference's
// fastest applicable CPU arms for the benchmarked products -- Q4_K, Q5_K, Q6_K and TQ2_0 weights x Q8_K
// activations, Q8_0 weights x Q8_0 activations (scalar definitions: src/backend/quant/q4_k.zig:895-913,
// q5_k.zig:1093-1111, q6_k.zig:617-631, ternary.zig:377-386, q8_0.zig:1074-1089; the reference dispatches AVX2 / AVX-512
// forms of the same block dots at run time, q8_0.zig:1572-1635, q5_k.zig:1031-1152, ternary.zig:284-402).
// Integer block dots are exact in any order and the f32 epilogue keeps the scalar oracle's
// association, so the results equal oracle.cpp's bit for bit; tests/test_oracle_golden.py checks that.
// Formats without a SIMD arm here (folded TQ2_0, Q2_0) run the scalar oracle code.
//
// The reference's fastest K-quant arm is not the compact row walk but a repack done once at load time: eight
// weight rows interleaved per 256-weight block (BlockQ4_Kx8 / BlockQ5_Kx8, src/backend/quant/types.zig:99-119,
// packed by q4_k.zig:127-192 / q5_k.zig:57-123, multiplied by q4_k.zig:1733-1782 / q5_k.zig:826-885). cpuk_pack_rows and
// cpuk_matmul_packed restate that arm: the same layout, eight columns per step against a broadcast of four activation
// bytes, integer sub-block sums scaled in int32, one f32 epilogue per block -- bit-equal to the compact kernels,
// as the reference's own tests require (q4_k_tests.zig:852-896, q5_k_tests.zig:92-137). Four or more activation rows
// are packed four at a time as well (BlockQ8_Kx4) and take the four-row kernels; Q6_K, Q8_0 and TQ2_0 have four-row
// weight packs (BlockQ6_Kx4, BlockQ8_0x4, BlockTQ2_0x4); the expert layer groups its pairs by expert (cpuk_moe_ffn_packed).
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

// Q6_K: levels 0..63 from ql nibbles and qh bit pairs (element 128 c + 32 s + l: ql[64 c + 32 (s & 1) + l], low nibble for
// s < 2, and bits 2s, 2s + 1 of qh[32 c + l]); one signed scale per 16 elements. Unsigned levels times signed activations
// (pair sums <= 2 * 63 * 127), each half of a 32-byte vector scaled by its own group scale, and the offset of 32 taken
// out through the activation block's sixteen group sums: the integer total of q6_k.zig:617-631, then f32(total) * (d_w * d_a).
__attribute__((target("avx2"))) inline float dot_q6_k_q8_k_avx2(const BlockQ6_K* w, const BlockQ8_K* a) {
    const __m256i m4 = _mm256_set1_epi8(0x0f), m2 = _mm256_set1_epi8(0x30);
    __m256i acc = _mm256_setzero_si256();
    for (int c = 0; c < 2; ++c) {
        const __m256i l0 = _mm256_loadu_si256((const __m256i*)(w->ql + 64 * c)), l1 = _mm256_loadu_si256((const __m256i*)(w->ql + 64 * c + 32));
        const __m256i h = _mm256_loadu_si256((const __m256i*)(w->qh + 32 * c));
        const __m256i q[4] = {
            _mm256_or_si256(_mm256_and_si256(l0, m4), _mm256_and_si256(_mm256_slli_epi16(h, 4), m2)),
            _mm256_or_si256(_mm256_and_si256(l1, m4), _mm256_and_si256(_mm256_slli_epi16(h, 2), m2)),
            _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l0, 4), m4), _mm256_and_si256(h, m2)),
            _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l1, 4), m4), _mm256_and_si256(_mm256_srli_epi16(h, 2), m2)),
        };
        for (int sec = 0; sec < 4; ++sec) {
            const __m256i av = _mm256_loadu_si256((const __m256i*)(a->qs + 128 * c + 32 * sec));
            const __m256i p = _mm256_maddubs_epi16(q[sec], av);  // lanes 0..7: elements l < 16, lanes 8..15: l >= 16
            const __m256i sc = _mm256_set_m128i(_mm_set1_epi16((short)w->scales[8 * c + 2 * sec + 1]), _mm_set1_epi16((short)w->scales[8 * c + 2 * sec]));
            acc = _mm256_add_epi32(acc, _mm256_madd_epi16(p, sc));
        }
    }
    int32_t corr = 0;
    for (int g = 0; g < 16; ++g) corr += (int32_t)w->scales[g] * (int32_t)a->bsums[g];
    const int32_t iacc = hsum_i32(acc) - 32 * corr;
    const float d = h2f(w->d) * a->d;
    return (float)iacc * d;
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
    return avx2 && (fmt == Q4_K || fmt == Q5_K || fmt == Q6_K || fmt == Q8_0 || fmt == TQ2_0);
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
        case Q6_K: {
            const BlockQ6_K* w = (const BlockQ6_K*)wrow;
            const BlockQ8_K* a = (const BlockQ8_K*)arow;
            for (size_t b = 0; b < k / 256; ++b) acc += dot_q6_k_q8_k_avx2(&w[b], &a[b]);
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

// ---- eight-row packs ------------------------------------------------------------------------------
// Column c of the group is weight row 8 * group + c. scales / mins: [sub-block][column]. Q4_K qs: byte
// pair * 256 + fg * 32 + c * 4 + l = payload byte pair * 32 + fg * 4 + l of column c (low nibble: sub-block 2 * pair,
// high nibble: 2 * pair + 1). Q5_K qs: byte sub * 256 + fg * 32 + c * 4 + l = the five-bit level of element
// sub * 32 + fg * 4 + l of column c.
struct BlockQ4_Kx8 {
    uint16_t d[8], dmin[8];
    uint8_t scales[64], mins[64];
    uint8_t qs[1024];
};
struct BlockQ5_Kx8 {
    uint16_t d[8], dmin[8];
    uint8_t scales[64], mins[64];
    uint8_t qs[2048];
};
static_assert(sizeof(BlockQ4_Kx8) == 1184 && sizeof(BlockQ5_Kx8) == 2208, "packed block sizes");

// Q8_0: four rows interleaved per 32-weight block (BlockQ8_0x4, types.zig:78-81, packed by q8_0.zig:259-303):
// qs byte fg * 16 + c * 4 + l = weight fg * 4 + l of column c.
struct BlockQ8_0x4 {
    uint16_t d[4];
    int8_t qs[128];
};
static_assert(sizeof(BlockQ8_0x4) == 136, "packed block size");

struct PackedRows {
    int fmt = 0, group = 8;  // rows interleaved per packed block: 8 (Q4_K, Q5_K) or 4 (Q6_K, Q8_0, TQ2_0)
    size_t n = 0, k = 0, blocks_per_row = 0;
    std::vector<uint8_t> data;  // [n / group][blocks_per_row] packed blocks
};

template <class Src, class Dst>
void pack_header_x8(const Src* const cols[8], Dst* dst) {
    for (int c = 0; c < 8; ++c) {
        dst->d[c] = cols[c]->dm[0];
        dst->dmin[c] = cols[c]->dm[1];
    }
    for (int sub = 0; sub < 8; ++sub)
        for (int c = 0; c < 8; ++c) get_scale_min_k4(cols[c]->scales, sub, &dst->scales[sub * 8 + c], &dst->mins[sub * 8 + c]);
}

inline int q5_level(const BlockQ5_K* b, int sub, int i) {  // q5_k.zig:1259-1264
    const int nib = (sub & 1) ? (b->qs[(sub >> 1) * 32 + i] >> 4) : (b->qs[(sub >> 1) * 32 + i] & 0x0f);
    return nib + (((b->qh[i] >> sub) & 1) << 4);
}

// dst[c] += d_w[c] d_a f32(iscale[c]) - dmin_w[c] d_a f32(imin[c]) for the eight columns of one packed block
__attribute__((target("avx2,f16c"))) inline __m256 epilogue_x8(const uint16_t* d, const uint16_t* dmin, float da, __m256i iscale, __m256i imin,
                                                              __m256 acc) {
    const __m256 dav = _mm256_set1_ps(da);
    const __m256 dd = _mm256_mul_ps(_mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)d)), dav);
    const __m256 dm = _mm256_mul_ps(_mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)dmin)), dav);
    const __m256 term = _mm256_sub_ps(_mm256_mul_ps(dd, _mm256_cvtepi32_ps(iscale)), _mm256_mul_ps(dm, _mm256_cvtepi32_ps(imin)));
    return _mm256_add_ps(acc, term);
}
__attribute__((target("avx2"))) inline __m256i widen_u8x8(const uint8_t* p) { return _mm256_cvtepu8_epi32(_mm_loadl_epi64((const __m128i*)p)); }
__attribute__((target("avx2"))) inline __m256i bcast4(const int8_t* p) {
    int32_t v;
    memcpy(&v, p, 4);
    return _mm256_set1_epi32(v);
}

__attribute__((target("avx2,f16c"))) inline __m256 accumulate_q4_kx8(const BlockQ4_Kx8* w, const BlockQ8_K* a, __m256 acc) {
    const __m256i low_mask = _mm256_set1_epi8(0x0f), ones = _mm256_set1_epi16(1);
    __m256i iscale = _mm256_setzero_si256(), imin = _mm256_setzero_si256();
    for (int pair = 0; pair < 4; ++pair) {
        const int even = 2 * pair, odd = even + 1;
        __m256i sum_e = _mm256_setzero_si256(), sum_o = _mm256_setzero_si256();
        for (int fg = 0; fg < 8; ++fg) {
            const __m256i q = _mm256_loadu_si256((const __m256i*)(w->qs + pair * 256 + fg * 32));
            const __m256i w_e = _mm256_and_si256(q, low_mask), w_o = _mm256_and_si256(_mm256_srli_epi16(q, 4), low_mask);
            // four levels (<= 15) times four activations per column: pair sums fit int16, group sums int32
            sum_e = _mm256_add_epi32(sum_e, _mm256_madd_epi16(_mm256_maddubs_epi16(w_e, bcast4(a->qs + even * 32 + fg * 4)), ones));
            sum_o = _mm256_add_epi32(sum_o, _mm256_madd_epi16(_mm256_maddubs_epi16(w_o, bcast4(a->qs + odd * 32 + fg * 4)), ones));
        }
        iscale = _mm256_add_epi32(iscale, _mm256_add_epi32(_mm256_mullo_epi32(sum_e, widen_u8x8(w->scales + even * 8)),
                                                          _mm256_mullo_epi32(sum_o, widen_u8x8(w->scales + odd * 8))));
        const __m256i bs_e = _mm256_set1_epi32((int32_t)a->bsums[2 * even] + (int32_t)a->bsums[2 * even + 1]);
        const __m256i bs_o = _mm256_set1_epi32((int32_t)a->bsums[2 * odd] + (int32_t)a->bsums[2 * odd + 1]);
        imin = _mm256_add_epi32(imin, _mm256_add_epi32(_mm256_mullo_epi32(bs_e, widen_u8x8(w->mins + even * 8)),
                                                      _mm256_mullo_epi32(bs_o, widen_u8x8(w->mins + odd * 8))));
    }
    return epilogue_x8(w->d, w->dmin, a->d, iscale, imin, acc);
}

__attribute__((target("avx2,f16c"))) inline __m256 accumulate_q5_kx8(const BlockQ5_Kx8* w, const BlockQ8_K* a, __m256 acc) {
    const __m256i ones = _mm256_set1_epi16(1);
    __m256i iscale = _mm256_setzero_si256(), imin = _mm256_setzero_si256();
    for (int sub = 0; sub < 8; ++sub) {
        __m256i sum = _mm256_setzero_si256();
        for (int fg = 0; fg < 8; ++fg) {
            const __m256i q = _mm256_loadu_si256((const __m256i*)(w->qs + sub * 256 + fg * 32));  // levels <= 31: pair sums fit int16
            sum = _mm256_add_epi32(sum, _mm256_madd_epi16(_mm256_maddubs_epi16(q, bcast4(a->qs + sub * 32 + fg * 4)), ones));
        }
        iscale = _mm256_add_epi32(iscale, _mm256_mullo_epi32(sum, widen_u8x8(w->scales + sub * 8)));
        const __m256i bs = _mm256_set1_epi32((int32_t)a->bsums[2 * sub] + (int32_t)a->bsums[2 * sub + 1]);
        imin = _mm256_add_epi32(imin, _mm256_mullo_epi32(bs, widen_u8x8(w->mins + sub * 8)));
    }
    return epilogue_x8(w->d, w->dmin, a->d, iscale, imin, acc);
}

// One packed Q8_0 block against one Q8_0 activation block: the reference's x4 law, (f32(t) * d_a) * d_w[c]
// (q8_0.zig:1591-1613) -- a different f32 association from the compact dot's f32(t) * (d_a * d_w), so this arm
// agrees with the compact kernels to rounding, not bit for bit.
__attribute__((target("avx2,f16c"))) inline __m128 accumulate_q8_0x4(const BlockQ8_0x4* w, const BlockQ8_0* a, __m128 acc) {
    const __m256i ones = _mm256_set1_epi16(1);
    __m256i sum = _mm256_setzero_si256();
    for (int g = 0; g < 4; ++g) {
        const __m256i r = _mm256_loadu_si256((const __m256i*)(w->qs + g * 32));  // feature groups 2g | 2g + 1, four columns each
        int32_t lo, hi;
        memcpy(&lo, a->qs + 8 * g, 4);
        memcpy(&hi, a->qs + 8 * g + 4, 4);
        const __m256i b = _mm256_set_m128i(_mm_set1_epi32(hi), _mm_set1_epi32(lo));
        // |w| as the unsigned operand, sign(w) moved onto the activation
        sum = _mm256_add_epi32(sum, _mm256_madd_epi16(_mm256_maddubs_epi16(_mm256_sign_epi8(r, r), _mm256_sign_epi8(b, r)), ones));
    }
    const __m128i t = _mm_add_epi32(_mm256_castsi256_si128(sum), _mm256_extracti128_si256(sum, 1));
    const __m128 dw = _mm_cvtph_ps(_mm_loadl_epi64((const __m128i*)w->d));
    return _mm_add_ps(acc, _mm_mul_ps(_mm_mul_ps(_mm_cvtepi32_ps(t), _mm_set1_ps(h2f(a->d))), dw));
}
__attribute__((target("avx2,f16c"))) inline void group_dot_q8_0x4(const PackedRows& P, size_t group, const BlockQ8_0* a, float* out4) {
    const BlockQ8_0x4* w = (const BlockQ8_0x4*)P.data.data() + group * P.blocks_per_row;
    __m128 acc = _mm_setzero_ps();
    for (size_t b = 0; b < P.blocks_per_row; ++b) acc = accumulate_q8_0x4(&w[b], &a[b], acc);
    _mm_storeu_ps(out4, acc);
}

// TQ2_0: four rows interleaved per 256-weight block (BlockTQ2_0x4, types.zig:150-159, packed by ternary.zig:423-446):
// qs byte half * 128 + fg * 16 + c * 4 + l = byte half * 32 + fg * 4 + l of column c; the four crumbs of a byte still
// are elements +0 / +32 / +64 / +96 of its half. The kernel is the ymm form of ternary.zig:556-575: one 32-byte load =
// two k-groups x four columns, the matching 8 activation bytes broadcast dword-wise, eight int32 lanes folded to the
// four columns once per block; then sums[c] += (d_c * d_a) * f32(dot_c - bsum), bit-equal to the compact kernel.
struct BlockTQ2_0x4 {
    uint16_t d[4];
    uint8_t qs[256];
};
static_assert(sizeof(BlockTQ2_0x4) == 264, "packed block size");

__attribute__((target("avx2,f16c"))) inline __m128 accumulate_tq2_0x4(const BlockTQ2_0x4* w, const BlockQ8_K* a, __m128 acc) {
    const __m256i three = _mm256_set1_epi8(3), ones = _mm256_set1_epi16(1);
    __m256i sum = _mm256_setzero_si256();
    for (int half = 0; half < 2; ++half)
        for (int fg2 = 0; fg2 < 4; ++fg2) {
            const __m256i wv = _mm256_loadu_si256((const __m256i*)(w->qs + half * 128 + fg2 * 32));
            for (int lane = 0; lane < 4; ++lane) {
                int32_t g0, g1;
                memcpy(&g0, a->qs + half * 128 + lane * 32 + fg2 * 8, 4);
                memcpy(&g1, a->qs + half * 128 + lane * 32 + fg2 * 8 + 4, 4);
                const __m256i act = _mm256_set_m128i(_mm_set1_epi32(g1), _mm_set1_epi32(g0));
                const __m256i crumb = _mm256_and_si256(_mm256_srli_epi16(wv, 2 * lane), three);  // codes 0..3 per byte
                sum = _mm256_add_epi32(sum, _mm256_madd_epi16(_mm256_maddubs_epi16(crumb, act), ones));
            }
        }
    const __m128i dot = _mm_add_epi32(_mm256_castsi256_si128(sum), _mm256_extracti128_si256(sum, 1));
    const __m128i isum = _mm_sub_epi32(dot, _mm_set1_epi32(bsum_total(a)));
    const __m128 dw = _mm_cvtph_ps(_mm_loadl_epi64((const __m128i*)w->d));
    return _mm_add_ps(acc, _mm_mul_ps(_mm_mul_ps(dw, _mm_set1_ps(a->d)), _mm_cvtepi32_ps(isum)));
}
__attribute__((target("avx2,f16c"))) inline void group_dot_tq2_0x4(const PackedRows& P, size_t group, const BlockQ8_K* a, float* out4) {
    const BlockTQ2_0x4* w = (const BlockTQ2_0x4*)P.data.data() + group * P.blocks_per_row;
    __m128 acc = _mm_setzero_ps();
    for (size_t b = 0; b < P.blocks_per_row; ++b) acc = accumulate_tq2_0x4(&w[b], &a[b], acc);
    _mm_storeu_ps(out4, acc);
}

// ---- activation-side pack: four quantised activation rows interleaved per block (BlockQ8_Kx4, types.zig:120-124,
// packed by q8k.zig:539-581): qs byte fg * 16 + r * 4 + l = byte fg * 4 + l of row r; bsums[(s / 4) * 16 + r * 4 + s % 4]
// = bsums[s] of row r. A weight pack multiplied against it loads and unpacks every weight chunk once for four
// activation rows (accumulateQ4_Kx8Q8_Kx4, q4_k.zig:1796-1870; accumulateQ5_Kx8Q8_Kx4, q5_k.zig:887-960): the same
// integers and the same f32 epilogue per (row, column) as the one-row form, so the results are bit-equal.
struct BlockQ8_Kx4 {
    float d[4];
    int8_t qs[1024];
    int16_t bsums[64];
};
static_assert(sizeof(BlockQ8_Kx4) == 1168, "packed activation block size");

// rows r0 .. r0 + 3 of compact Q8_K rows (stride `astride` bytes); rows at or past m are zero rows
void pack_q8_kx4(const uint8_t* qa, size_t astride, size_t m, size_t r0, size_t blocks_per_row, BlockQ8_Kx4* dst) {
    for (size_t b = 0; b < blocks_per_row; ++b) {
        BlockQ8_Kx4* d = dst + b;
        memset(d, 0, sizeof *d);
        for (int r = 0; r < 4; ++r) {
            if (r0 + r >= m) continue;
            const BlockQ8_K* src = (const BlockQ8_K*)(qa + (r0 + r) * astride) + b;
            d->d[r] = src->d;
            for (int fg = 0; fg < 64; ++fg) memcpy(d->qs + fg * 16 + r * 4, src->qs + fg * 4, 4);
            for (int sb = 0; sb < 16; ++sb) d->bsums[(sb / 4) * 16 + r * 4 + sb % 4] = src->bsums[sb];
        }
    }
}
inline int32_t kx4_bsum32(const BlockQ8_Kx4* a, int sub, int r) {  // sum of the 32 elements of sub-block `sub` of row r
    const int s0 = 2 * sub, s1 = 2 * sub + 1;
    return (int32_t)a->bsums[(s0 / 4) * 16 + r * 4 + s0 % 4] + (int32_t)a->bsums[(s1 / 4) * 16 + r * 4 + s1 % 4];
}

__attribute__((target("avx2,f16c"))) inline void accumulate_q4_kx8_x4(const BlockQ4_Kx8* w, const BlockQ8_Kx4* a, __m256 (&acc)[4]) {
    const __m256i low_mask = _mm256_set1_epi8(0x0f), ones = _mm256_set1_epi16(1);
    __m256i iscale[4], imin[4];
    for (int r = 0; r < 4; ++r) iscale[r] = imin[r] = _mm256_setzero_si256();
    for (int pair = 0; pair < 4; ++pair) {
        const int even = 2 * pair, odd = even + 1;
        __m256i sum_e[4], sum_o[4];
        for (int r = 0; r < 4; ++r) sum_e[r] = sum_o[r] = _mm256_setzero_si256();
        for (int fg = 0; fg < 8; ++fg) {
            const __m256i q = _mm256_loadu_si256((const __m256i*)(w->qs + pair * 256 + fg * 32));
            const __m256i w_e = _mm256_and_si256(q, low_mask), w_o = _mm256_and_si256(_mm256_srli_epi16(q, 4), low_mask);
            for (int r = 0; r < 4; ++r) {
                sum_e[r] = _mm256_add_epi32(sum_e[r], _mm256_madd_epi16(_mm256_maddubs_epi16(w_e, bcast4(a->qs + pair * 256 + fg * 16 + r * 4)), ones));
                sum_o[r] = _mm256_add_epi32(sum_o[r], _mm256_madd_epi16(_mm256_maddubs_epi16(w_o, bcast4(a->qs + pair * 256 + 128 + fg * 16 + r * 4)), ones));
            }
        }
        const __m256i sc_e = widen_u8x8(w->scales + even * 8), sc_o = widen_u8x8(w->scales + odd * 8);
        const __m256i mn_e = widen_u8x8(w->mins + even * 8), mn_o = widen_u8x8(w->mins + odd * 8);
        for (int r = 0; r < 4; ++r) {
            iscale[r] = _mm256_add_epi32(iscale[r], _mm256_add_epi32(_mm256_mullo_epi32(sum_e[r], sc_e), _mm256_mullo_epi32(sum_o[r], sc_o)));
            imin[r] = _mm256_add_epi32(imin[r], _mm256_add_epi32(_mm256_mullo_epi32(_mm256_set1_epi32(kx4_bsum32(a, even, r)), mn_e),
                                                                _mm256_mullo_epi32(_mm256_set1_epi32(kx4_bsum32(a, odd, r)), mn_o)));
        }
    }
    for (int r = 0; r < 4; ++r) acc[r] = epilogue_x8(w->d, w->dmin, a->d[r], iscale[r], imin[r], acc[r]);
}

__attribute__((target("avx2,f16c"))) inline void accumulate_q5_kx8_x4(const BlockQ5_Kx8* w, const BlockQ8_Kx4* a, __m256 (&acc)[4]) {
    const __m256i ones = _mm256_set1_epi16(1);
    __m256i iscale[4], imin[4];
    for (int r = 0; r < 4; ++r) iscale[r] = imin[r] = _mm256_setzero_si256();
    for (int sub = 0; sub < 8; ++sub) {
        __m256i sum[4];
        for (int r = 0; r < 4; ++r) sum[r] = _mm256_setzero_si256();
        for (int fg = 0; fg < 8; ++fg) {
            const __m256i q = _mm256_loadu_si256((const __m256i*)(w->qs + sub * 256 + fg * 32));
            for (int r = 0; r < 4; ++r)
                sum[r] = _mm256_add_epi32(sum[r], _mm256_madd_epi16(_mm256_maddubs_epi16(q, bcast4(a->qs + sub * 128 + fg * 16 + r * 4)), ones));
        }
        const __m256i sc = widen_u8x8(w->scales + sub * 8), mn = widen_u8x8(w->mins + sub * 8);
        for (int r = 0; r < 4; ++r) {
            iscale[r] = _mm256_add_epi32(iscale[r], _mm256_mullo_epi32(sum[r], sc));
            imin[r] = _mm256_add_epi32(imin[r], _mm256_mullo_epi32(_mm256_set1_epi32(kx4_bsum32(a, sub, r)), mn));
        }
    }
    for (int r = 0; r < 4; ++r) acc[r] = epilogue_x8(w->d, w->dmin, a->d[r], iscale[r], imin[r], acc[r]);
}

// eight columns x four activation rows: out[r * ldo + 0..7] for the valid rows of the group
__attribute__((target("avx2,f16c"))) inline void group_dot_x8_rows4(const PackedRows& P, size_t group, const BlockQ8_Kx4* a, int valid_rows, float* out,
                                                                   size_t ldo) {
    __m256 acc[4] = {_mm256_setzero_ps(), _mm256_setzero_ps(), _mm256_setzero_ps(), _mm256_setzero_ps()};
    if (P.fmt == Q4_K) {
        const BlockQ4_Kx8* w = (const BlockQ4_Kx8*)P.data.data() + group * P.blocks_per_row;
        for (size_t b = 0; b < P.blocks_per_row; ++b) accumulate_q4_kx8_x4(&w[b], &a[b], acc);
    } else {
        const BlockQ5_Kx8* w = (const BlockQ5_Kx8*)P.data.data() + group * P.blocks_per_row;
        for (size_t b = 0; b < P.blocks_per_row; ++b) accumulate_q5_kx8_x4(&w[b], &a[b], acc);
    }
    for (int r = 0; r < valid_rows; ++r) _mm256_storeu_ps(out + (size_t)r * ldo, acc[r]);
}

// Q6_K: four rows interleaved per block with the levels re-centred to signed bytes at pack time (BlockQ6_Kx4,
// types.zig:125-129, packed by q6_k.zig:56-98): scales[g * 4 + c] = scale g of column c; qs byte
// g * 64 + fg * 16 + c * 4 + l = level - 32 of element g * 16 + fg * 4 + l of column c. Per 16-element group the four
// columns' dots against a broadcast of the activations, times the group's scale; f32(total) * (d_c * d_a) at the end
// of the block: bit-equal to the compact kernel.
struct BlockQ6_Kx4 {
    uint16_t d[4];
    int8_t scales[64];
    int8_t qs[1024];
};
static_assert(sizeof(BlockQ6_Kx4) == 1096, "packed block size");

__attribute__((target("avx2,f16c"))) inline __m128 accumulate_q6_kx4(const BlockQ6_Kx4* w, const BlockQ8_K* a, __m128 acc) {
    const __m256i ones = _mm256_set1_epi16(1);
    __m128i iacc = _mm_setzero_si128();
    for (int g = 0; g < 16; ++g) {
        __m256i sum = _mm256_setzero_si256();
        for (int fg2 = 0; fg2 < 2; ++fg2) {
            const __m256i r = _mm256_loadu_si256((const __m256i*)(w->qs + g * 64 + fg2 * 32));  // feature groups 2 fg2 | 2 fg2 + 1
            int32_t lo, hi;
            memcpy(&lo, a->qs + g * 16 + fg2 * 8, 4);
            memcpy(&hi, a->qs + g * 16 + fg2 * 8 + 4, 4);
            const __m256i b = _mm256_set_m128i(_mm_set1_epi32(hi), _mm_set1_epi32(lo));
            sum = _mm256_add_epi32(sum, _mm256_madd_epi16(_mm256_maddubs_epi16(_mm256_sign_epi8(r, r), _mm256_sign_epi8(b, r)), ones));
        }
        const __m128i dot = _mm_add_epi32(_mm256_castsi256_si128(sum), _mm256_extracti128_si256(sum, 1));
        int32_t sc4;
        memcpy(&sc4, w->scales + g * 4, 4);
        iacc = _mm_add_epi32(iacc, _mm_mullo_epi32(dot, _mm_cvtepi8_epi32(_mm_cvtsi32_si128(sc4))));
    }
    const __m128 dw = _mm_cvtph_ps(_mm_loadl_epi64((const __m128i*)w->d));
    return _mm_add_ps(acc, _mm_mul_ps(_mm_cvtepi32_ps(iacc), _mm_mul_ps(dw, _mm_set1_ps(a->d))));
}
__attribute__((target("avx2,f16c"))) inline void group_dot_q6_kx4(const PackedRows& P, size_t group, const BlockQ8_K* a, float* out4) {
    const BlockQ6_Kx4* w = (const BlockQ6_Kx4*)P.data.data() + group * P.blocks_per_row;
    __m128 acc = _mm_setzero_ps();
    for (size_t b = 0; b < P.blocks_per_row; ++b) acc = accumulate_q6_kx4(&w[b], &a[b], acc);
    _mm_storeu_ps(out4, acc);
}

// eight outputs (rows 8 * group .. + 7 of the packed matrix) against one quantised activation row, blocks ascending
__attribute__((target("avx2,f16c"))) inline void group_dot_x8(const PackedRows& P, size_t group, const BlockQ8_K* a, float* out8) {
    __m256 acc = _mm256_setzero_ps();
    if (P.fmt == Q4_K) {
        const BlockQ4_Kx8* w = (const BlockQ4_Kx8*)P.data.data() + group * P.blocks_per_row;
        for (size_t b = 0; b < P.blocks_per_row; ++b) acc = accumulate_q4_kx8(&w[b], &a[b], acc);
    } else {
        const BlockQ5_Kx8* w = (const BlockQ5_Kx8*)P.data.data() + group * P.blocks_per_row;
        for (size_t b = 0; b < P.blocks_per_row; ++b) acc = accumulate_q5_kx8(&w[b], &a[b], acc);
    }
    _mm256_storeu_ps(out8, acc);
}

bool x8_supported() {
    static const bool ok = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("f16c");
    return ok;
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

// ---- eight-row packs: the reference's load-time repack and its kernels (see the header comment) ----
// Packs n rows of Q4_K or Q5_K blocks (n a multiple of 8) or of Q6_K / Q8_0 / TQ2_0 blocks (a multiple of 4); returns an opaque
// handle, or null when the format has no pack, n does not fit or the host lacks AVX2 / F16C.
void* cpuk_pack_rows(int fmt, const void* w, size_t nb01, size_t n, size_t k) {
    if (!x8_supported() || n == 0 || k == 0 || row_bytes(fmt, k) == 0 || nb01 < row_bytes(fmt, k)) return nullptr;
    const uint8_t* wb = (const uint8_t*)w;
    if (fmt == Q8_0) {
        if (n % 4 != 0) return nullptr;
        PackedRows* P = new PackedRows();
        P->fmt = fmt, P->group = 4, P->n = n, P->k = k, P->blocks_per_row = k / 32;
        P->data.resize((n / 4) * P->blocks_per_row * sizeof(BlockQ8_0x4));
#pragma omp parallel for schedule(static) num_threads(workers())
        for (long long g = 0; g < (long long)(n / 4); ++g)
            for (size_t b = 0; b < P->blocks_per_row; ++b) {
                BlockQ8_0x4* d = (BlockQ8_0x4*)P->data.data() + (size_t)g * P->blocks_per_row + b;
                for (int c = 0; c < 4; ++c) {
                    const BlockQ8_0* src = (const BlockQ8_0*)(wb + ((size_t)g * 4 + c) * nb01) + b;
                    d->d[c] = src->d;
                    for (int fg = 0; fg < 8; ++fg) memcpy(d->qs + fg * 16 + c * 4, src->qs + fg * 4, 4);
                }
            }
        return P;
    }
    if (fmt == TQ2_0) {
        if (n % 4 != 0 || k % 256 != 0) return nullptr;
        PackedRows* P = new PackedRows();
        P->fmt = fmt, P->group = 4, P->n = n, P->k = k, P->blocks_per_row = k / 256;
        P->data.resize((n / 4) * P->blocks_per_row * sizeof(BlockTQ2_0x4));
#pragma omp parallel for schedule(static) num_threads(workers())
        for (long long g = 0; g < (long long)(n / 4); ++g)
            for (size_t b = 0; b < P->blocks_per_row; ++b) {
                BlockTQ2_0x4* d = (BlockTQ2_0x4*)P->data.data() + (size_t)g * P->blocks_per_row + b;
                for (int c = 0; c < 4; ++c) {
                    const BlockTQ2_0* src = (const BlockTQ2_0*)(wb + ((size_t)g * 4 + c) * nb01) + b;
                    d->d[c] = src->d;
                    for (int half = 0; half < 2; ++half)
                        for (int fg = 0; fg < 8; ++fg) memcpy(d->qs + half * 128 + fg * 16 + c * 4, src->qs + half * 32 + fg * 4, 4);
                }
            }
        return P;
    }
    if (fmt == Q6_K) {
        if (n % 4 != 0 || k % 256 != 0) return nullptr;
        PackedRows* P = new PackedRows();
        P->fmt = fmt, P->group = 4, P->n = n, P->k = k, P->blocks_per_row = k / 256;
        P->data.resize((n / 4) * P->blocks_per_row * sizeof(BlockQ6_Kx4));
#pragma omp parallel for schedule(static) num_threads(workers())
        for (long long g = 0; g < (long long)(n / 4); ++g)
            for (size_t b = 0; b < P->blocks_per_row; ++b) {
                BlockQ6_Kx4* d = (BlockQ6_Kx4*)P->data.data() + (size_t)g * P->blocks_per_row + b;
                for (int c = 0; c < 4; ++c) {
                    const BlockQ6_K* src = (const BlockQ6_K*)(wb + ((size_t)g * 4 + c) * nb01) + b;
                    d->d[c] = src->d;
                    for (int sg = 0; sg < 16; ++sg) {
                        d->scales[sg * 4 + c] = src->scales[sg];
                        for (int fg = 0; fg < 4; ++fg)
                            for (int l = 0; l < 4; ++l) d->qs[sg * 64 + fg * 16 + c * 4 + l] = q6k_value(src, sg * 16 + fg * 4 + l);
                    }
                }
            }
        return P;
    }
    if ((fmt != Q4_K && fmt != Q5_K) || n % 8 != 0) return nullptr;
    PackedRows* P = new PackedRows();
    P->fmt = fmt, P->n = n, P->k = k, P->blocks_per_row = k / 256;
    const size_t bsz = fmt == Q4_K ? sizeof(BlockQ4_Kx8) : sizeof(BlockQ5_Kx8);
    P->data.resize((n / 8) * P->blocks_per_row * bsz);
#pragma omp parallel for schedule(static) num_threads(workers())
    for (long long g = 0; g < (long long)(n / 8); ++g)
        for (size_t b = 0; b < P->blocks_per_row; ++b) {
            uint8_t* dst = P->data.data() + ((size_t)g * P->blocks_per_row + b) * bsz;
            if (fmt == Q4_K) {
                const BlockQ4_K* cols[8];
                for (int c = 0; c < 8; ++c) cols[c] = (const BlockQ4_K*)(wb + ((size_t)g * 8 + c) * nb01) + b;
                BlockQ4_Kx8* d = (BlockQ4_Kx8*)dst;
                pack_header_x8(cols, d);
                for (int pair = 0; pair < 4; ++pair)
                    for (int fg = 0; fg < 8; ++fg)
                        for (int c = 0; c < 8; ++c) memcpy(d->qs + pair * 256 + fg * 32 + c * 4, cols[c]->qs + pair * 32 + fg * 4, 4);
            } else {
                const BlockQ5_K* cols[8];
                for (int c = 0; c < 8; ++c) cols[c] = (const BlockQ5_K*)(wb + ((size_t)g * 8 + c) * nb01) + b;
                BlockQ5_Kx8* d = (BlockQ5_Kx8*)dst;
                pack_header_x8(cols, d);
                for (int sub = 0; sub < 8; ++sub)
                    for (int fg = 0; fg < 8; ++fg)
                        for (int c = 0; c < 8; ++c)
                            for (int l = 0; l < 4; ++l) d->qs[sub * 256 + fg * 32 + c * 4 + l] = (uint8_t)q5_level(cols[c], sub, fg * 4 + l);
            }
        }
    return P;
}
void cpuk_free_packed(void* packed) { delete (PackedRows*)packed; }
size_t cpuk_packed_bytes(const void* packed) { return packed ? ((const PackedRows*)packed)->data.size() : 0; }

// c[m, n] = a[m, k] . dequant(w)^T over a packed matrix: the same values as cpuk_matmul on the compact blocks.
// Column arm as in cpuk_matmul, in whole groups of eight columns (QuantizedRhsParallel with col_group 8,
// matmul_quant.zig:574-590; for these packs the reference keeps the column arm up to m < 64). Larger products split
// the column groups over all workers here instead of the rows; values do not depend on the split.
int cpuk_matmul_packed(const void* packed, const float* a, float* c, size_t m) {
    if (!packed) return 1;
    const PackedRows& P = *(const PackedRows*)packed;
    size_t astride = 0;
    std::vector<uint8_t> qa = quantize_acts(P.fmt, a, m, P.k, &astride);
    const size_t G = (size_t)P.group, groups = P.n / G;
    const int T = workers();
    const unsigned __int128 work = (unsigned __int128)m * P.n * P.k;
    long long tasks = m < 64 ? (work >= ((unsigned __int128)1 << 20) ? (long long)(P.n / 64) : 1) : T;
    if (tasks > T) tasks = T;
    if (tasks > (long long)groups) tasks = (long long)groups;
    if (tasks < 1) tasks = 1;
    // four or more activation rows against a K-quant pack: the rows are packed four at a time (BlockQ8_Kx4, the last
    // group padded with zero rows) so that every weight chunk is loaded and unpacked once per four rows
    std::vector<BlockQ8_Kx4> a4;
    const bool rows4 = P.group == 8 && m >= 4;
    const size_t row_groups = (m + 3) / 4;
    if (rows4) {
        a4.resize(row_groups * P.blocks_per_row);
#pragma omp parallel for schedule(static) num_threads(T)
        for (long long rg = 0; rg < (long long)row_groups; ++rg)
            pack_q8_kx4(qa.data(), astride, m, (size_t)rg * 4, P.blocks_per_row, a4.data() + (size_t)rg * P.blocks_per_row);
    }
#pragma omp parallel for schedule(static, 1) num_threads((int)tasks)
    for (long long t = 0; t < tasks; ++t) {
        const size_t g0 = groups * (size_t)t / (size_t)tasks, g1 = groups * (size_t)(t + 1) / (size_t)tasks;
        float out8[8];
        for (size_t g = g0; g < g1 && rows4; ++g)
            for (size_t rg = 0; rg < row_groups; ++rg) {
                const size_t left = m - rg * 4;
                group_dot_x8_rows4(P, g, a4.data() + rg * P.blocks_per_row, (int)(left < 4 ? left : 4), c + rg * 4 * P.n + g * 8, P.n);
            }
        for (size_t g = g0; g < g1 && !rows4; ++g)
            for (size_t i = 0; i < m; ++i) {
                if (P.fmt == Q8_0) group_dot_q8_0x4(P, g, (const BlockQ8_0*)(qa.data() + i * astride), out8);
                else if (P.fmt == TQ2_0) group_dot_tq2_0x4(P, g, (const BlockQ8_K*)(qa.data() + i * astride), out8);
                else if (P.fmt == Q6_K) group_dot_q6_kx4(P, g, (const BlockQ8_K*)(qa.data() + i * astride), out8);
                else group_dot_x8(P, g, (const BlockQ8_K*)(qa.data() + i * astride), out8);
                memcpy(c + i * P.n + g * G, out8, G * sizeof(float));
            }
    }
    return 0;
}

// The expert layer over packed stacks (gate / up: n_expert * out_pe rows of `hidden`; down: n_expert * hidden rows of
// out_pe; out_pe and hidden multiples of 8): cpuk_moe_ffn's structure with eight outputs per step.
int cpuk_moe_ffn_packed(const void* gate, const void* up, const void* down, const float* x, size_t seq, size_t hidden, size_t out_pe,
                    size_t n_expert, size_t top_k, const int64_t* selected, const float* weights, float* out) {
    if (!gate || !up || !down) return 1;
    const PackedRows &G = *(const PackedRows*)gate, &U = *(const PackedRows*)up, &D = *(const PackedRows*)down;
    if (G.group != 8 || U.group != 8 || D.group != 8 || hidden % 256 || out_pe % 256 || G.k != hidden || U.k != hidden || D.k != out_pe || G.n != n_expert * out_pe || U.n != G.n || D.n != n_expert * hidden || G.fmt != U.fmt ||
        out_pe % 8 || hidden % 8)
        return 1;
    for (size_t p = 0; p < seq * top_k; ++p)
        if (selected[p] < 0 || (size_t)selected[p] >= n_expert) return 1;
    std::vector<float> pair_out(seq * top_k * hidden);
    const size_t pairs = seq * top_k;
    if (pairs >= 2 * n_expert) {
        // Batched form (exec/moe.zig:1865-2088 `moeExpertFfnBatch`, route plan of exec/moe_chain.zig:236-299): the pairs
        // are grouped by expert and an expert's rows go through its matrices four at a time, so its weights are read
        // and unpacked once per four rows instead of once per pair. Per (row, column) the integers and the f32 epilogue
        // are those of the one-row form: the same bits.
        std::vector<size_t> start(n_expert + 1, 0), order(pairs);
        for (size_t p = 0; p < pairs; ++p) ++start[(size_t)selected[p] + 1];
        for (size_t e = 0; e < n_expert; ++e) start[e + 1] += start[e];
        {
            std::vector<size_t> at(start.begin(), start.end() - 1);
            for (size_t p = 0; p < pairs; ++p) order[at[(size_t)selected[p]]++] = p;
        }
        const size_t bx = hidden / 256, bg = out_pe / 256;
#pragma omp parallel num_threads(workers())
        {
            std::vector<float> xs, gate_v, up_v, gs;
            std::vector<BlockQ8_Kx4> a4;
#pragma omp for schedule(dynamic, 1)
            for (long long e = 0; e < (long long)n_expert; ++e) {
                const size_t rows = start[e + 1] - start[e];
                if (rows == 0) continue;
                const size_t rgs = (rows + 3) / 4;
                xs.resize(rows * hidden), gate_v.resize(rows * out_pe), up_v.resize(rows * out_pe), gs.resize(rows * out_pe);
                for (size_t r = 0; r < rows; ++r) memcpy(xs.data() + r * hidden, x + (order[start[e] + r] / top_k) * hidden, hidden * sizeof(float));
                size_t s_in = 0, s_g = 0;
                std::vector<uint8_t> qx = quantize_acts(G.fmt, xs.data(), rows, hidden, &s_in);
                a4.resize(rgs * (bx > bg ? bx : bg));
                for (size_t rg = 0; rg < rgs; ++rg) pack_q8_kx4(qx.data(), s_in, rows, rg * 4, bx, a4.data() + rg * bx);
                for (size_t j = 0; j < out_pe; j += 8)
                    for (size_t rg = 0; rg < rgs; ++rg) {
                        const int valid = (int)(rows - rg * 4 < 4 ? rows - rg * 4 : 4);
                        group_dot_x8_rows4(G, ((size_t)e * out_pe + j) / 8, a4.data() + rg * bx, valid, gate_v.data() + rg * 4 * out_pe + j, out_pe);
                        group_dot_x8_rows4(U, ((size_t)e * out_pe + j) / 8, a4.data() + rg * bx, valid, up_v.data() + rg * 4 * out_pe + j, out_pe);
                    }
                for (size_t i = 0; i < rows * out_pe; ++i) gs[i] = swiglu_pair(gate_v[i], up_v[i]);
                std::vector<uint8_t> qg = quantize_acts(D.fmt, gs.data(), rows, out_pe, &s_g);
                for (size_t rg = 0; rg < rgs; ++rg) pack_q8_kx4(qg.data(), s_g, rows, rg * 4, bg, a4.data() + rg * bg);
                std::vector<float> rows_out(4 * hidden);
                for (size_t rg = 0; rg < rgs; ++rg) {
                    const int valid = (int)(rows - rg * 4 < 4 ? rows - rg * 4 : 4);
                    for (size_t j = 0; j < hidden; j += 8)
                        group_dot_x8_rows4(D, ((size_t)e * hidden + j) / 8, a4.data() + rg * bg, valid, rows_out.data() + j, hidden);
                    for (int r = 0; r < valid; ++r)
                        memcpy(pair_out.data() + order[start[e] + rg * 4 + r] * hidden, rows_out.data() + (size_t)r * hidden, hidden * sizeof(float));
                }
            }
        }
    } else
#pragma omp parallel num_threads(workers())
    {
        std::vector<float> gate_v(out_pe), up_v(out_pe), g(out_pe);
#pragma omp for schedule(dynamic, 1)
        for (long long p = 0; p < (long long)(seq * top_k); ++p) {
            const size_t t = (size_t)p / top_k;
            const size_t e = (size_t)selected[p];
            size_t s_in = 0, s_g = 0;
            std::vector<uint8_t> qx = quantize_acts(G.fmt, x + t * hidden, 1, hidden, &s_in);
            for (size_t j = 0; j < out_pe; j += 8) {
                group_dot_x8(G, (e * out_pe + j) / 8, (const BlockQ8_K*)qx.data(), gate_v.data() + j);
                group_dot_x8(U, (e * out_pe + j) / 8, (const BlockQ8_K*)qx.data(), up_v.data() + j);
            }
            for (size_t j = 0; j < out_pe; ++j) g[j] = swiglu_pair(gate_v[j], up_v[j]);
            std::vector<uint8_t> qg = quantize_acts(D.fmt, g.data(), 1, out_pe, &s_g);
            float* po = pair_out.data() + (size_t)p * hidden;
            for (size_t j = 0; j < hidden; j += 8) group_dot_x8(D, (e * hidden + j) / 8, (const BlockQ8_K*)qg.data(), po + j);
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
