// TEST INFRASTRUCTURE ONLY -- CPU oracle for the quantized-matmul path.
//
// A plain C++ restatement of the reference's CPU arithmetic for GGUF block
// quantized weight x activation products. Nothing in the shipped library may
// link or call this file; it exists so tests, the smoke check and the bench's
// CPU-baseline leg have something independent to compare against.
//
// Parity is PINNED: the encoders reproduce the reference's stored ggml golden
// blocks byte for byte and the decoders reproduce its stored f32 bit patterns
// (see tests/golden and tests/test_oracle_golden.py).
//
// Every function names the reference file:line it follows (paths relative to
// the reference project root). All float arithmetic is f32, evaluated in the
// written order; build with -ffp-contract=off so nothing is fused.
#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <vector>

namespace {

// ---- f16 <-> f32 (src/backend/quant/common.zig:87-95: IEEE RNE both ways) --
inline float h2f(uint16_t bits) {
    _Float16 h;
    std::memcpy(&h, &bits, 2);
    return (float)h;
}
inline uint16_t f2h(float x) {
    _Float16 h = (_Float16)x;
    uint16_t bits;
    std::memcpy(&bits, &h, 2);
    return bits;
}

// ---- block layouts (src/dtype.zig:78-86, :128-152, :215-218;
//      src/backend/quant/types.zig:177-180) ---------------------------------
#pragma pack(push, 1)
struct BlockQ8_0 { uint16_t d; int8_t qs[32]; };
struct BlockQ4_K { uint16_t dm[2]; uint8_t scales[12]; uint8_t qs[128]; };
struct BlockQ5_K { uint16_t dm[2]; uint8_t scales[12]; uint8_t qh[32]; uint8_t qs[128]; };
struct BlockQ6_K { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; };  // dtype.zig:141-146
struct BlockQ8_K { float d; int8_t qs[256]; int16_t bsums[16]; };
struct BlockTQ2_0 { uint8_t qs[64]; uint16_t d; };
struct BlockTQ2_0Folded { uint8_t qs[128]; uint16_t d; };
struct BlockQ2_0 { uint16_t d; uint8_t qs[32]; };
#pragma pack(pop)
static_assert(sizeof(BlockQ8_0) == 34, "");
static_assert(sizeof(BlockQ4_K) == 144, "");
static_assert(sizeof(BlockQ5_K) == 176, "");
static_assert(sizeof(BlockQ6_K) == 210, "");
static_assert(sizeof(BlockQ8_K) == 292, "");
static_assert(sizeof(BlockTQ2_0) == 66, "");
static_assert(sizeof(BlockTQ2_0Folded) == 130, "");
static_assert(sizeof(BlockQ2_0) == 34, "");

// ---- rounding helpers ------------------------------------------------------
// common.zig:33-40: round half away from zero, clamp to +-127.
inline int8_t quantize_to_i8(float x) {
    float r = std::round(x);
    r = std::max(-127.0f, std::min(127.0f, r));
    return (int8_t)r;
}
// common.zig:42-49.
inline float round_nearest_even(float x) {
    float rounded = std::round(x);
    if (std::fabs(rounded - x) == 0.5f) {
        int32_t ri = (int32_t)rounded;
        if ((ri % 2) != 0) rounded -= (x < 0) ? -1.0f : 1.0f;
    }
    return rounded;
}
// q8k.zig:650-655: the 12582912.0f magic-add nearest-int.
inline int32_t nearest_int(float fval) {
    float val = fval + 12582912.0f;
    int32_t bits;
    std::memcpy(&bits, &val, 4);
    return (bits & 0x007fffff) - 0x00400000;
}

// q8k.zig:637-648.
inline void get_scale_min_k4(const uint8_t* q, int j, uint8_t* sc, uint8_t* mn) {
    if (j < 4) {
        *sc = q[j] & 63;
        *mn = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0x0f) | ((q[j - 4] >> 6) << 4));
        *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

// ---- Q8_0 (q8k.zig:49-69 non-aarch64 arm, :95-114) -------------------------
void quantize_row_q8_0(BlockQ8_0* dst, const float* src, size_t k) {
    for (size_t b = 0; b < k / 32; ++b) {
        const float* row = src + b * 32;
        float amax = 0;
        for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(row[i]));
        const float d = amax / 127.0f;
        const float inv_d = (d == 0) ? 0.0f : 1.0f / d;
        dst[b].d = f2h(d);
        for (int i = 0; i < 32; ++i) dst[b].qs[i] = quantize_to_i8(row[i] * inv_d);
    }
}
void dequantize_row_q8_0(float* dst, const BlockQ8_0* src, size_t k) {
    for (size_t b = 0; b < k / 32; ++b) {
        const float d = h2f(src[b].d);
        for (int i = 0; i < 32; ++i) dst[b * 32 + i] = (float)src[b].qs[i] * d;
    }
}

// ---- Q8_K activations (q8k.zig:268-313) ------------------------------------
void quantize_row_q8_k(BlockQ8_K* dst, const float* src, size_t k) {
    for (size_t b = 0; b < k / 256; ++b) {
        const float* row = src + b * 256;
        float amax = 0;
        for (int i = 0; i < 256; ++i) amax = std::max(amax, std::fabs(row[i]));
        float max_value = 0;
        for (int i = 0; i < 256; ++i) {
            if (std::fabs(row[i]) == amax) { max_value = row[i]; break; }
        }
        if (amax == 0) {
            dst[b].d = 0;
            std::memset(dst[b].qs, 0, 256);
            std::memset(dst[b].bsums, 0, 32);
            continue;
        }
        const float inv_scale = -127.0f / max_value;
        for (int i = 0; i < 256; ++i) {
            const float q = round_nearest_even(inv_scale * row[i]);
            dst[b].qs[i] = (int8_t)std::min(127.0f, q);
        }
        for (int g = 0; g < 16; ++g) {
            int32_t acc = 0;
            for (int i = 0; i < 16; ++i) acc += dst[b].qs[g * 16 + i];
            dst[b].bsums[g] = (int16_t)acc;
        }
        dst[b].d = 1.0f / inv_scale;
    }
}

// ---- make_qkx2_quants (q8k.zig:734-818) ------------------------------------
float make_qkx2_quants(int nmax, const float* x, const float* weights, uint8_t* L, float* the_min,
                       uint8_t* Laux, float rmin, float rdelta, int nstep, bool use_mad) {
    const int n = 32;
    float min = x[0], max = x[0];
    float sum_w = weights[0];
    float sum_x = sum_w * x[0];
    for (int i = 1; i < n; ++i) {
        if (x[i] < min) min = x[i];
        if (x[i] > max) max = x[i];
        sum_w += weights[i];
        sum_x += weights[i] * x[i];
    }
    if (min > 0) min = 0;
    if (max == min) {
        std::memset(L, 0, n);
        *the_min = -min;
        return 0;
    }
    const float nmax_f = (float)nmax;
    float iscale = nmax_f / (max - min);
    float scale = 1 / iscale;
    float best_error = 0;
    for (int i = 0; i < n; ++i) {
        int l = nearest_int(iscale * (x[i] - min));
        L[i] = (uint8_t)std::max(0, std::min(nmax, l));
        float diff = scale * (float)L[i] + min - x[i];
        diff = use_mad ? std::fabs(diff) : diff * diff;
        best_error += weights[i] * diff;
    }
    if (nstep < 1) {
        *the_min = -min;
        return scale;
    }
    for (int is = 0; is <= nstep; ++is) {
        iscale = (rmin + rdelta * (float)is + nmax_f) / (max - min);
        float sum_l = 0, sum_l2 = 0, sum_xl = 0;
        for (int i = 0; i < n; ++i) {
            int l = nearest_int(iscale * (x[i] - min));
            l = std::max(0, std::min(nmax, l));
            Laux[i] = (uint8_t)l;
            const float lf = (float)l;
            sum_l += weights[i] * lf;
            sum_l2 += weights[i] * lf * lf;
            sum_xl += weights[i] * lf * x[i];
        }
        const float determinant = sum_w * sum_l2 - sum_l * sum_l;
        if (determinant > 0) {
            float this_scale = (sum_w * sum_xl - sum_x * sum_l) / determinant;
            float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / determinant;
            if (this_min > 0) {
                this_min = 0;
                this_scale = sum_xl / sum_l2;
            }
            float cur_error = 0;
            for (int i = 0; i < n; ++i) {
                float diff = this_scale * (float)Laux[i] + this_min - x[i];
                diff = use_mad ? std::fabs(diff) : diff * diff;
                cur_error += weights[i] * diff;
            }
            if (cur_error < best_error) {
                std::memcpy(L, Laux, n);
                best_error = cur_error;
                scale = this_scale;
                min = this_min;
            }
        }
    }
    *the_min = -min;
    return scale;
}

// Shared first half of the Q4_K / Q5_K block encoders
// (q4_k.zig:1977-2030, q5_k.zig:1172-1228): per-sub-block search, 6-bit scale
// packing, and the re-derivation of every level against the rounded scales.
void kquant_levels(const float* src, int nmax, float rmin, int nstep, uint16_t dm[2],
                   uint8_t scales_out[12], uint8_t L[256]) {
    uint8_t Laux[32];
    float weights[32], mins[8], scales[8];
    float max_scale = 0, max_min = 0;
    for (int j = 0; j < 8; ++j) {
        const float* xs = src + 32 * j;
        float sum_x2 = 0;
        for (int i = 0; i < 32; ++i) sum_x2 += xs[i] * xs[i];
        const float av_x = std::sqrt(sum_x2 / 32);
        for (int i = 0; i < 32; ++i) weights[i] = av_x + std::fabs(xs[i]);
        scales[j] = make_qkx2_quants(nmax, xs, weights, L + 32 * j, &mins[j], Laux, rmin, 0.1f, nstep, false);
        if (scales[j] > max_scale) max_scale = scales[j];
        if (mins[j] > max_min) max_min = mins[j];
    }
    const float inv_scale = max_scale > 0 ? 63.0f / max_scale : 0.0f;
    const float inv_min = max_min > 0 ? 63.0f / max_min : 0.0f;
    std::memset(scales_out, 0, 12);
    for (int j = 0; j < 8; ++j) {
        // the rounded int is truncated to u8 before the 63 clamp
        uint8_t ls = (uint8_t)(uint32_t)nearest_int(inv_scale * scales[j]);
        uint8_t lm = (uint8_t)(uint32_t)nearest_int(inv_min * mins[j]);
        ls = std::min<uint8_t>(63, ls);
        lm = std::min<uint8_t>(63, lm);
        if (j < 4) {
            scales_out[j] = ls;
            scales_out[j + 4] = lm;
        } else {
            scales_out[j + 4] = (uint8_t)((ls & 0x0f) | ((lm & 0x0f) << 4));
            scales_out[j - 4] |= (uint8_t)((ls >> 4) << 6);
            scales_out[j] |= (uint8_t)((lm >> 4) << 6);
        }
    }
    dm[0] = f2h(max_scale / 63.0f);
    dm[1] = f2h(max_min / 63.0f);
    for (int j = 0; j < 8; ++j) {
        uint8_t sc, mn;
        get_scale_min_k4(scales_out, j, &sc, &mn);
        const float d = h2f(dm[0]) * (float)sc;
        if (d == 0) continue;  // keeps the search's levels
        const float dmv = h2f(dm[1]) * (float)mn;
        for (int i = 0; i < 32; ++i) {
            int l = nearest_int((src[32 * j + i] + dmv) / d);
            L[32 * j + i] = (uint8_t)std::max(0, std::min(nmax, l));
        }
    }
}

// q4_k.zig:1977-2039.
void quantize_block_q4_k(BlockQ4_K* dst, const float* src) {
    uint8_t L[256];
    kquant_levels(src, 15, -1.0f, 20, dst->dm, dst->scales, L);
    int qs_offset = 0;
    for (int j = 0; j < 256; j += 64) {
        for (int l = 0; l < 32; ++l) dst->qs[qs_offset + l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 4));
        qs_offset += 32;
    }
}
// q5_k.zig:1172-1248.
void quantize_block_q5_k(BlockQ5_K* dst, const float* src) {
    uint8_t L[256];
    kquant_levels(src, 31, -0.5f, 15, dst->dm, dst->scales, L);
    std::memset(dst->qh, 0, 32);
    int qs_offset = 0;
    for (int n = 0; n < 256; n += 64) {
        const int shift = (n / 64) * 2;
        const uint8_t m1 = (uint8_t)(1u << shift), m2 = (uint8_t)(2u << shift);
        for (int jj = 0; jj < 32; ++jj) {
            uint8_t l1 = L[n + jj];
            if (l1 > 15) { l1 -= 16; dst->qh[jj] |= m1; }
            uint8_t l2 = L[n + jj + 32];
            if (l2 > 15) { l2 -= 16; dst->qh[jj] |= m2; }
            dst->qs[qs_offset + jj] = (uint8_t)(l1 | (l2 << 4));
        }
        qs_offset += 32;
    }
}

// q4_k.zig:1954-1972.
inline uint8_t q4k_value(const BlockQ4_K* w, int s, int i) {
    const uint8_t byte = w->qs[(s / 2) * 32 + i];
    return (s % 2 == 0) ? (byte & 0x0f) : (byte >> 4);
}
void dequantize_block_q4_k(float* dst, const BlockQ4_K* src) {
    const float d = h2f(src->dm[0]), dmin = h2f(src->dm[1]);
    for (int s = 0; s < 8; ++s) {
        uint8_t sc, mn;
        get_scale_min_k4(src->scales, s, &sc, &mn);
        for (int i = 0; i < 32; ++i) {
            const float q = (float)q4k_value(src, s, i);
            dst[s * 32 + i] = d * (float)sc * q - dmin * (float)mn;
        }
    }
}
// q5_k.zig:1154-1167, :1259-1264.
inline uint8_t q5k_value(const BlockQ5_K* w, int s, int i) {
    const uint8_t byte = w->qs[(s / 2) * 32 + i];
    const uint8_t low = (s % 2 == 0) ? (byte & 0x0f) : (byte >> 4);
    return (uint8_t)(low + (((w->qh[i] >> s) & 1) ? 16 : 0));
}
void dequantize_block_q5_k(float* dst, const BlockQ5_K* src) {
    const float d = h2f(src->dm[0]), dmin = h2f(src->dm[1]);
    for (int s = 0; s < 8; ++s) {
        uint8_t sc, mn;
        get_scale_min_k4(src->scales, s, &sc, &mn);
        for (int i = 0; i < 32; ++i) {
            const float q = (float)q5k_value(src, s, i);
            dst[s * 32 + i] = d * (float)sc * q - dmin * (float)mn;
        }
    }
}

// ---- ternary (ternary.zig:79-144, ptqtp.zig:684-697, cold.zig:651-670) -----
// ---- Q6_K (backend/quant/q6_k.zig) ------------------------------------------
// q6_k.zig:1239-1259: element `index` of a block: chunk of 128, section of 32; low nibble of ql for sections 0-1,
// high nibble for 2-3; two bits of qh; value minus 32. One i8 scale per 16 elements.
inline int8_t q6k_value(const BlockQ6_K* w, int index) {
    const int chunk = index / 128, local = index % 128, section = local / 32, l = local % 32;
    const int ql_index = chunk * 64 + ((section == 1 || section == 3) ? 32 + l : l);
    const int low = (section < 2) ? (w->ql[ql_index] & 0x0f) : (w->ql[ql_index] >> 4);
    const int high = (w->qh[chunk * 32 + l] >> (section * 2)) & 0x03;
    return (int8_t)((low | (high << 4)) - 32);
}
inline int q6k_scale_index(int index) {
    const int chunk = index / 128, local = index % 128, section = local / 32, l = local % 32;
    return chunk * 8 + section * 2 + l / 16;
}
// q6_k.zig:1159-1167: d * f32(scale) * f32(q), left to right.
void dequantize_block_q6_k(float* dst, const BlockQ6_K* src) {
    const float d = h2f(src->d);
    for (int i = 0; i < 256; ++i) dst[i] = d * (float)src->scales[q6k_scale_index(i)] * (float)q6k_value(src, i);
}
// q8k.zig:665-733 `makeQxQuants` without an external weight table (qw = null): the rmse_type-weighted scale
// search ggml's make_qx_quants does. n elements, levels in [-nmax, nmax - 1] stored biased by nmax.
float make_qx_quants(int nmax, const float* x, int n, int8_t* L, int rmse_type_in) {
    auto weight = [](int rmse_type, float v) -> float {
        switch (rmse_type) {
            case 1: return v * v;
            case 2: return 1.0f;
            case 3: return std::fabs(v);
            default: return std::sqrt(std::fabs(v));
        }
    };
    float max = 0, amax = 0;
    for (int i = 0; i < n; ++i) {
        const float ax = std::fabs(x[i]);
        if (ax > amax) {
            amax = ax;
            max = x[i];
        }
    }
    if (amax < 1e-15f) {  // group_max_eps: all zero
        for (int i = 0; i < n; ++i) L[i] = 0;
        return 0.0f;
    }
    const float nmax_f = (float)nmax;
    float iscale = -nmax_f / max;
    int rmse_type = rmse_type_in;
    if (rmse_type == 0) {
        for (int i = 0; i < n; ++i) {
            const int l = nearest_int(iscale * x[i]);
            L[i] = (int8_t)(nmax + std::max(-nmax, std::min(nmax - 1, l)));
        }
        return 1 / iscale;
    }
    bool return_early = false;
    if (rmse_type < 0) {
        rmse_type = -rmse_type;
        return_early = true;
    }
    float sumlx = 0, suml2 = 0;
    for (int i = 0; i < n; ++i) {
        int l = nearest_int(iscale * x[i]);
        l = std::max(-nmax, std::min(nmax - 1, l));
        L[i] = (int8_t)(l + nmax);
        const float w = weight(rmse_type, x[i]);
        const float lf = (float)l;
        sumlx += w * x[i] * lf;
        suml2 += w * lf * lf;
    }
    float scale = (suml2 != 0) ? sumlx / suml2 : 0.0f;
    if (return_early) return (suml2 > 0) ? 0.5f * (scale + 1 / iscale) : 1 / iscale;
    float best = scale * sumlx;
    for (int is = -9; is <= 9; ++is) {
        if (is == 0) continue;
        iscale = -(nmax_f + 0.1f * (float)is) / max;
        sumlx = 0;
        suml2 = 0;
        for (int i = 0; i < n; ++i) {
            int l = nearest_int(iscale * x[i]);
            l = std::max(-nmax, std::min(nmax - 1, l));
            const float w = weight(rmse_type, x[i]);
            const float lf = (float)l;
            sumlx += w * x[i] * lf;
            suml2 += w * lf * lf;
        }
        if (suml2 > 0 && sumlx * sumlx > best * suml2) {
            for (int i = 0; i < n; ++i) {
                const int l = nearest_int(iscale * x[i]);
                L[i] = (int8_t)(nmax + std::max(-nmax, std::min(nmax - 1, l)));
            }
            scale = sumlx / suml2;
            best = scale * sumlx;
        }
    }
    return scale;
}
// q6_k.zig:1172-1229, the port of ggml's quantize_row_q6_K_ref.
void quantize_block_q6_k(BlockQ6_K* dst, const float* src) {
    int8_t L[256];
    float scales[16];
    float max_scale = 0, max_abs_scale = 0;
    for (int ib = 0; ib < 16; ++ib) {
        const float scale = make_qx_quants(32, src + 16 * ib, 16, L + 16 * ib, 1);
        scales[ib] = scale;
        const float abs_scale = std::fabs(scale);
        if (abs_scale > max_abs_scale) {
            max_abs_scale = abs_scale;
            max_scale = scale;
        }
    }
    if (max_abs_scale < 1e-15f) {
        std::memset(dst, 0, sizeof *dst);
        return;
    }
    const float iscale = -128.0f / max_scale;
    dst->d = f2h(1 / iscale);
    for (int ib = 0; ib < 16; ++ib) dst->scales[ib] = (int8_t)std::min(127, nearest_int(iscale * scales[ib]));
    for (int j = 0; j < 16; ++j) {
        const float d = h2f(dst->d) * (float)dst->scales[j];
        if (d == 0) continue;  // keeps the make_qx_quants levels, like ggml
        for (int i = 0; i < 16; ++i) {
            const int l = nearest_int(src[16 * j + i] / d);
            L[16 * j + i] = (int8_t)(std::max(-32, std::min(31, l)) + 32);
        }
    }
    for (int j = 0, ql_offset = 0, qh_offset = 0; j < 256; j += 128, ql_offset += 64, qh_offset += 32)
        for (int l = 0; l < 32; ++l) {
            const uint8_t q1 = (uint8_t)L[j + l], q2 = (uint8_t)L[j + l + 32], q3 = (uint8_t)L[j + l + 64], q4 = (uint8_t)L[j + l + 96];
            dst->ql[ql_offset + l] = (uint8_t)((q1 & 0x0f) | ((q3 & 0x0f) << 4));
            dst->ql[ql_offset + l + 32] = (uint8_t)((q2 & 0x0f) | ((q4 & 0x0f) << 4));
            dst->qh[qh_offset + l] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
        }
}

inline int tq2_code(const BlockTQ2_0* b, int e) {
    const int hg = e / 128, n = (e % 128) / 32, m = e % 32;
    return (b->qs[hg * 32 + m] >> (2 * n)) & 3;
}
void encode_crumbs(BlockTQ2_0* block, const float* x, float id) {
    for (int group = 0; group < 2; ++group) {
        for (int m = 0; m < 32; ++m) {
            uint8_t q = 0;
            for (int n = 0; n < 4; ++n) {
                const float rounded = std::round(x[group * 128 + n * 32 + m] * id);
                const float bounded = std::isnan(rounded) ? 0.0f : std::min(1.0f, std::max(-1.0f, rounded));
                const int xi = (int)bounded;
                q = (uint8_t)(q + (((xi + 1) & 3) << (2 * n)));
            }
            block->qs[group * 32 + m] = q;
        }
    }
}
void quantize_row_tq2_0(BlockTQ2_0* dst, const float* src, size_t k) {
    for (size_t b = 0; b < k / 256; ++b) {
        const float* x = src + b * 256;
        float amax = 0;
        for (int i = 0; i < 256; ++i) amax = std::max(amax, std::fabs(x[i]));
        const float d = amax;
        const float id = (d != 0) ? 1.0f / d : 0.0f;
        dst[b].d = f2h(d);
        encode_crumbs(&dst[b], x, id);
    }
}
void dequantize_row_tq2_0(float* dst, const BlockTQ2_0* src, size_t k) {
    for (size_t b = 0; b < k / 256; ++b) {
        const float d = h2f(src[b].d);
        size_t offset = 0;
        for (int j = 0; j < 64; j += 32)
            for (int lane = 0; lane < 4; ++lane)
                for (int m = 0; m < 32; ++m) {
                    const int q = (src[b].qs[j + m] >> (lane * 2)) & 3;
                    dst[b * 256 + offset++] = (float)(q - 1) * d;
                }
    }
}
// ternary.zig:659-666 (foldedCode), :707-735 (row-major fold).
inline uint8_t folded_code(const BlockTQ2_0* b1, const BlockTQ2_0* b2, int e) {
    return (uint8_t)(3 * tq2_code(b1, e) + tq2_code(b2, e));
}
// ternary.zig:850-876 decode law on the row-major block (types.zig:177-180).
inline int folded_cu(const BlockTQ2_0Folded* b, int e) {
    const int s = e / 32, j = e % 32;
    return (j < 16) ? (b->qs[s * 16 + j] & 0x0f) : (b->qs[s * 16 + j - 16] >> 4);
}
// cold.zig:285-301, :309-332.
void quantize_row_q2_0(BlockQ2_0* dst, const float* src, size_t k) {
    for (size_t b = 0; b < k / 128; ++b) {
        const float* x = src + b * 128;
        float amax = 0;
        for (int i = 0; i < 128; ++i) amax = std::max(amax, std::fabs(x[i]));
        const float d = amax;
        float inv_d = (d != 0) ? 1.0f / d : 0.0f;
        if (!std::isfinite(inv_d)) inv_d = 0;
        dst[b].d = f2h(d);
        std::memset(dst[b].qs, 0, 32);
        for (int j = 0; j < 128; ++j) {
            const float r = std::max(0.0f, std::min(3.0f, std::round(x[j] * inv_d) + 1.0f));
            const uint8_t q = (uint8_t)r;
            dst[b].qs[j / 4] |= (uint8_t)(q << ((j % 4) * 2));
        }
    }
}

// ---- per-block dots (Oracle A) ---------------------------------------------
// q8_0.zig:1074-1089.
inline float dot_q8_0_q8_0(const BlockQ8_0* a, const BlockQ8_0* b) {
    const float d = h2f(a->d) * h2f(b->d);
    int32_t dot = 0;
    for (int i = 0; i < 32; ++i) dot += (int32_t)a->qs[i] * (int32_t)b->qs[i];
    return (float)dot * d;
}
// q4_k.zig:895-913 / :2090-2110.
inline float dot_q4_k_q8_k(const BlockQ4_K* w, const BlockQ8_K* a) {
    const float d = h2f(w->dm[0]) * a->d;
    const float dmin = h2f(w->dm[1]) * a->d;
    int32_t iscale = 0, imin = 0;
    for (int s = 0; s < 8; ++s) {
        uint8_t sc, mn;
        get_scale_min_k4(w->scales, s, &sc, &mn);
        int32_t acc = 0;
        for (int i = 0; i < 32; ++i) acc += (int32_t)q4k_value(w, s, i) * (int32_t)a->qs[s * 32 + i];
        const int32_t bsum = (int32_t)a->bsums[s * 2] + (int32_t)a->bsums[s * 2 + 1];
        iscale += (int32_t)sc * acc;
        imin += (int32_t)mn * bsum;
    }
    return d * (float)iscale - dmin * (float)imin;
}
// q5_k.zig:1093-1111.
inline float dot_q5_k_q8_k(const BlockQ5_K* w, const BlockQ8_K* a) {
    int32_t iscale = 0, imin = 0;
    for (int s = 0; s < 8; ++s) {
        uint8_t sc, mn;
        get_scale_min_k4(w->scales, s, &sc, &mn);
        int32_t dot = 0;
        for (int i = 0; i < 32; ++i) dot += (int32_t)q5k_value(w, s, i) * (int32_t)a->qs[s * 32 + i];
        const int32_t bsum = (int32_t)a->bsums[s * 2] + (int32_t)a->bsums[s * 2 + 1];
        iscale += (int32_t)sc * dot;
        imin += (int32_t)mn * bsum;
    }
    const float d = h2f(w->dm[0]) * a->d;
    const float dmin = h2f(w->dm[1]) * a->d;
    return d * (float)iscale - dmin * (float)imin;
}
// q6_k.zig:617-631 `dotQ6_KQ8_KScalar` (the SIMD tiers give the same integer total and the same f32 epilogue).
inline float dot_q6_k_q8_k(const BlockQ6_K* w, const BlockQ8_K* a) {
    int32_t iacc = 0;
    for (int group = 0; group < 16; ++group) {
        int32_t dot = 0;
        for (int i = 0; i < 16; ++i) {
            const int feature = group * 16 + i;
            dot += (int32_t)q6k_value(w, feature) * (int32_t)a->qs[feature];
        }
        iacc += dot * (int32_t)w->scales[q6k_scale_index(group * 16)];
    }
    const float d = h2f(w->d) * a->d;
    return (float)iacc * d;
}
inline int32_t bsum_total(const BlockQ8_K* a) {
    int32_t t = 0;
    for (int g = 0; g < 16; ++g) t += a->bsums[g];
    return t;
}
// ternary.zig:377-386 (hot tile) == cold.zig:1959-1976 (scalar).
inline float dot_tq2_0_q8_k(const BlockTQ2_0* w, const BlockQ8_K* a) {
    int32_t dots = 0;
    for (int e = 0; e < 256; ++e) dots += tq2_code(w, e) * (int32_t)a->qs[e];
    const int32_t isum = dots - bsum_total(a);
    return h2f(w->d) * a->d * (float)isum;
}
// ternary.zig:780-786.
inline float dot_folded_q8_k(const BlockTQ2_0Folded* w, const BlockQ8_K* a) {
    int32_t acc = 0;
    for (int e = 0; e < 256; ++e) acc += folded_cu(w, e) * (int32_t)a->qs[e];
    const int32_t isum = acc - 4 * bsum_total(a);
    return h2f(w->d) * a->d * (float)isum;
}
// cold.zig:1988-2010: four lanes (one per 32-sub-block of the 128-block),
// folded pairwise at the end.
float dot_q2_0_row_q8_0(const BlockQ2_0* w, const BlockQ8_0* arow, size_t nblocks) {
    float lanes[4] = {0, 0, 0, 0};
    for (size_t bi = 0; bi < nblocks; ++bi) {
        const float d0 = h2f(w[bi].d);
        for (int kk = 0; kk < 4; ++kk) {
            const BlockQ8_0* ab = &arow[bi * 4 + kk];
            int32_t isum = 0;
            for (int byte = 0; byte < 8; ++byte)
                for (int slot = 0; slot < 4; ++slot) {
                    const int q = ((w[bi].qs[kk * 8 + byte] >> (2 * slot)) & 3) - 1;
                    isum += q * (int32_t)ab->qs[byte * 4 + slot];
                }
            lanes[kk] += d0 * h2f(ab->d) * (float)isum;
        }
    }
    return (lanes[0] + lanes[1]) + (lanes[2] + lanes[3]);
}

// exec/topk.zig:50-86.
void router_topk_row(const float* logits, size_t experts, size_t k, bool normalize, int64_t* selected,
                     float* weights) {
    float max = logits[0];
    for (size_t s = 0; s < k; ++s) {
        selected[s] = 0;
        weights[s] = -INFINITY;
    }
    for (size_t i = 0; i < experts; ++i) {
        const float v = logits[i];
        if (v > max) max = v;
        if (v <= weights[k - 1]) continue;
        size_t slot = k - 1;
        while (slot > 0 && v > weights[slot - 1]) {
            weights[slot] = weights[slot - 1];
            selected[slot] = selected[slot - 1];
            --slot;
        }
        weights[slot] = v;
        selected[slot] = (int64_t)i;
    }
    float exp_sum = 0;
    for (size_t i = 0; i < experts; ++i) exp_sum += std::exp(logits[i] - max);
    const float inv_sum = 1.0f / exp_sum;
    float total = 0;
    for (size_t s = 0; s < k; ++s) {
        const float e = std::exp(weights[s] - max) * inv_sum;
        weights[s] = e;
        total += e;
    }
    if (normalize && total > 0) {
        const float inv_total = 1.0f / total;
        for (size_t s = 0; s < k; ++s) weights[s] *= inv_total;
    }
}

// backend/ops.zig:150-190: swiglu pair = up * (gate * 1/(1+exp(-gate))).
inline float swiglu_pair(float gate, float up) {
    const float sig = 1 / (1 + std::exp(-gate));
    return up * (gate * sig);
}
// backend/ops.zig:89-107 `GatedOp`, :150-190 `gatedActivationScalar` / `gatedSourceScalar` / `gatedPairScalar`.
// Codes: 0 swiglu, 1 geglu, 2 swiglu_clamp10, 3 glu, 4 situ.
inline float sigmoid_scalar(float v) { return 1 / (1 + std::exp(-v)); }
inline float gated_activation(int op, float v) {
    switch (op) {
        case 1: {  // geluScalar: 0.5 * v * (1 + tanh(sqrt(2/pi) * (v + 0.044715 v^3)))  (ops.zig:200-213)
            const float sqrt_2_over_pi = 0.7978845608028654f;
            const float arg = sqrt_2_over_pi * (v + 0.044715f * v * v * v);
            return 0.5f * v * (1 + std::tanh(arg));
        }
        case 2: {
            const float g = std::min(v, 10.0f);
            return g * sigmoid_scalar(g);
        }
        case 3: return sigmoid_scalar(v);
        case 4: return 4.0f * std::tanh(v * 0.25f) * sigmoid_scalar(v);
        default: return v * sigmoid_scalar(v);
    }
}
inline float gated_source(int op, float up) {
    if (op == 2) return std::min(std::max(up, -10.0f), 10.0f);
    if (op == 4) return 25.0f * std::tanh(up * 0.04f);
    return up;
}
inline float gated_pair(int op, float gate, float up) { return gated_source(op, up) * gated_activation(op, gate); }

enum Fmt { Q8_0 = 0, Q6_K = 1, Q4_K = 2, Q5_K = 3, TQ2_0 = 16, TQ2_0_FOLDED = 17, Q2_0 = 18 };

size_t row_bytes(int fmt, size_t k) {
    switch (fmt) {
        case Q8_0: return k / 32 * 34;
        case Q4_K: return k / 256 * 144;
        case Q5_K: return k / 256 * 176;
        case Q6_K: return k / 256 * 210;
        case TQ2_0: return k / 256 * 66;
        case TQ2_0_FOLDED: return k / 256 * 130;
        case Q2_0: return k / 128 * 34;
    }
    return 0;
}

// One output element of the CPU-kernel replica: blocks ascending, f32 adds in
// that order (q8_0.zig:326-346, q4_k.zig:503-509, ternary.zig:389-399).
float row_dot(int fmt, const uint8_t* wrow, const void* arow, size_t k) {
    float acc = 0;
    switch (fmt) {
        case Q8_0: {
            const BlockQ8_0* w = (const BlockQ8_0*)wrow;
            const BlockQ8_0* a = (const BlockQ8_0*)arow;
            for (size_t b = 0; b < k / 32; ++b) acc += dot_q8_0_q8_0(&a[b], &w[b]);
            return acc;
        }
        case Q4_K: {
            const BlockQ4_K* w = (const BlockQ4_K*)wrow;
            const BlockQ8_K* a = (const BlockQ8_K*)arow;
            for (size_t b = 0; b < k / 256; ++b) acc += dot_q4_k_q8_k(&w[b], &a[b]);
            return acc;
        }
        case Q5_K: {
            const BlockQ5_K* w = (const BlockQ5_K*)wrow;
            const BlockQ8_K* a = (const BlockQ8_K*)arow;
            for (size_t b = 0; b < k / 256; ++b) acc += dot_q5_k_q8_k(&w[b], &a[b]);
            return acc;
        }
        case Q6_K: {  // q6_k.zig:109-148 `matmulQ6_KRhsTile`: blocks ascending
            const BlockQ6_K* w = (const BlockQ6_K*)wrow;
            const BlockQ8_K* a = (const BlockQ8_K*)arow;
            for (size_t b = 0; b < k / 256; ++b) acc += dot_q6_k_q8_k(&w[b], &a[b]);
            return acc;
        }
        case TQ2_0: {
            const BlockTQ2_0* w = (const BlockTQ2_0*)wrow;
            const BlockQ8_K* a = (const BlockQ8_K*)arow;
            for (size_t b = 0; b < k / 256; ++b) acc += dot_tq2_0_q8_k(&w[b], &a[b]);
            return acc;
        }
        case TQ2_0_FOLDED: {
            const BlockTQ2_0Folded* w = (const BlockTQ2_0Folded*)wrow;
            const BlockQ8_K* a = (const BlockQ8_K*)arow;
            for (size_t b = 0; b < k / 256; ++b) acc += dot_folded_q8_k(&w[b], &a[b]);
            return acc;
        }
        case Q2_0:
            return dot_q2_0_row_q8_0((const BlockQ2_0*)wrow, (const BlockQ8_0*)arow, k / 128);
    }
    return 0;
}

bool acts_are_q8_0(int fmt) { return fmt == Q8_0 || fmt == Q2_0; }

// Quantise m activation rows the way backend/native.zig:427-452 (Q8_0 rows)
// and :473-490 (Q8_K rows) do before the integer kernels run.
std::vector<uint8_t> quantize_acts(int fmt, const float* a, size_t m, size_t k, size_t* row_stride) {
    if (acts_are_q8_0(fmt)) {
        *row_stride = k / 32 * sizeof(BlockQ8_0);
        std::vector<uint8_t> out(m * *row_stride);
        for (size_t i = 0; i < m; ++i) quantize_row_q8_0((BlockQ8_0*)(out.data() + i * *row_stride), a + i * k, k);
        return out;
    }
    *row_stride = k / 256 * sizeof(BlockQ8_K);
    std::vector<uint8_t> out(m * *row_stride);
    for (size_t i = 0; i < m; ++i) quantize_row_q8_k((BlockQ8_K*)(out.data() + i * *row_stride), a + i * k, k);
    return out;
}

void dequantize_row(int fmt, float* dst, const uint8_t* wrow, size_t k) {
    switch (fmt) {
        case Q8_0: dequantize_row_q8_0(dst, (const BlockQ8_0*)wrow, k); break;
        case Q4_K:
            for (size_t b = 0; b < k / 256; ++b) dequantize_block_q4_k(dst + b * 256, (const BlockQ4_K*)wrow + b);
            break;
        case Q5_K:
            for (size_t b = 0; b < k / 256; ++b) dequantize_block_q5_k(dst + b * 256, (const BlockQ5_K*)wrow + b);
            break;
        case Q6_K:
            for (size_t b = 0; b < k / 256; ++b) dequantize_block_q6_k(dst + b * 256, (const BlockQ6_K*)wrow + b);
            break;
        case TQ2_0: dequantize_row_tq2_0(dst, (const BlockTQ2_0*)wrow, k); break;
        case TQ2_0_FOLDED:
            for (size_t b = 0; b < k / 256; ++b) {
                const BlockTQ2_0Folded* blk = (const BlockTQ2_0Folded*)wrow + b;
                const float scale = h2f(blk->d);
                for (int e = 0; e < 256; ++e) dst[b * 256 + e] = scale * ((float)folded_cu(blk, e) - 4.0f);
            }
            break;
        case Q2_0:
            for (size_t b = 0; b < k / 128; ++b) {
                const BlockQ2_0* blk = (const BlockQ2_0*)wrow + b;
                const float d = h2f(blk->d);
                for (int j = 0; j < 128; ++j) {
                    const int q = (blk->qs[j / 4] >> ((j % 4) * 2)) & 3;
                    dst[b * 128 + j] = (float)(q - 1) * d;
                }
            }
            break;
    }
}

inline float round_bf16(float x) {
    uint32_t u;
    std::memcpy(&u, &x, 4);
    if ((u & 0x7f800000u) == 0x7f800000u) return x;
    u += 0x7fffu + ((u >> 16) & 1);
    u &= 0xffff0000u;
    float r;
    std::memcpy(&r, &u, 4);
    return r;
}

}  // namespace

extern "C" {

size_t orc_row_bytes(int fmt, size_t k) { return row_bytes(fmt, k); }

// Weight encoders: n rows of k floats -> n rows of blocks (row-parallel; each
// row is independent so threading does not change a byte).
int orc_quantize_rows(int fmt, const float* src, size_t n, size_t k, void* dst) {
    const size_t rb = row_bytes(fmt, k);
    if (rb == 0) return 1;
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < (long long)n; ++r) {
        uint8_t* out = (uint8_t*)dst + (size_t)r * rb;
        const float* in = src + (size_t)r * k;
        switch (fmt) {
            case Q8_0: quantize_row_q8_0((BlockQ8_0*)out, in, k); break;
            case Q4_K:
                for (size_t b = 0; b < k / 256; ++b) quantize_block_q4_k((BlockQ4_K*)out + b, in + b * 256);
                break;
            case Q5_K:
                for (size_t b = 0; b < k / 256; ++b) quantize_block_q5_k((BlockQ5_K*)out + b, in + b * 256);
                break;
            case Q6_K:
                for (size_t b = 0; b < k / 256; ++b) quantize_block_q6_k((BlockQ6_K*)out + b, in + b * 256);
                break;
            case TQ2_0: quantize_row_tq2_0((BlockTQ2_0*)out, in, k); break;
            case Q2_0: quantize_row_q2_0((BlockQ2_0*)out, in, k); break;
            default: break;
        }
    }
    return 0;
}

// ptqtp.zig:684-697: one TQ2_0 plane from seeded trits and per-block scales.
int orc_pack_ptqtp_plane(const int8_t* trits, const float* scales, size_t n, size_t k, void* dst) {
    const size_t bpr = k / 256;
    for (size_t r = 0; r < n; ++r)
        for (size_t b = 0; b < bpr; ++b) {
            BlockTQ2_0* blk = (BlockTQ2_0*)dst + r * bpr + b;
            const int8_t* t = trits + r * k + b * 256;
            blk->d = f2h(scales[r * bpr + b]);
            for (int hg = 0; hg < 2; ++hg)
                for (int m = 0; m < 32; ++m) {
                    uint8_t q = 0;
                    for (int nn = 0; nn < 4; ++nn) q |= (uint8_t)((t[hg * 128 + nn * 32 + m] + 1) << (2 * nn));
                    blk->qs[hg * 32 + m] = q;
                }
        }
    return 0;
}

// Q2_0 g128 blocks straight from trits + per-128 scales (layout cold.zig:285-301).
int orc_pack_q2_0(const int8_t* trits, const float* scales, size_t n, size_t k, void* dst) {
    const size_t bpr = k / 128;
    for (size_t r = 0; r < n; ++r)
        for (size_t b = 0; b < bpr; ++b) {
            BlockQ2_0* blk = (BlockQ2_0*)dst + r * bpr + b;
            const int8_t* t = trits + r * k + b * 128;
            blk->d = f2h(scales[r * bpr + b]);
            std::memset(blk->qs, 0, 32);
            for (int j = 0; j < 128; ++j) blk->qs[j / 4] |= (uint8_t)((t[j] + 1) << ((j % 4) * 2));
        }
    return 0;
}

// ternary.zig:707-735: row-major fold of a coarse and a fine plane.
int orc_fold_planes(const void* plane1, const void* plane2, size_t n, size_t k, void* dst) {
    const size_t bpr = k / 256;
    for (size_t i = 0; i < n * bpr; ++i) {
        const BlockTQ2_0* b1 = (const BlockTQ2_0*)plane1 + i;
        const BlockTQ2_0* b2 = (const BlockTQ2_0*)plane2 + i;
        BlockTQ2_0Folded* out = (BlockTQ2_0Folded*)dst + i;
        out->d = b2->d;
        for (int sub = 0; sub < 8; ++sub)
            for (int j = 0; j < 16; ++j) {
                const uint8_t lo = folded_code(b1, b2, sub * 32 + j);
                const uint8_t hi = folded_code(b1, b2, sub * 32 + 16 + j);
                out->qs[sub * 16 + j] = (uint8_t)(lo | (hi << 4));
            }
    }
    return 0;
}

int orc_dequantize_rows(int fmt, const void* src, size_t n, size_t k, float* dst) {
    const size_t rb = row_bytes(fmt, k);
    if (rb == 0) return 1;
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < (long long)n; ++r)
        dequantize_row(fmt, dst + (size_t)r * k, (const uint8_t*)src + (size_t)r * rb, k);
    return 0;
}

// Activation quantisers exposed for tests of the device-side twins.
int orc_quantize_acts_q8_k(const float* a, size_t m, size_t k, void* dst) {
    for (size_t i = 0; i < m; ++i) quantize_row_q8_k((BlockQ8_K*)dst + i * (k / 256), a + i * k, k);
    return 0;
}
int orc_quantize_acts_q8_0(const float* a, size_t m, size_t k, void* dst) {
    for (size_t i = 0; i < m; ++i) quantize_row_q8_0((BlockQ8_0*)dst + i * (k / 32), a + i * k, k);
    return 0;
}

// The row operations the CPU path fuses in front of its activation quantiser (exec/quant_matmul.zig:480-757).
// rms_norm_mul, the scalar loop of exec/row_ops.zig:96-106: sumsq over the row element by element in f32,
// scale = 1 / sqrt(sumsq * (1/k) + eps), out = value * scale * weight (left to right).
int orc_rms_norm_mul(const float* x, const float* w, float eps, float* out, size_t m, size_t k) {
    const float inv_cols = 1.0f / (float)k;
    for (size_t r = 0; r < m; ++r) {
        const float* row = x + r * k;
        float sumsq = 0.0f;
        for (size_t i = 0; i < k; ++i) sumsq += row[i] * row[i];
        const float scale = 1.0f / std::sqrt(sumsq * inv_cols + eps);
        for (size_t i = 0; i < k; ++i) out[r * k + i] = row[i] * scale * w[i];
    }
    return 0;
}
// split_swiglu, the vector body of exec/row_ops.zig:711-722 (k is a multiple of 4 here): a row holds the gate half
// then the up half; out = up * gate * (1 / (1 + exp(-gate))), left to right.
int orc_split_swiglu(const float* gate_up, float* out, size_t m, size_t k) {
    for (size_t r = 0; r < m; ++r)
        for (size_t i = 0; i < k; ++i) {
            const float gate = gate_up[r * 2 * k + i], up = gate_up[r * 2 * k + k + i];
            out[r * k + i] = up * gate * (1.0f / (1.0f + std::exp(-gate)));
        }
    return 0;
}

// Oracle A: c[m,n] = a[m,k] . dequant(W[n,k])^T the way the CPU kernels do it
// (activations to int8 first, integer block dots, f32 epilogue, blocks
// ascending). nb01 = bytes per weight row. Threads split output columns
// (backend/vector/matmul_quant.zig:578-596); per-element results do not
// depend on the split.
int orc_matmul(int fmt, const void* w, size_t nb01, const float* a, float* c, size_t m, size_t n, size_t k) {
    if (row_bytes(fmt, k) == 0) return 1;
    size_t astride = 0;
    std::vector<uint8_t> qa = quantize_acts(fmt, a, m, k, &astride);
#pragma omp parallel for schedule(static)
    for (long long j = 0; j < (long long)n; ++j) {
        const uint8_t* wrow = (const uint8_t*)w + (size_t)j * nb01;
        for (size_t i = 0; i < m; ++i) c[i * n + (size_t)j] = row_dot(fmt, wrow, qa.data() + i * astride, k);
    }
    return 0;
}

// PTQTP with `planes` TQ2_0 planes: per element dot_plane0 + dot_plane1 (+ ...)
// left to right (exec/moe.zig:573-631, weights.zig:286-300).
int orc_matmul_ptqtp(const void* const* planes, int n_planes, size_t nb01, const float* a, float* c, size_t m,
                     size_t n, size_t k) {
    size_t astride = 0;
    std::vector<uint8_t> qa = quantize_acts(TQ2_0, a, m, k, &astride);
#pragma omp parallel for schedule(static)
    for (long long j = 0; j < (long long)n; ++j)
        for (size_t i = 0; i < m; ++i) {
            float out = row_dot(TQ2_0, (const uint8_t*)planes[0] + (size_t)j * nb01, qa.data() + i * astride, k);
            for (int p = 1; p < n_planes; ++p)
                out += row_dot(TQ2_0, (const uint8_t*)planes[p] + (size_t)j * nb01, qa.data() + i * astride, k);
            c[i * n + (size_t)j] = out;
        }
    return 0;
}

// Oracle B: f64 dot over the dequantised weights, operands optionally rounded
// to bf16 first (the reference's GPU-test oracle, backend/cuda.zig:3016-3044,
// with the tensor-core operand precision of this build). round_mode: 0 none,
// 1 bf16 on both operands.
int orc_matmul_dequant_f64(int fmt, const void* w, size_t nb01, const float* a, double* c, size_t m, size_t n,
                           size_t k, int round_mode) {
    if (row_bytes(fmt, k) == 0) return 1;
    std::vector<float> ar(a, a + m * k);
    if (round_mode == 1)
        for (auto& v : ar) v = round_bf16(v);
#pragma omp parallel
    {
        std::vector<float> wr(k);
#pragma omp for schedule(static)
        for (long long j = 0; j < (long long)n; ++j) {
            dequantize_row(fmt, wr.data(), (const uint8_t*)w + (size_t)j * nb01, k);
            if (round_mode == 1)
                for (auto& v : wr) v = round_bf16(v);
            for (size_t i = 0; i < m; ++i) {
                double acc = 0;
                const float* arow = ar.data() + i * k;
                for (size_t e = 0; e < k; ++e) acc += (double)arow[e] * (double)wr[e];
                c[i * n + (size_t)j] = acc;
            }
        }
    }
    return 0;
}

// One weight block against one explicit activation block (Q8_K, or Q8_0 for
// Q8_0 weights): the per-block kernels the reference's pattern-block tests
// exercise (q4_k.zig:2060-2082, q5_k.zig:1293-1315).
float orc_block_dot(int fmt, const void* wblock, const void* ablock) {
    switch (fmt) {
        case Q8_0: return dot_q8_0_q8_0((const BlockQ8_0*)ablock, (const BlockQ8_0*)wblock);
        case Q4_K: return dot_q4_k_q8_k((const BlockQ4_K*)wblock, (const BlockQ8_K*)ablock);
        case Q5_K: return dot_q5_k_q8_k((const BlockQ5_K*)wblock, (const BlockQ8_K*)ablock);
        case Q6_K: return dot_q6_k_q8_k((const BlockQ6_K*)wblock, (const BlockQ8_K*)ablock);
        case TQ2_0: return dot_tq2_0_q8_k((const BlockTQ2_0*)wblock, (const BlockQ8_K*)ablock);
        case TQ2_0_FOLDED: return dot_folded_q8_k((const BlockTQ2_0Folded*)wblock, (const BlockQ8_K*)ablock);
    }
    return NAN;
}

int orc_router_topk(const float* logits, size_t rows, size_t experts, size_t k, int normalize, int64_t* selected,
                    float* weights) {
    if (k == 0 || k > experts) return 1;
    for (size_t r = 0; r < rows; ++r)
        router_topk_row(logits + r * experts, experts, k, normalize != 0, selected + r * k, weights + r * k);
    return 0;
}

// exec/moe_chain.zig:236-299: counting sort of (token, slot) pairs by expert.
int orc_route_plan(const int64_t* selected, size_t pairs, size_t n_expert, int64_t* count, int64_t* offset,
                   int64_t* order, int64_t* inv) {
    for (size_t p = 0; p < pairs; ++p)
        if (selected[p] < 0 || (size_t)selected[p] >= n_expert) return 1;
    std::fill(count, count + n_expert, 0);
    for (size_t p = 0; p < pairs; ++p) count[selected[p]] += 1;
    offset[0] = 0;
    for (size_t e = 0; e < n_expert; ++e) offset[e + 1] = offset[e] + count[e];
    std::vector<int64_t> place(offset, offset + n_expert);
    for (size_t p = 0; p < pairs; ++p) {
        const int64_t pos = place[selected[p]]++;
        order[pos] = (int64_t)p;
        inv[p] = pos;
    }
    return 0;
}

// The expert FFN layer (exec/moe.zig:890-920 per pair, :1334-1401 batched,
// exec/moe_chain.zig:307-330 combine). gate/up are [E][out_pe][hidden] block
// rows, down is [E][hidden][out_pe]; selected/weights are [seq*top_k].
// Decode and batched forms produce the same numbers per element: quantise the
// token row, gate/up dots, swiglu, requantise, down dot, w*row, add in slot
// order with the first slot assigned.
int orc_moe_ffn_gated(int fmt, int fmt_down, int gated_op, const void* gate, const void* up, const void* down, const float* x, size_t seq,
                      size_t hidden, size_t out_pe, size_t n_expert, size_t top_k, const int64_t* selected,
                      const float* weights, float* out);
int orc_moe_ffn(int fmt, const void* gate, const void* up, const void* down, const float* x, size_t seq,
                size_t hidden, size_t out_pe, size_t n_expert, size_t top_k, const int64_t* selected,
                const float* weights, float* out) {
    return orc_moe_ffn_gated(fmt, fmt, 0, gate, up, down, x, seq, hidden, out_pe, n_expert, top_k, selected, weights, out);
}
// The same layer with any gated op (0 swiglu, 1 geglu, 2 swiglu_clamp10, 3 glu, 4 situ) and a down tensor that may
// come in another format than gate/up (g is then requantised the way that format's kernels want it,
// exec/moe.zig:904-907).
int orc_moe_ffn_gated(int fmt, int fmt_down, int gated_op, const void* gate, const void* up, const void* down, const float* x, size_t seq,
                      size_t hidden, size_t out_pe, size_t n_expert, size_t top_k, const int64_t* selected,
                      const float* weights, float* out) {
    const size_t rb_in = row_bytes(fmt, hidden), rb_g = row_bytes(fmt_down, out_pe);
    if (rb_in == 0 || rb_g == 0) return 1;
    for (size_t p = 0; p < seq * top_k; ++p)
        if (selected[p] < 0 || (size_t)selected[p] >= n_expert) return 1;
    std::vector<float> pair_out(seq * top_k * hidden);
#pragma omp parallel
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
                gate_v[j] = row_dot(fmt, wg + j * rb_in, qx.data(), hidden);
                up_v[j] = row_dot(fmt, wu + j * rb_in, qx.data(), hidden);
            }
            for (size_t j = 0; j < out_pe; ++j) g[j] = gated_pair(gated_op, gate_v[j], up_v[j]);
            std::vector<uint8_t> qg = quantize_acts(fmt_down, g.data(), 1, out_pe, &s_g);
            float* po = pair_out.data() + (size_t)p * hidden;
            for (size_t j = 0; j < hidden; ++j) po[j] = row_dot(fmt_down, wd + j * rb_g, qg.data(), out_pe);
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

// Oracle B for the expert layer: the reference's GPU arm multiplies operands rounded to the
// tensor-core precision with wide accumulation and applies the activation in f32 between the two
// products (src/llm/gemma/moe.zig:696-901, src/backend/cuda.zig:3016-3044). Here: bf16 operands,
// f64 dots rounded to f32, swiglu in f32, g rounded to bf16, weighted combine in slot order.
int orc_moe_ffn_bf16_gated(int fmt, int fmt_down, int gated_op, const void* gate, const void* up, const void* down, const float* x, size_t seq,
                           size_t hidden, size_t out_pe, size_t n_expert, size_t top_k, const int64_t* selected,
                           const float* weights, float* out);
int orc_moe_ffn_bf16(int fmt, const void* gate, const void* up, const void* down, const float* x, size_t seq,
                     size_t hidden, size_t out_pe, size_t n_expert, size_t top_k, const int64_t* selected,
                     const float* weights, float* out) {
    return orc_moe_ffn_bf16_gated(fmt, fmt, 0, gate, up, down, x, seq, hidden, out_pe, n_expert, top_k, selected, weights, out);
}
int orc_moe_ffn_bf16_gated(int fmt, int fmt_down, int gated_op, const void* gate, const void* up, const void* down, const float* x, size_t seq,
                           size_t hidden, size_t out_pe, size_t n_expert, size_t top_k, const int64_t* selected,
                           const float* weights, float* out) {
    const size_t rb_in = row_bytes(fmt, hidden), rb_g = row_bytes(fmt_down, out_pe);
    if (rb_in == 0 || rb_g == 0) return 1;
    for (size_t p = 0; p < seq * top_k; ++p)
        if (selected[p] < 0 || (size_t)selected[p] >= n_expert) return 1;
    std::vector<float> pair_out(seq * top_k * hidden);
#pragma omp parallel
    {
        std::vector<float> wrow(std::max(hidden, out_pe)), xb(hidden), g(out_pe), gate_v(out_pe), up_v(out_pe);
#pragma omp for schedule(dynamic, 1)
        for (long long p = 0; p < (long long)(seq * top_k); ++p) {
            const size_t t = (size_t)p / top_k, e = (size_t)selected[p];
            for (size_t i = 0; i < hidden; ++i) xb[i] = round_bf16(x[t * hidden + i]);
            const uint8_t* wg = (const uint8_t*)gate + e * out_pe * rb_in;
            const uint8_t* wu = (const uint8_t*)up + e * out_pe * rb_in;
            const uint8_t* wd = (const uint8_t*)down + e * hidden * rb_g;
            for (size_t j = 0; j < out_pe; ++j) {
                dequantize_row(fmt, wrow.data(), wg + j * rb_in, hidden);
                double acc = 0;
                for (size_t i = 0; i < hidden; ++i) acc += (double)round_bf16(wrow[i]) * (double)xb[i];
                gate_v[j] = (float)acc;
                dequantize_row(fmt, wrow.data(), wu + j * rb_in, hidden);
                acc = 0;
                for (size_t i = 0; i < hidden; ++i) acc += (double)round_bf16(wrow[i]) * (double)xb[i];
                up_v[j] = (float)acc;
            }
            for (size_t j = 0; j < out_pe; ++j) g[j] = round_bf16(gated_pair(gated_op, gate_v[j], up_v[j]));
            float* po = pair_out.data() + (size_t)p * hidden;
            for (size_t j = 0; j < hidden; ++j) {
                dequantize_row(fmt_down, wrow.data(), wd + j * rb_g, out_pe);
                double acc = 0;
                for (size_t i = 0; i < out_pe; ++i) acc += (double)round_bf16(wrow[i]) * (double)g[i];
                po[j] = (float)acc;
            }
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

// Expert layer over multi-plane ternary (PTQTP) experts: every projection is K TQ2_0 plane stacks with the
// geometry of a TQ2_0 expert stack; a tile dot runs once per plane and the results add per element in plane
// order (exec/moe.zig:51-78 `MoePtqtpRhs`, :591-631 `moePtqtpTileDotRange`), then the layer proceeds as
// orc_moe_ffn_gated does.
int orc_moe_ffn_ptqtp(int n_planes, int gated_op, const void* const* gate, const void* const* up, const void* const* down, const float* x,
                      size_t seq, size_t hidden, size_t out_pe, size_t n_expert, size_t top_k, const int64_t* selected,
                      const float* weights, float* out) {
    const int fmt = TQ2_0;
    const size_t rb_in = row_bytes(fmt, hidden), rb_g = row_bytes(fmt, out_pe);
    if (rb_in == 0 || rb_g == 0 || n_planes < 1 || n_planes > 3) return 1;
    for (size_t p = 0; p < seq * top_k; ++p)
        if (selected[p] < 0 || (size_t)selected[p] >= n_expert) return 1;
    std::vector<float> pair_out(seq * top_k * hidden);
#pragma omp parallel
    {
        std::vector<float> gate_v(out_pe), up_v(out_pe), g(out_pe);
#pragma omp for schedule(dynamic, 1)
        for (long long p = 0; p < (long long)(seq * top_k); ++p) {
            const size_t t = (size_t)p / top_k, e = (size_t)selected[p];
            size_t s_in = 0, s_g = 0;
            std::vector<uint8_t> qx = quantize_acts(fmt, x + t * hidden, 1, hidden, &s_in);
            for (size_t j = 0; j < out_pe; ++j) {
                float gsum = 0, usum = 0;
                for (int pl = 0; pl < n_planes; ++pl) {
                    const float gd = row_dot(fmt, (const uint8_t*)gate[pl] + (e * out_pe + j) * rb_in, qx.data(), hidden);
                    const float ud = row_dot(fmt, (const uint8_t*)up[pl] + (e * out_pe + j) * rb_in, qx.data(), hidden);
                    gsum = pl ? gsum + gd : gd;
                    usum = pl ? usum + ud : ud;
                }
                gate_v[j] = gsum, up_v[j] = usum;
            }
            for (size_t j = 0; j < out_pe; ++j) g[j] = gated_pair(gated_op, gate_v[j], up_v[j]);
            std::vector<uint8_t> qg = quantize_acts(fmt, g.data(), 1, out_pe, &s_g);
            float* po = pair_out.data() + (size_t)p * hidden;
            for (size_t j = 0; j < hidden; ++j) {
                float dsum = 0;
                for (int pl = 0; pl < n_planes; ++pl) {
                    const float dd = row_dot(fmt, (const uint8_t*)down[pl] + (e * hidden + j) * rb_g, qg.data(), out_pe);
                    dsum = pl ? dsum + dd : dd;
                }
                po[j] = dsum;
            }
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
