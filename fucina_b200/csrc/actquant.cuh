// Warp-level activation quantisers shared by the stand-alone quantise kernels
// and by the decode kernel's fused prologue. One warp handles 256 consecutive
// activations; lane l owns elements 8l..8l+7. Every float operation uses an
// explicitly rounded intrinsic, so the values do not depend on the
// translation unit's contraction setting and equal the reference CPU code
// bit for bit.
#pragma once
#include "common.cuh"

namespace fq {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ int warp_min_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Q8_K values of one 256-element block (reference
// src/backend/quant/q8k.zig:268-313): the scale comes from the FIRST element
// whose magnitude equals the block maximum, inv = -127/max_value,
// q = min(127, round_even(inv * v)), d = 1/inv. Returns d; q[] per lane.
__device__ __forceinline__ float q8k_block(const float v[8], int lane, int q[8]) {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    amax = warp_max(amax);
    int first = 1 << 20;
    float cand = 0.0f;
#pragma unroll
    for (int j = 7; j >= 0; --j)
        if (fabsf(v[j]) == amax) {
            first = lane * 8 + j;
            cand = v[j];
        }
    const int idx = warp_min_i(first);
    const float max_value = __shfl_sync(0xffffffffu, cand, (idx >> 3) & 31);
    if (amax == 0.0f) {
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = 0;
        return 0.0f;
    }
    const float inv = __fdiv_rn(-127.0f, max_value);
#pragma unroll
    for (int j = 0; j < 8; ++j) q[j] = (int)fminf(127.0f, rintf(__fmul_rn(inv, v[j])));
    return __fdiv_rn(1.0f, inv);
}

// Q8_0 values (q8k.zig:49-69): d = amax/127 over 32 elements (4 lanes),
// q = clamp(round_half_away(v * (1/d)), +-127); the stored scale is f16.
__device__ __forceinline__ uint16_t q8_0_quarter(const float v[8], int q[8]) {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float d = __fdiv_rn(amax, 127.0f);
    const float inv_d = (d == 0.0f) ? 0.0f : __fdiv_rn(1.0f, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) q[j] = (int)fmaxf(-127.0f, fminf(127.0f, roundf(__fmul_rn(v[j], inv_d))));
    return __half_as_ushort(__float2half_rn(d));
}

__device__ __forceinline__ uint32_t pack4(const int* q) {
    return (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) |
           ((uint32_t)(q[3] & 0xff) << 24);
}

// "Natural" activation record used by the row-per-lane decode kernel: values
// in element order plus what the block epilogues need.
//   Q8_K formats: [aq: K int8][bs32: K/32 int32, sum of each 32-element
//                 sub-block (= bsums[2s] + bsums[2s+1])][ad: K/256 f32]
//   Q8_0 formats: [aq: K int8][ad: K/32 f32 (the f16-rounded scale)]
struct NatSizes {
    size_t aq, sums, ad, row;
};
__host__ __device__ inline NatSizes nat_sizes(bool q8k, size_t k) {
    NatSizes s;
    s.aq = k;
    s.sums = q8k ? k / 8 : 0;
    s.ad = q8k ? ((k / 64 + 15) & ~(size_t)15) : k / 8;
    s.row = s.aq + s.sums + s.ad;
    return s;
}

// ---- activation prologues fused in front of the quantiser ------------------------------------------------------
// The reference CPU path fuses two row operations into its activation quantiser so the [m, k] intermediate is never
// written (src/exec/quant_matmul.zig:480-757, src/exec/row_ops.zig:39-137):
//   rms_norm_mul   out = (x * scale) * weight, scale = 1 / sqrt(sum(x^2) / k + eps)      (row_ops.zig:96-106)
//   split_swiglu   row = [gate: k][up: k], out = (up * gate) * (1 / (1 + exp(-gate)))     (row_ops.zig:711-728)
// Sum of squares, fixed order: lane partial over its 8 elements in element order, xor tree over the warp, then the
// 256-element block sums added in block order. Every caller uses these helpers, so the fused and the stand-alone
// forms agree bit for bit.
__device__ __forceinline__ void load8(const float* src, float v[8]) {
    const float4 v0 = *reinterpret_cast<const float4*>(src);
    const float4 v1 = *reinterpret_cast<const float4*>(src + 4);
    v[0] = v0.x, v[1] = v0.y, v[2] = v0.z, v[3] = v0.w, v[4] = v1.x, v[5] = v1.y, v[6] = v1.z, v[7] = v1.w;
}
__device__ __forceinline__ float block_sumsq(const float v[8]) {
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) s = __fadd_rn(s, __fmul_rn(v[j], v[j]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, o));
    return s;
}
__device__ __forceinline__ float rms_scale(const float* block_sums, int nblk, float eps) {
    float total = 0.0f;
    for (int i = 0; i < nblk; ++i) total = __fadd_rn(total, block_sums[i]);
    const float inv_cols = __fdiv_rn(1.0f, (float)(nblk * 256));
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(total, inv_cols), eps)));
}
// The 8 prologue outputs of lane `lane` in block `blk` of one row. `row` is the row's first input element (2k
// inputs per row for split_swiglu), `scale` the row's rms scale.
__device__ __forceinline__ void load_block_pre(const PreArgs& P, const float* row, size_t k, int blk, int lane, float scale, float v[8]) {
    const size_t e0 = (size_t)blk * 256 + lane * 8;
    load8(row + e0, v);
    if (P.op == FQ_PRE_RMS_NORM_MUL) {
        float w[8];
        load8(P.w + e0, w);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(__fmul_rn(v[j], scale), w[j]);
    } else if (P.op == FQ_PRE_SPLIT_SWIGLU) {
        float up[8];
        load8(row + k + e0, up);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(__fmul_rn(up[j], v[j]), __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-v[j]))));
    }
}

// Quantise 256 activations (block `blk` of a row), given as the 8 values of each lane, into a natural record.
// Call with a full warp. `k` must be a multiple of 256.
// `q8k`: 0 = Q8_0 records; 1 = Q8_K records with eight int32 sums of 32 elements per block (the K-quants' sub-blocks);
// 2 = Q8_K records with the sixteen int16 sums of 16 elements per block in the same 32 bytes (Q8_K's own bsums,
// dtype.zig:148-152: Q6_K has a scale per 16 elements).
__device__ __forceinline__ void quantize_values_natural(const float v[8], int blk, int q8k, size_t k, uint8_t* rec, int lane) {
    const NatSizes S = nat_sizes(q8k != 0, k);
    int q[8];
    uint2 packed;
    if (q8k) {
        const float d = q8k_block(v, lane, q);
        if (lane == 0) reinterpret_cast<float*>(rec + S.aq + S.sums)[blk] = d;
        int sum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += q[j];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        if (q8k == 2) {
            if ((lane & 1) == 0) reinterpret_cast<int16_t*>(rec + S.aq)[blk * 16 + (lane >> 1)] = (int16_t)sum;
        } else {
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if ((lane & 3) == 0) reinterpret_cast<int32_t*>(rec + S.aq)[blk * 8 + (lane >> 2)] = sum;
        }
    } else {
        const uint16_t dh = q8_0_quarter(v, q);
        if ((lane & 3) == 0) reinterpret_cast<float*>(rec + S.aq)[blk * 8 + (lane >> 2)] = h2f(dh);
    }
    packed.x = pack4(q);
    packed.y = pack4(q + 4);
    *reinterpret_cast<uint2*>(rec + (size_t)blk * 256 + lane * 8) = packed;
}
__device__ __forceinline__ void quantize_block_natural(const float* __restrict__ src_row, int blk, int q8k, size_t k,
                                                       uint8_t* rec, int lane) {
    float v[8];
    load8(src_row + (size_t)blk * 256 + lane * 8, v);
    quantize_values_natural(v, blk, q8k, k, rec, lane);
}

}  // namespace fq
