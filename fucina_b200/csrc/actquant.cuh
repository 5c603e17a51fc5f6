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

// Quantise 256 activations (block `blk` of a row) into a natural record.
// Call with a full warp. `k` must be a multiple of 256.
__device__ __forceinline__ void quantize_block_natural(const float* __restrict__ src_row, int blk, bool q8k, size_t k,
                                                       uint8_t* rec, int lane) {
    const NatSizes S = nat_sizes(q8k, k);
    const float* src = src_row + (size_t)blk * 256 + lane * 8;
    const float4 v0 = *reinterpret_cast<const float4*>(src);
    const float4 v1 = *reinterpret_cast<const float4*>(src + 4);
    const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    int q[8];
    uint2 packed;
    if (q8k) {
        const float d = q8k_block(v, lane, q);
        if (lane == 0) reinterpret_cast<float*>(rec + S.aq + S.sums)[blk] = d;
        int sum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += q[j];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((lane & 3) == 0) reinterpret_cast<int32_t*>(rec + S.aq)[blk * 8 + (lane >> 2)] = sum;
    } else {
        const uint16_t dh = q8_0_quarter(v, q);
        if ((lane & 3) == 0) reinterpret_cast<float*>(rec + S.aq)[blk * 8 + (lane >> 2)] = h2f(dh);
    }
    packed.x = pack4(q);
    packed.y = pack4(q + 4);
    *reinterpret_cast<uint2*>(rec + (size_t)blk * 256 + lane * 8) = packed;
}

}  // namespace fq
