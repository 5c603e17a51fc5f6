// Shared device/host helpers for the sm_100a quantized-matmul kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fucina_b200.h"

namespace fq {

// ---- GGUF block geometry (reference src/dtype.zig:78-86, :128-152, :215-218;
//      src/backend/quant/types.zig:177-180) ---------------------------------
struct FormatInfo {
    int block_elems;  // weights per block
    int block_bytes;  // GGUF bytes per block
    int qs_bytes;     // payload bytes per block in the device layout
    int sc_bytes;     // scale bytes per block in the device layout (0 = block kept whole)
};

__host__ __device__ inline FormatInfo format_info(int fmt) {
    switch (fmt) {
        case FQ_Q8_0: return {32, 34, 32, 2};
        case FQ_Q4_K: return {256, 144, 144, 0};
        case FQ_Q5_K: return {256, 176, 176, 0};
        case FQ_Q6_K: return {256, 210, 208, 2};  // ql[128] qh[64] scales[16] | d: the 208 payload bytes are 13 aligned chunks
        case FQ_TQ2_0: return {256, 66, 64, 2};
        case FQ_TQ2_0_FOLDED: return {256, 130, 128, 2};
        case FQ_Q2_0: return {128, 34, 32, 2};
        default: return {0, 0, 0, 0};
    }
}

// Device weight layout ("gpu_formats"). K-quant rows are the GGUF rows
// unchanged (their 144/176-byte blocks are already 16-byte multiples). The
// 34/66/130-byte formats and Q6_K (210) are split per row into a payload plane followed by
// an f16 scale plane so every payload chunk is 16-byte aligned:
//   row = [ qs of block 0 | qs of block 1 | ... ][ d0 d1 ... ] padded to 16 B.
//
// Dense K-quant matrices that the streaming decode kernel serves (one matrix,
// K >= 2048) are additionally stored TILE-MAJOR (tile_rows = 32): rows are
// grouped 32 at a time and, inside a group, the 256-weight unit u of all 32
// rows is contiguous:
//   tile t = [ unit 0 of rows 32t..32t+31 | unit 1 of rows 32t.. | ... ]
// so the 32 rows x one unit a warp consumes per step is ONE contiguous run of
// 32*unit_bytes in HBM -- a single bulk copy that lands in shared memory as
// 32 slots of unit_bytes (an odd number of 16-byte chunks: no bank conflicts).
// Bytes only move; the byte count is unchanged apart from padding n to 32.
struct DevWeights {
    const uint8_t* base;
    size_t row_stride;  // bytes between rows (row-major) / bytes of one row's units (tile-major)
    size_t mat_stride;  // bytes between stacked matrices
    int fmt;
    int n;       // rows per matrix
    int k;       // elements per row
    int n_mats;
    int tile_rows;  // 0 = row-major, 32 = tile-major (K-quants only)
};

// Unit 0 of `row` and the byte distance between consecutive units of that row.
__host__ __device__ inline const uint8_t* row_unit0(const DevWeights& w, const uint8_t* mat_base, int row, int unit_bytes) {
    if (!w.tile_rows) return mat_base + (size_t)row * w.row_stride;
    return mat_base + (size_t)(row >> 5) * ((size_t)32 * w.row_stride) + (size_t)(row & 31) * unit_bytes;
}
__host__ __device__ inline size_t unit_stride(const DevWeights& w, int unit_bytes) {
    return w.tile_rows ? (size_t)32 * unit_bytes : (size_t)unit_bytes;
}

__host__ __device__ inline size_t dev_row_stride(int fmt, size_t k) {
    const FormatInfo f = format_info(fmt);
    if (f.block_elems == 0) return 0;
    const size_t blocks = k / f.block_elems;
    const size_t raw = blocks * (size_t)(f.qs_bytes + f.sc_bytes);
    return (raw + 15) & ~(size_t)15;
}

// Activation prologue of a product (see actquant.cuh): op is one of FQ_PRE_*, `w` the [k] norm weights of
// rms_norm_mul, `eps` its epsilon. With split_swiglu an input row holds 2k values.
struct PreArgs {
    int op;
    const float* w;
    float eps;
};

// Programmatic dependent launch for chains of short kernels: the kernel waits for its predecessor to complete (and its
// writes to be visible) before it touches global memory, then lets its own successor begin launching. A kernel
// launched without the attribute (or after a kernel that never signals) sees both as no-ops.
__device__ __forceinline__ void pdl_wait_then_release() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---- small device helpers ---------------------------------------------------
__device__ __forceinline__ float h2f(uint16_t bits) { return __half2float(__ushort_as_half(bits)); }

// Gated pair of an FFN (reference backend/ops.zig:150-190): g = source(up) * activation(gate), every product
// rounded on its own as the scalar code does. `op` is one of FQ_GATED_*.
__device__ __forceinline__ float fq_sigmoid(float v) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-v))); }
__device__ __forceinline__ float gated_activation(int op, float g) {
    switch (op) {
        case FQ_GATED_GEGLU: {
            // 0.5 * v * (1 + tanh(sqrt(2/pi) * (v + 0.044715 v^3))), left to right
            const float arg = __fmul_rn(0.7978845608028654f, __fadd_rn(g, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, g), g), g)));
            return __fmul_rn(__fmul_rn(0.5f, g), __fadd_rn(1.0f, tanhf(arg)));
        }
        case FQ_GATED_SWIGLU_CLAMP10: {
            const float c = fminf(g, 10.0f);
            return __fmul_rn(c, fq_sigmoid(c));
        }
        case FQ_GATED_GLU: return fq_sigmoid(g);
        case FQ_GATED_SITU: return __fmul_rn(__fmul_rn(4.0f, tanhf(__fmul_rn(g, 0.25f))), fq_sigmoid(g));
        default: return __fmul_rn(g, fq_sigmoid(g));
    }
}
__device__ __forceinline__ float gated_source(int op, float u) {
    if (op == FQ_GATED_SWIGLU_CLAMP10) return fminf(fmaxf(u, -10.0f), 10.0f);
    if (op == FQ_GATED_SITU) return __fmul_rn(25.0f, tanhf(__fmul_rn(u, 0.04f)));
    return u;
}
__device__ __forceinline__ float gated_pair(int op, float gate, float up) { return __fmul_rn(gated_source(op, up), gated_activation(op, gate)); }

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    // 128-bit read-only load that does not allocate in L1: weights are used once.
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ldg_cached16(const void* p) { return __ldg((const uint4*)p); }


// K-quant 6-bit scale/min pair j of the 12-byte field held in three words
// (reference backend/quant/q8k.zig:637-648).
__device__ __forceinline__ void scale_min_k4(const uint32_t s[3], int j, int& sc, int& mn) {
    const uint8_t* q = reinterpret_cast<const uint8_t*>(s);
    if (j < 4) {
        sc = q[j] & 63;
        mn = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0x0f) | ((q[j - 4] >> 6) << 4);
        mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

template <int WIDTH>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int o = WIDTH / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace fq
