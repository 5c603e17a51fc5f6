// gpu_formats: weight repacking, bit-exact dequantisation, activation
// quantisation and weight encoders.
//
// This translation unit is compiled with -fmad=false: every value it produces
// must equal the reference's CPU code bit for bit, and that code never fuses a
// multiply with an add (Zig does not contract). Division and square root are
// IEEE-rounded under nvcc's defaults (-prec-div=true -prec-sqrt=true), and
// denormals are kept (-ftz=false).
#include "actquant.cuh"
#include "acts.cuh"
#include "internal.h"

namespace fq {

// ===========================================================================
// Repack GGUF rows <-> device rows.
// ===========================================================================
// One thread per block of the split formats (Q8_0, TQ2_0, folded, Q2_0): the
// payload goes to the row's payload plane, the f16 scale to its scale plane.
// GGUF blocks of these formats are only 2-byte aligned, so bytes move as u16.
template <bool TO_DEVICE>
__global__ void repack_split_kernel(uint8_t* dev, size_t dev_row_stride, size_t dev_mat_stride, uint8_t* gguf,
                                    size_t nb01, size_t nb02, int fmt, int n, int blocks_per_row, int n_mats) {
    const FormatInfo f = format_info(fmt);
    const size_t total = (size_t)n_mats * n * blocks_per_row;
    const bool scale_first = (fmt == FQ_Q8_0 || fmt == FQ_Q2_0);  // d precedes qs in the GGUF struct
    for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
        const int b = (int)(t % blocks_per_row);
        const size_t rowlin = t / blocks_per_row;
        const int row = (int)(rowlin % n);
        const int mat = (int)(rowlin / n);
        uint16_t* g = reinterpret_cast<uint16_t*>(gguf + (size_t)mat * nb02 + (size_t)row * nb01 + (size_t)b * f.block_bytes);
        uint8_t* drow = dev + (size_t)mat * dev_mat_stride + (size_t)row * dev_row_stride;
        uint16_t* dq = reinterpret_cast<uint16_t*>(drow + (size_t)b * f.qs_bytes);
        uint16_t* ds = reinterpret_cast<uint16_t*>(drow + (size_t)blocks_per_row * f.qs_bytes) + b;
        uint16_t* gq = scale_first ? g + 1 : g;
        uint16_t* gs = scale_first ? g : g + f.qs_bytes / 2;
        if (TO_DEVICE) {
            for (int i = 0; i < f.qs_bytes / 2; ++i) dq[i] = gq[i];
            *ds = *gs;
        } else {
            for (int i = 0; i < f.qs_bytes / 2; ++i) gq[i] = dq[i];
            *gs = *ds;
        }
    }
}

// K-quant rows keep their bytes; 16-byte pieces move between the GGUF rows and the
// device layout (row-major or tile-major, see common.cuh).
template <bool TO_DEVICE>
__global__ void kquant_rows_kernel(DevWeights w, uint8_t* gguf, size_t nb01, size_t nb02, int unit_bytes) {
    const size_t pieces = (size_t)(w.k >> 8) * unit_bytes / 16;
    const size_t total = (size_t)w.n_mats * w.n * pieces;
    const size_t ustride = unit_stride(w, unit_bytes);
    for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
        const size_t q = t % pieces;
        const size_t rowlin = t / pieces;
        const int row = (int)(rowlin % w.n), mat = (int)(rowlin / w.n);
        const size_t byte = q * 16, u = byte / unit_bytes, off = byte % unit_bytes;
        uint8_t* dev = const_cast<uint8_t*>(row_unit0(w, w.base + (size_t)mat * w.mat_stride, row, unit_bytes)) + u * ustride + off;
        uint8_t* g = gguf + (size_t)mat * nb02 + (size_t)row * nb01 + byte;
        if (TO_DEVICE)
            *reinterpret_cast<uint4*>(dev) = *reinterpret_cast<const uint4*>(g);
        else
            *reinterpret_cast<uint4*>(g) = *reinterpret_cast<const uint4*>(dev);
    }
}

static int grid_for(size_t total, int block) {
    size_t g = (total + block - 1) / block;
    if (g > 148 * 16) g = 148 * 16;
    if (g == 0) g = 1;
    return (int)g;
}

cudaError_t launch_repack(const DevWeights& w, const uint8_t* gguf_dev, size_t nb01, size_t nb02, bool to_device,
                          cudaStream_t st) {
    const FormatInfo f = format_info(w.fmt);
    const int bpr = w.k / f.block_elems;
    uint8_t* dev = const_cast<uint8_t*>(w.base);
    uint8_t* gg = const_cast<uint8_t*>(gguf_dev);
    if (f.sc_bytes == 0) {
        const size_t row_bytes = (size_t)bpr * f.block_bytes;
        const size_t total = (size_t)w.n_mats * w.n * (row_bytes / 16);
        (void)dev;
        if (to_device)
            kquant_rows_kernel<true><<<grid_for(total, 256), 256, 0, st>>>(w, gg, nb01, nb02, f.block_bytes);
        else
            kquant_rows_kernel<false><<<grid_for(total, 256), 256, 0, st>>>(w, gg, nb01, nb02, f.block_bytes);
    } else {
        const size_t total = (size_t)w.n_mats * w.n * bpr;
        if (to_device)
            repack_split_kernel<true><<<grid_for(total, 256), 256, 0, st>>>(dev, w.row_stride, w.mat_stride, gg, nb01, nb02, w.fmt, w.n, bpr, w.n_mats);
        else
            repack_split_kernel<false><<<grid_for(total, 256), 256, 0, st>>>(dev, w.row_stride, w.mat_stride, gg, nb01, nb02, w.fmt, w.n, bpr, w.n_mats);
    }
    return cudaGetLastError();
}

// ===========================================================================
// Dequantisation (bit-exact): one thread per element of the device layout.
// ===========================================================================
__device__ __forceinline__ void scale_min_one(const uint8_t* q, int j, int& sc, int& mn) {
    if (j < 4) {
        sc = q[j] & 63;
        mn = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0x0f) | ((q[j - 4] >> 6) << 4);
        mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

// Value of element e of one device row. Formulas, in the written order:
//   Q8_0   f32(q) * d                                  (q8k.zig:104-112)
//   Q4_K   d*f32(sc)*f32(q) - dmin*f32(mn)             (q4_k.zig:1954-1972)
//   Q5_K   same with q = nibble + 16*bit               (q5_k.zig:1154-1167, :1259-1264)
//   Q6_K   d*f32(scale)*f32(q6 - 32)                   (q6_k.zig:1159-1167)
//   TQ2_0  f32(code-1) * d                             (cold.zig:651-670)
//   folded d * (f32(cu) - 4)                           (ternary.zig:850-876)
//   Q2_0   f32(q-1) * d                                (cold.zig:289-301)
__device__ float dequant_element(const uint8_t* row, size_t ustride, int fmt, int k, int e) {
    switch (fmt) {
        case FQ_Q8_0: {
            const int8_t q = (int8_t)row[e];
            const uint16_t d = reinterpret_cast<const uint16_t*>(row + k)[e >> 5];
            return (float)q * h2f(d);
        }
        case FQ_Q4_K: {
            const uint8_t* b = row + (size_t)(e >> 8) * ustride;
            const int r = e & 255, s = r >> 5, i = r & 31;
            const float d = h2f(*reinterpret_cast<const uint16_t*>(b));
            const float dmin = h2f(*reinterpret_cast<const uint16_t*>(b + 2));
            int sc, mn;
            scale_min_one(b + 4, s, sc, mn);
            const uint8_t byte = b[16 + (s >> 1) * 32 + i];
            const int q = (s & 1) ? (byte >> 4) : (byte & 15);
            return d * (float)sc * (float)q - dmin * (float)mn;
        }
        case FQ_Q5_K: {
            const uint8_t* b = row + (size_t)(e >> 8) * ustride;
            const int r = e & 255, s = r >> 5, i = r & 31;
            const float d = h2f(*reinterpret_cast<const uint16_t*>(b));
            const float dmin = h2f(*reinterpret_cast<const uint16_t*>(b + 2));
            int sc, mn;
            scale_min_one(b + 4, s, sc, mn);
            const uint8_t byte = b[48 + (s >> 1) * 32 + i];
            const int q = ((s & 1) ? (byte >> 4) : (byte & 15)) + (((b[16 + i] >> s) & 1) ? 16 : 0);
            return d * (float)sc * (float)q - dmin * (float)mn;
        }
        case FQ_Q6_K: {  // d * f32(scale) * f32(q), left to right (q6_k.zig:1159-1167, :1239-1259)
            const int blk = e >> 8, r = e & 255, c2 = r >> 7, sec = (r >> 5) & 3, l = r & 31;
            const uint8_t* b = row + (size_t)blk * 208;
            const uint8_t qlb = b[c2 * 64 + (sec & 1) * 32 + l];
            const int low = (sec < 2) ? (qlb & 0x0f) : (qlb >> 4);
            const int high = (b[128 + c2 * 32 + l] >> (sec * 2)) & 3;
            const int q = (low | (high << 4)) - 32;
            const int sc = (int8_t)b[192 + c2 * 8 + sec * 2 + (l >> 4)];
            const uint16_t d = reinterpret_cast<const uint16_t*>(row + (size_t)(k >> 8) * 208)[blk];
            return h2f(d) * (float)sc * (float)q;
        }
        case FQ_TQ2_0: {
            const int blk = e >> 8, r = e & 255, hg = r >> 7, n = (r >> 5) & 3, m = r & 31;
            const int code = (row[blk * 64 + hg * 32 + m] >> (2 * n)) & 3;
            const uint16_t d = reinterpret_cast<const uint16_t*>(row + k / 4)[blk];
            return (float)(code - 1) * h2f(d);
        }
        case FQ_TQ2_0_FOLDED: {
            const int blk = e >> 8, r = e & 255, s = r >> 5, j = r & 31;
            const uint8_t byte = row[blk * 128 + s * 16 + (j & 15)];
            const int cu = (j < 16) ? (byte & 15) : (byte >> 4);
            const uint16_t d = reinterpret_cast<const uint16_t*>(row + k / 2)[blk];
            return h2f(d) * ((float)cu - 4.0f);
        }
        case FQ_Q2_0: {
            const int q = (row[e >> 2] >> ((e & 3) * 2)) & 3;
            const uint16_t d = reinterpret_cast<const uint16_t*>(row + k / 4)[e >> 7];
            return (float)(q - 1) * h2f(d);
        }
    }
    return 0.0f;
}

__global__ void dequant_rows_kernel(DevWeights w, int mat, int row0, int rows, float* out) {
    const size_t total = (size_t)rows * w.k;
    for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
        const int e = (int)(t % w.k);
        const int r = (int)(t / w.k);
        const int ub = format_info(w.fmt).block_bytes;  // K-quants: the unit is the block
        const uint8_t* row = row_unit0(w, w.base + (size_t)mat * w.mat_stride, row0 + r, ub);
        out[t] = dequant_element(row, unit_stride(w, ub), w.fmt, w.k, e);
    }
}

cudaError_t launch_dequant_rows(const DevWeights& w, int mat, int row0, int rows, float* out, cudaStream_t st) {
    const size_t total = (size_t)rows * w.k;
    dequant_rows_kernel<<<grid_for(total, 256), 256, 0, st>>>(w, mat, row0, rows, out);
    return cudaGetLastError();
}

// ===========================================================================
// Activation quantisation.
// ===========================================================================
// One warp per 256 activations of one row, written in the decode layout of
// acts.cuh. grid.x covers rows * k/256 warps.
__global__ void quantize_acts_layout_kernel(const float* __restrict__ a, const int* __restrict__ src_rows, int src_div, int m, int k,
                                            int fmt, uint8_t* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
    const int blocks_per_row = (k + 255) >> 8;
    if (warp >= (size_t)m * blocks_per_row) return;
    const int row = (int)(warp / blocks_per_row), blk = (int)(warp % blocks_per_row);
    const bool valid = blk * 256 + lane * 8 < k;  // only Q8_0-type rows can end inside a warp's span
    const ActLayout L = act_layout(fmt);
    const ActSizes S = act_sizes(fmt, k);
    const int C = k / L.chunk_elems;
    uint8_t* rec = out + (size_t)row * S.row;
    int8_t* aq = reinterpret_cast<int8_t*>(rec);
    uint8_t* aaux = rec + S.aq;
    float* ad = reinterpret_cast<float*>(rec + S.aq + S.aaux);

    const int srow = src_rows ? src_rows[row] / src_div : row;
    const float* src = a + (size_t)srow * k + (size_t)blk * 256 + lane * 8;
    float v[8];
    float4 v0 = make_float4(0, 0, 0, 0), v1 = v0;
    if (valid) {
        v0 = *reinterpret_cast<const float4*>(src);
        v1 = *reinterpret_cast<const float4*>(src + 4);
    }
    v[0] = v0.x, v[1] = v0.y, v[2] = v0.z, v[3] = v0.w, v[4] = v1.x, v[5] = v1.y, v[6] = v1.z, v[7] = v1.w;
    int q[8];
    const int e0 = blk * 256 + lane * 8;

    if (L.act_block == 256) {
        const float d = q8k_block(v, lane, q);
        if (lane == 0) ad[blk] = d;
        int c, s, i;
        act_pos(fmt, e0, c, s, i);
        uint2 packed;
        packed.x = pack4(q);
        packed.y = pack4(q + 4);
        *reinterpret_cast<uint2*>(aq + ((size_t)s * C + c) * 16 + i) = packed;
        int sum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += q[j];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);  // the Q8_K bsum of this 16-element group
        if (fmt == FQ_Q4_K || fmt == FQ_Q5_K || fmt == FQ_Q6_K) {
            // (Q6_K levels are re-centred to signed bytes in the kernel, which needs no sums; the word is kept defined)
            if ((lane & 1) == 0) reinterpret_cast<int16_t*>(aaux)[c * 2 + s] = (int16_t)sum;
        } else if (fmt == FQ_TQ2_0) {
            // chunk = the four crumb lanes n (lane bits 2,3) of one (half-group, half)
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            sum += __shfl_xor_sync(0xffffffffu, sum, 8);
            if ((lane & 13) == 0) reinterpret_cast<int32_t*>(aaux)[c] = sum;
        } else {  // folded: chunk = 32 elements, offset term is 4 * sum(a)
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if ((lane & 3) == 0) reinterpret_cast<int32_t*>(aaux)[c] = 4 * sum;
        }
    } else {
        const uint16_t dh = q8_0_quarter(v, q);
        // invalid lanes carry zeros and only skip their stores, so every
        // shuffle below still runs with the full warp
        if (valid && (lane & 3) == 0) ad[blk * 8 + (lane >> 2)] = h2f(dh);
        if (fmt == FQ_Q8_0) {
            if (valid) {
                uint2 packed;
                packed.x = pack4(q);
                packed.y = pack4(q + 4);
                *reinterpret_cast<uint2*>(aq + e0) = packed;
            }
        } else {  // FQ_Q2_0
            if (valid) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    int c, s, i;
                    act_pos(fmt, e0 + j, c, s, i);
                    aq[((size_t)s * C + c) * 16 + i] = (int8_t)q[j];
                }
            }
            int sum = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) sum += q[j];
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);  // sum over one 32-element activation block
            const int other = __shfl_xor_sync(0xffffffffu, sum, 4);
            // k % 128 == 0 for Q2_0: the 8 lanes of a 64-element chunk are valid together
            if (valid && (lane & 7) == 0)
                reinterpret_cast<uint32_t*>(aaux)[e0 >> 6] = ((uint32_t)sum & 0xffffu) | ((uint32_t)other << 16);
        }
    }
}

cudaError_t launch_quantize_acts_layout(const float* a, const int* src_rows, int src_div, int m, int k, int fmt, uint8_t* out,
                                        cudaStream_t st) {
    const size_t warps = (size_t)m * ((k + 255) / 256);
    const int threads = 128;
    const size_t blocks = (warps * 32 + threads - 1) / threads;
    quantize_acts_layout_kernel<<<(unsigned)blocks, threads, 0, st>>>(a, src_rows, src_div, m, k, fmt, out);
    return cudaGetLastError();
}

// Reference block structs (dtype.zig:148-152 BlockQ8_K, :83-86 BlockQ8_0), for
// callers that want the CPU representation and for parity checks.
__global__ void quantize_acts_struct_kernel(const float* __restrict__ a, int m, int k, int q8k, uint8_t* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
    const int blocks_per_row = (k + 255) >> 8;
    if (warp >= (size_t)m * blocks_per_row) return;
    const int row = (int)(warp / blocks_per_row), b256 = (int)(warp % blocks_per_row);
    const bool valid = b256 * 256 + lane * 8 < k;
    const float* src = a + (size_t)row * k + (size_t)b256 * 256 + lane * 8;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = valid ? src[j] : 0.0f;
    int q[8];
    if (q8k) {
        uint8_t* blk = out + warp * 292;
        const float d = q8k_block(v, lane, q);
        if (lane == 0) *reinterpret_cast<float*>(blk) = d;
        uint32_t* qs = reinterpret_cast<uint32_t*>(blk + 4 + lane * 8);
        qs[0] = pack4(q);
        qs[1] = pack4(q + 4);
        int sum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += q[j];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        if ((lane & 1) == 0) reinterpret_cast<int16_t*>(blk + 260)[lane >> 1] = (int16_t)sum;
    } else {
        const uint16_t dh = q8_0_quarter(v, q);
        if (!valid) return;
        uint8_t* blk = out + ((size_t)row * (k / 32) + b256 * 8 + (lane >> 2)) * 34;
        if ((lane & 3) == 0) *reinterpret_cast<uint16_t*>(blk) = dh;
#pragma unroll
        for (int j = 0; j < 8; ++j) blk[2 + (lane & 3) * 8 + j] = (uint8_t)q[j];
    }
}

cudaError_t launch_quantize_acts_struct(const float* a, int m, int k, bool q8k, uint8_t* out, cudaStream_t st) {
    const size_t warps = (size_t)m * ((k + 255) / 256);
    const int threads = 128;
    const size_t blocks = (warps * 32 + threads - 1) / threads;
    quantize_acts_struct_kernel<<<(unsigned)blocks, threads, 0, st>>>(a, m, k, q8k ? 1 : 0, out);
    return cudaGetLastError();
}

// Natural-order records for the row-per-lane decode kernel (actquant.cuh).
__global__ void quantize_acts_natural_kernel(const float* __restrict__ a, int m, int k, int q8k, uint8_t* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
    const int blocks_per_row = k >> 8;
    if (warp >= (size_t)m * blocks_per_row) return;
    const int row = (int)(warp / blocks_per_row), blk = (int)(warp % blocks_per_row);
    const NatSizes S = nat_sizes(q8k != 0, k);
    quantize_block_natural(a + (size_t)row * k, blk, q8k, k, out + (size_t)row * S.row, lane);
}

// `q8k`: 0, 1 or 2 as in quantize_values_natural
cudaError_t launch_quantize_acts_natural(const float* a, int m, int k, int q8k, uint8_t* out, cudaStream_t st) {
    const size_t warps = (size_t)m * (k / 256);
    const int threads = 128;
    const size_t blocks = (warps * 32 + threads - 1) / threads;
    quantize_acts_natural_kernel<<<(unsigned)blocks, threads, 0, st>>>(a, m, k, q8k, out);
    return cudaGetLastError();
}

// Stand-alone activation prologue (actquant.cuh): one CTA per row, its warps over the row's 256-element blocks. The
// arithmetic and its order are those of the decode kernel's fused prologue, so both forms give the same bits.
__global__ void __launch_bounds__(256) act_prologue_kernel(const PreArgs P, const float* __restrict__ a, float* __restrict__ out, int k) {
    extern __shared__ float block_sums[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int nblk = k >> 8;
    const float* row = a + (size_t)blockIdx.x * (P.op == FQ_PRE_SPLIT_SWIGLU ? (size_t)2 * k : (size_t)k);
    float scale = 0.0f;
    if (P.op == FQ_PRE_RMS_NORM_MUL) {
        for (int blk = warp; blk < nblk; blk += nwarps) {
            float v[8];
            load8(row + (size_t)blk * 256 + lane * 8, v);
            const float ss = block_sumsq(v);
            if (lane == 0) block_sums[blk] = ss;
        }
        __syncthreads();
        scale = rms_scale(block_sums, nblk, P.eps);
    }
    float* orow = out + (size_t)blockIdx.x * k;
    for (int blk = warp; blk < nblk; blk += nwarps) {
        float v[8];
        load_block_pre(P, row, (size_t)k, blk, lane, scale, v);
        float* dst = orow + (size_t)blk * 256 + lane * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
}
cudaError_t launch_act_prologue(const PreArgs& pre, const float* a, float* out, int m, int k, cudaStream_t st) {
    act_prologue_kernel<<<(unsigned)m, 256, (size_t)(k >> 8) * sizeof(float), st>>>(pre, a, out, k);
    return cudaGetLastError();
}

// ===========================================================================
// Weight encoders (raw GGUF blocks out, byte-identical to the CPU encoders).
// ===========================================================================
__device__ __forceinline__ int max_i(int a, int b) { return a > b ? a : b; }
__device__ __forceinline__ int min_i(int a, int b) { return a < b ? a : b; }
__device__ __forceinline__ int nearest_int_dev(float fval) {
    const float val = fval + 12582912.0f;
    return (__float_as_int(val) & 0x007fffff) - 0x00400000;
}

// q8k.zig:734-818 for one 32-element sub-block; L/Laux live in shared memory.
__device__ float make_qkx2_quants_dev(int nmax, const float* x, const float* weights, uint8_t* L, float* the_min,
                                      uint8_t* Laux, float rmin, float rdelta, int nstep) {
    float mn = x[0], mx = x[0];
    float sum_w = weights[0];
    float sum_x = sum_w * x[0];
    for (int i = 1; i < 32; ++i) {
        if (x[i] < mn) mn = x[i];
        if (x[i] > mx) mx = x[i];
        sum_w += weights[i];
        sum_x += weights[i] * x[i];
    }
    if (mn > 0) mn = 0;
    if (mx == mn) {
        for (int i = 0; i < 32; ++i) L[i] = 0;
        *the_min = -mn;
        return 0.0f;
    }
    const float nmax_f = (float)nmax;
    float iscale = nmax_f / (mx - mn);
    float scale = 1 / iscale;
    float best_error = 0;
    for (int i = 0; i < 32; ++i) {
        const int l = nearest_int_dev(iscale * (x[i] - mn));
        L[i] = (uint8_t)max(0, min(nmax, l));
        float diff = scale * (float)L[i] + mn - x[i];
        diff = diff * diff;
        best_error += weights[i] * diff;
    }
    for (int is = 0; is <= nstep; ++is) {
        iscale = (rmin + rdelta * (float)is + nmax_f) / (mx - mn);
        float sum_l = 0, sum_l2 = 0, sum_xl = 0;
        for (int i = 0; i < 32; ++i) {
            int l = nearest_int_dev(iscale * (x[i] - mn));
            l = max(0, min(nmax, l));
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
            for (int i = 0; i < 32; ++i) {
                float diff = this_scale * (float)Laux[i] + this_min - x[i];
                diff = diff * diff;
                cur_error += weights[i] * diff;
            }
            if (cur_error < best_error) {
                for (int i = 0; i < 32; ++i) L[i] = Laux[i];
                best_error = cur_error;
                scale = this_scale;
                mn = this_min;
            }
        }
    }
    *the_min = -mn;
    return scale;
}

// Q4_K (q4_k.zig:1977-2048) and Q5_K (q5_k.zig:1172-1257): eight threads per
// 256-element block, one per 32-element sub-block. 128 threads = 16 blocks.
template <bool Q5>
__global__ void __launch_bounds__(128) quantize_kquant_kernel(const float* __restrict__ src, size_t nblocks, uint8_t* __restrict__ dst) {
    __shared__ uint8_t sL[16][256];
    __shared__ uint8_t sLaux[128][32];
    constexpr int NMAX = Q5 ? 31 : 15;
    constexpr int BYTES = Q5 ? 176 : 144;
    const int j = threadIdx.x & 7;
    const int lb = threadIdx.x >> 3;
    const size_t bi = blockIdx.x * (size_t)16 + lb;
    const bool live = bi < nblocks;
    const size_t bsafe = live ? bi : (nblocks - 1);
    const float* xs = src + bsafe * 256 + j * 32;
    float x[32], wts[32];
    float sum_x2 = 0;
    for (int i = 0; i < 32; ++i) {
        x[i] = xs[i];
        sum_x2 += x[i] * x[i];
    }
    const float av_x = sqrtf(sum_x2 / 32);
    for (int i = 0; i < 32; ++i) wts[i] = av_x + fabsf(x[i]);
    uint8_t* L = &sL[lb][j * 32];
    float the_min;
    const float scale = make_qkx2_quants_dev(NMAX, x, wts, L, &the_min, sLaux[threadIdx.x], Q5 ? -0.5f : -1.0f, 0.1f, Q5 ? 15 : 20);
    float max_scale = fmaxf(0.0f, scale), max_min = fmaxf(0.0f, the_min);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
        max_scale = fmaxf(max_scale, __shfl_xor_sync(0xffffffffu, max_scale, o));
        max_min = fmaxf(max_min, __shfl_xor_sync(0xffffffffu, max_min, o));
    }
    const float inv_scale = max_scale > 0 ? 63.0f / max_scale : 0.0f;
    const float inv_min = max_min > 0 ? 63.0f / max_min : 0.0f;
    int ls = nearest_int_dev(inv_scale * scale) & 0xff;  // truncated to u8 before the clamp
    int lm = nearest_int_dev(inv_min * the_min) & 0xff;
    ls = min(63, ls);
    lm = min(63, lm);
    const int ls_hi = __shfl_down_sync(0xffffffffu, ls, 4, 8);
    const int lm_hi = __shfl_down_sync(0xffffffffu, lm, 4, 8);
    const uint16_t dh = __half_as_ushort(__float2half_rn(max_scale / 63.0f));
    const uint16_t dmh = __half_as_ushort(__float2half_rn(max_min / 63.0f));
    uint8_t* out = dst + bsafe * BYTES;
    if (live) {
        if (j == 0) {
            reinterpret_cast<uint16_t*>(out)[0] = dh;
            reinterpret_cast<uint16_t*>(out)[1] = dmh;
        }
        if (j < 4) {
            out[4 + j] = (uint8_t)(ls | ((ls_hi >> 4) << 6));
            out[4 + j + 4] = (uint8_t)(lm | ((lm_hi >> 4) << 6));
        } else {
            out[4 + j + 4] = (uint8_t)((ls & 0x0f) | ((lm & 0x0f) << 4));
        }
    }
    const float d = h2f(dh) * (float)ls;
    if (d != 0) {
        const float dm = h2f(dmh) * (float)lm;
        for (int i = 0; i < 32; ++i) {
            const int l = nearest_int_dev((x[i] + dm) / d);
            L[i] = (uint8_t)max(0, min(NMAX, l));
        }
    }
    __syncwarp();
    // thread j packs payload bytes j*16 .. j*16+15: byte q pairs levels of
    // sub-blocks 2p (low nibble) and 2p+1 (high), p = q/32
    if (live) {
        const uint8_t* LB = sL[lb];
        uint8_t* qs = out + (Q5 ? 48 : 16);
        for (int t = 0; t < 16; ++t) {
            const int qb = j * 16 + t, p = qb >> 5, l = qb & 31;
            const uint8_t l1 = LB[p * 64 + l], l2 = LB[p * 64 + 32 + l];
            qs[qb] = (uint8_t)((l1 & 15) | ((l2 & 15) << 4));
        }
        if (Q5) {
            for (int t = 0; t < 4; ++t) {
                const int jj = j * 4 + t;
                uint8_t h = 0;
                for (int p = 0; p < 4; ++p) {
                    if (LB[p * 64 + jj] > 15) h |= (uint8_t)(1u << (2 * p));
                    if (LB[p * 64 + 32 + jj] > 15) h |= (uint8_t)(2u << (2 * p));
                }
                out[16 + jj] = h;
            }
        }
    }
}

// q8k.zig:665-733 `makeQxQuants` for one 16-element group with rmse_type 1 (weights v*v), nmax 32: the scale search of
// ggml's make_qx_quants. Levels come back biased by nmax.
__device__ float make_qx_quants16_dev(const float* x, int8_t* L) {
    constexpr int nmax = 32;
    float max = 0, amax = 0;
    for (int i = 0; i < 16; ++i) {
        const float ax = fabsf(x[i]);
        if (ax > amax) {
            amax = ax;
            max = x[i];
        }
    }
    if (amax < 1e-15f) {
        for (int i = 0; i < 16; ++i) L[i] = 0;
        return 0.0f;
    }
    float iscale = -32.0f / max;
    float sumlx = 0, suml2 = 0;
    for (int i = 0; i < 16; ++i) {
        int l = nearest_int_dev(iscale * x[i]);
        l = max_i(-nmax, min_i(nmax - 1, l));
        L[i] = (int8_t)(l + nmax);
        const float w = x[i] * x[i];
        const float lf = (float)l;
        sumlx += w * x[i] * lf;
        suml2 += w * lf * lf;
    }
    float scale = (suml2 != 0) ? sumlx / suml2 : 0.0f;
    float best = scale * sumlx;
    for (int is = -9; is <= 9; ++is) {
        if (is == 0) continue;
        iscale = -(32.0f + 0.1f * (float)is) / max;
        sumlx = 0;
        suml2 = 0;
        for (int i = 0; i < 16; ++i) {
            int l = nearest_int_dev(iscale * x[i]);
            l = max_i(-nmax, min_i(nmax - 1, l));
            const float w = x[i] * x[i];
            const float lf = (float)l;
            sumlx += w * x[i] * lf;
            suml2 += w * lf * lf;
        }
        if (suml2 > 0 && sumlx * sumlx > best * suml2) {
            for (int i = 0; i < 16; ++i) {
                const int l = nearest_int_dev(iscale * x[i]);
                L[i] = (int8_t)(nmax + max_i(-nmax, min_i(nmax - 1, l)));
            }
            scale = sumlx / suml2;
            best = scale * sumlx;
        }
    }
    return scale;
}

// Q6_K (q6_k.zig:1172-1229, the port of ggml's quantize_row_q6_K_ref): sixteen threads per 256-element block,
// one per 16-element group. 128 threads = 8 blocks.
__global__ void __launch_bounds__(128) quantize_q6_k_kernel(const float* __restrict__ src, size_t nblocks, uint8_t* __restrict__ dst) {
    __shared__ int8_t sL[8][256];
    const int j = threadIdx.x & 15;
    const int lb = threadIdx.x >> 4;
    const size_t bi = blockIdx.x * (size_t)8 + lb;
    const bool live = bi < nblocks;
    const size_t bsafe = live ? bi : (nblocks - 1);
    const float* xs = src + bsafe * 256 + j * 16;
    float x[16];
    for (int i = 0; i < 16; ++i) x[i] = xs[i];
    int8_t* L = &sL[lb][j * 16];
    const float scale = make_qx_quants16_dev(x, L);
    // the scale of largest magnitude, the first one on ties (a strict > in the sequential walk)
    float best_abs = fabsf(scale);
    int best_j = j;
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, best_abs, o, 16);
        const int oj = __shfl_xor_sync(0xffffffffu, best_j, o, 16);
        if (oa > best_abs || (oa == best_abs && oj < best_j)) best_abs = oa, best_j = oj;
    }
    const float max_scale = __shfl_sync(0xffffffffu, scale, best_j, 16);
    uint8_t* out = dst + bsafe * 210;
    if (best_abs < 1e-15f) {
        if (live)
            for (int i = j; i < 105; i += 16) reinterpret_cast<uint16_t*>(out)[i] = 0;
        return;  // the sixteen threads of a block leave together
    }
    const float iscale = -128.0f / max_scale;
    const uint16_t dh = __half_as_ushort(__float2half_rn(1 / iscale));
    const int sc = min_i(127, nearest_int_dev(iscale * scale));
    const float d = h2f(dh) * (float)sc;
    if (d != 0) {
        for (int i = 0; i < 16; ++i) {
            const int l = nearest_int_dev(x[i] / d);
            L[i] = (int8_t)(max_i(-32, min_i(31, l)) + 32);
        }
    }
    __syncwarp();
    if (!live) return;
    out[192 + j] = (uint8_t)(int8_t)sc;
    if (j == 0) reinterpret_cast<uint16_t*>(out + 208)[0] = dh;
    // thread j packs ql bytes j*8 .. j*8+7 and qh bytes j*4 .. j*4+3
    const int8_t* LB = sL[lb];
    for (int t = 0; t < 8; ++t) {
        const int qb = j * 8 + t, c2 = qb >> 6, r = qb & 63, hi32 = r >> 5, l = r & 31;
        const uint8_t qa = (uint8_t)LB[c2 * 128 + hi32 * 32 + l], qc = (uint8_t)LB[c2 * 128 + (hi32 + 2) * 32 + l];
        out[qb] = (uint8_t)((qa & 0x0f) | ((qc & 0x0f) << 4));
    }
    for (int t = 0; t < 4; ++t) {
        const int hb = j * 4 + t, c2 = hb >> 5, l = hb & 31;
        const uint8_t q1 = (uint8_t)LB[c2 * 128 + l], q2 = (uint8_t)LB[c2 * 128 + 32 + l], q3 = (uint8_t)LB[c2 * 128 + 64 + l],
                      q4 = (uint8_t)LB[c2 * 128 + 96 + l];
        out[128 + hb] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
    }
}

// Q8_0 (q8k.zig:49-69), TQ2_0 (ternary.zig:79-144), Q2_0 (cold.zig:309-332):
// one warp per 256 source elements.
__global__ void quantize_simple_kernel(const float* __restrict__ src, size_t total, int fmt, uint8_t* __restrict__ dst) {
    const int lane = threadIdx.x & 31;
    const size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
    if (warp * 256 >= total) return;
    const float* s = src + warp * 256;
    // blocks never straddle the end (total is a multiple of the block size), so
    // whole 4-lane (Q8_0) or 16-lane (Q2_0) groups are valid together
    const bool valid = warp * 256 + (size_t)lane * 8 < total;
    if (fmt == FQ_Q8_0) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = valid ? s[lane * 8 + j] : 0.0f;
        int q[8];
        const uint16_t dh = q8_0_quarter(v, q);
        if (!valid) return;
        uint8_t* blk = dst + (warp * 8 + (lane >> 2)) * 34;
        if ((lane & 3) == 0) *reinterpret_cast<uint16_t*>(blk) = dh;
#pragma unroll
        for (int j = 0; j < 8; ++j) blk[2 + (lane & 3) * 8 + j] = (uint8_t)q[j];
    } else if (fmt == FQ_TQ2_0) {
        float amax = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(s[lane * 8 + j]));
        amax = warp_max(amax);
        const float id = (amax != 0) ? 1.0f / amax : 0.0f;
        uint8_t* blk = dst + warp * 66;
        if (lane == 0) *reinterpret_cast<uint16_t*>(blk + 64) = __half_as_ushort(__float2half_rn(amax));
        for (int b = lane; b < 64; b += 32) {
            const int hg = b >> 5, m = b & 31;
            uint8_t qb = 0;
            for (int n = 0; n < 4; ++n) {
                const float r = roundf(s[hg * 128 + n * 32 + m] * id);
                const float bounded = isnan(r) ? 0.0f : fminf(1.0f, fmaxf(-1.0f, r));
                qb = (uint8_t)(qb + ((((int)bounded + 1) & 3) << (2 * n)));
            }
            blk[b] = qb;
        }
    } else {  // FQ_Q2_0: two 128-element blocks per warp, 16 lanes each, 4 elements per byte
        const int half = lane >> 4, l16 = lane & 15;
        const float* x = s + half * 128;
        float amax = 0;
        if (valid)
            for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(x[l16 * 8 + j]));
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (!valid) return;
        float inv_d = (amax != 0) ? 1.0f / amax : 0.0f;
        if (!isfinite(inv_d)) inv_d = 0;
        uint8_t* blk = dst + (warp * 2 + half) * 34;
        if (l16 == 0) *reinterpret_cast<uint16_t*>(blk) = __half_as_ushort(__float2half_rn(amax));
        for (int b = l16; b < 32; b += 16) {
            uint8_t qb = 0;
            for (int t = 0; t < 4; ++t) {
                const float r = fmaxf(0.0f, fminf(3.0f, roundf(x[b * 4 + t] * inv_d) + 1.0f));
                qb |= (uint8_t)((int)r << (t * 2));
            }
            blk[2 + b] = qb;
        }
    }
}

cudaError_t launch_quantize_weights(int fmt, const float* src, size_t n, size_t k, uint8_t* dst, cudaStream_t st) {
    const size_t total = n * k;
    if (fmt == FQ_Q4_K || fmt == FQ_Q5_K) {
        const size_t nblocks = total / 256;
        const unsigned grid = (unsigned)((nblocks + 15) / 16);
        if (fmt == FQ_Q4_K)
            quantize_kquant_kernel<false><<<grid, 128, 0, st>>>(src, nblocks, dst);
        else
            quantize_kquant_kernel<true><<<grid, 128, 0, st>>>(src, nblocks, dst);
    } else if (fmt == FQ_Q6_K) {
        const size_t nblocks = total / 256;
        quantize_q6_k_kernel<<<(unsigned)((nblocks + 7) / 8), 128, 0, st>>>(src, nblocks, dst);
    } else {
        const size_t n256 = (total + 255) / 256;
        const unsigned grid = (unsigned)((n256 * 32 + 127) / 128);
        quantize_simple_kernel<<<grid, 128, 0, st>>>(src, total, fmt, dst);
    }
    return cudaGetLastError();
}

}  // namespace fq
