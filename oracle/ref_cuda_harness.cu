// Launch shim for the reference's own CUDA kernels (test and bench infrastructure, never shipped, never linked
// into the product library).
//
// The build recipe (oracle/build.py, build_ref_cuda) compiles this file with the reference's
// src/backend/cuda/kernels.cu force-included in front of it (nvcc -include <reference>/src/backend/cuda/kernels.cu),
// from the place where the reference lies, for sm_100a, into oracle/_ref/libref_cuda.so. Nothing of the reference
// is copied: the kernels below are the reference's symbols, this file only launches them with the grid and block
// shapes its host code uses:
//   gemv            backend/cuda.zig:2054-2073   grid ceil(n/4), block 128
//   mul_mm_mma      backend/cuda.zig:2075-2140   grid (tiles, ceil(n/n_tile), split_k), block (16, 16 | 8)
//   launch plan     backend/cuda.zig:1940-1987   N64 / N32 tiles and split-K 2 (3 for Q6_K) below 7/8 of the SMs
//   split-K reduce  backend/cuda/kernels.cu:454-483, launched as backend/cuda.zig:2136-2143
//   attention       backend/cuda.zig:2684-2708   grid (ceil(q_seq/4), heads), block 128
// Format ids follow the reference's QFormat order: 0 q8_0, 1 q6_K, 2 q4_K, 3 q5_K.
#include <cuda_runtime.h>

extern "C" {

int refk_gemv(int fmt, const void* w, const float* x, float* y, int k, int n, int m, unsigned long long nb01, void* stream) {
    if (m < 1 || m > 8 || n < 1 || k < 1 || k % 16) return 1;
    dim3 grid((n + GEMV_WARPS - 1) / GEMV_WARPS), block(32 * GEMV_WARPS);
    cudaStream_t st = (cudaStream_t)stream;
    const char* src0 = (const char*)w;
    switch (fmt) {
        case 0: fucina_gemv_q8_0<<<grid, block, 0, st>>>(src0, x, y, k, n, m, nb01); break;
        case 1: fucina_gemv_q6_K<<<grid, block, 0, st>>>(src0, x, y, k, n, m, nb01); break;
        case 2: fucina_gemv_q4_K<<<grid, block, 0, st>>>(src0, x, y, k, n, m, nb01); break;
        case 3: fucina_gemv_q5_K<<<grid, block, 0, st>>>(src0, x, y, k, n, m, nb01); break;
        default: return 1;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// The reference's tile-shape rule restated: n_tile 64 or 32 and the split-K factor for a table of grid_x tiles.
void refk_plan(int fmt, int sm_count, long long grid_x, long long n, long long k, int allow_split_k, int* n_tile, int* split_k) {
    *n_tile = 64, *split_k = 1;
    if (sm_count <= 0) return;
    const long long n64_blocks = grid_x * ((n + 63) / 64);
    const long long ceiling = sm_count - sm_count / 8;
    if (allow_split_k && n64_blocks < ceiling) {
        const long long desired = (sm_count + n64_blocks - 1) / n64_blocks;
        const long long cap = fmt == 1 ? 3 : 2;
        long long by_k = k / 128;
        if (by_k < 1) by_k = 1;
        const long long max_split = cap < by_k ? cap : by_k;
        const long long s = desired < max_split ? desired : max_split;
        if (s > 1) {
            *split_k = (int)s;
            return;
        }
    }
    if (n64_blocks * 3 < 2LL * sm_count) *n_tile = 32;
}

// One grouped launch over `n_tiles` entries of {expert, base_row, m, tile_m} (device memory). `partial` holds
// split_k planes of partial_stride floats when split_k > 1 and the reduction is queued behind the product.
int refk_mul_mm(int fmt, const void* w, const float* a, const void* tiles, int n_tiles, float* dst, int k, int n,
                unsigned long long nb01, unsigned long long nb02, float* partial, int split_k, unsigned long long partial_stride,
                int n_tile, void* stream) {
    if (n_tiles < 1 || k % 32 || n < 1 || split_k < 1 || (split_k > 1 && !partial) || (n_tile != 64 && n_tile != 32)) return 1;
    if (((unsigned long long)a & 15) != 0) return 1;  // the reference keeps unaligned inputs on its scalar kernel
    dim3 grid(n_tiles, (n + n_tile - 1) / n_tile, split_k), block(16, n_tile == 64 ? 16 : 8);
    cudaStream_t st = (cudaStream_t)stream;
    const char* src0 = (const char*)w;
    const fucina_qmm_tile* t = (const fucina_qmm_tile*)tiles;
#define REFK_CASE(ID, NAME)                                                                                              \
    case ID:                                                                                                             \
        if (n_tile == 64) fucina_mul_mm_mma_##NAME<<<grid, block, 0, st>>>(src0, a, t, dst, k, n, nb01, nb02, partial, split_k, partial_stride); \
        else fucina_mul_mm_mma_n32_##NAME<<<grid, block, 0, st>>>(src0, a, t, dst, k, n, nb01, nb02, partial, split_k, partial_stride);         \
        break;
    switch (fmt) {
        REFK_CASE(0, q8_0)
        REFK_CASE(1, q6_K)
        REFK_CASE(2, q4_K)
        REFK_CASE(3, q5_K)
        default: return 1;
    }
#undef REFK_CASE
    if (cudaGetLastError() != cudaSuccess) return -1;
    if (split_k > 1) {
        const unsigned long long elements = partial_stride;
        const unsigned threads = 256;
        const unsigned long long quads = (elements + 3) / 4;
        fucina_reduce_split_k<<<(unsigned)((quads + threads - 1) / threads), threads, 0, st>>>(partial, dst, elements, split_k);
        if (cudaGetLastError() != cudaSuccess) return -1;
    }
    return 0;
}

// Streaming attention forward: q/o [q_seq][heads][d] f32, k/v [kv_seq][kv_heads][d] f16 or f32, kvmap [heads],
// stats (may be null) [heads][q_seq][2].
int refk_attn_fwd(int kv_is_f16, const float* q, const void* k, const void* v, float* o, float* stats, const int* kvmap, int q_seq,
                  int kv_seq, int heads, int kv_heads, int d, int source_offset, float scale, int window, int causal, void* stream) {
    if (q_seq < 1 || kv_seq < 1 || heads < 1 || kv_heads < 1 || d < 1 || d > ATTN_MAX_D) return 1;
    dim3 grid((q_seq + ATTN_WARPS - 1) / ATTN_WARPS, heads), block(32 * ATTN_WARPS);
    cudaStream_t st = (cudaStream_t)stream;
    if (kv_is_f16)
        fucina_attn_fwd_f16<<<grid, block, 0, st>>>(q, (const __half*)k, (const __half*)v, o, stats, kvmap, q_seq, kv_seq, heads, kv_heads, d,
                                                    source_offset, scale, window, causal);
    else
        fucina_attn_fwd_f32<<<grid, block, 0, st>>>(q, (const float*)k, (const float*)v, o, stats, kvmap, q_seq, kv_seq, heads, kv_heads, d,
                                                    source_offset, scale, window, causal);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"
