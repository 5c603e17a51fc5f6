// Decode-shaped quantized GEMV / small-batch GEMM for sm_100a.
//
// c[b, j] = sum_e a[b, e] * dequant(W)[j, e] for b < m <= 16, computed the way
// the reference's CPU kernels do: activations are int8 (Q8_K or Q8_0 blocks,
// src/backend/native.zig:427-490), block dots are exact integers, and the f32
// epilogue per block keeps the reference's association
//   Q8_0   f32(idot) * (d_a * d_w)                      q8_0.zig:1074-1089
//   Q4_K   (d_w*d_a)*f32(iscale) - (dmin_w*d_a)*f32(imin)   q4_k.zig:895-913
//   Q5_K   same with 5-bit levels                       q5_k.zig:1093-1111
//   TQ2_0  (d_w*d_a) * f32(sum(code*a) - sum(a))        ternary.zig:377-386
//   folded (d_w*d_a) * f32(sum(cu*a) - 4*sum(a))        ternary.zig:780-786
//   Q2_0   d_w*d_a*f32(sum((q-1)*a)) per 32 activations cold.zig:1988-2010
// Only the order in which per-block terms are added differs (lanes hold
// partial sums that a shuffle tree combines), which moves results by a few
// f32 ulps.
//
// Work split: a group of LPR lanes owns R consecutive weight rows; lane l of
// the group walks the row's 16-byte payload chunks l, l+LPR, ... . Each chunk
// is one coalesced 128-bit load per lane (a warp reads 512 contiguous bytes
// per instruction), unpacked in registers, and multiplied with dp4a against
// the activation segments staged once per CTA in shared memory. The kernel is
// HBM-bound: per weight row it reads the row once and nothing else from DRAM.
#include "acts.cuh"
#include "internal.h"

namespace fq {

// y extent of a grouped launch (the hardware limit; a test seam lowers it to exercise the striding walk)
static int g_gemv_grid_y_limit = 65535;

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ uint4 ld_weight16(const void* p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint16_t ld_scale16(const void* p) { return __ldg(reinterpret_cast<const uint16_t*>(p)); }

__device__ __forceinline__ int dot16_u(const uint32_t w[4], const int4& a) {
    int d = __dp4a((int)w[0], a.x, 0);
    d = __dp4a((int)w[1], a.y, d);
    d = __dp4a((int)w[2], a.z, d);
    return __dp4a((int)w[3], a.w, d);
}

// ---- per-format chunk handling ---------------------------------------------
// load():   issue the global loads for chunk c of one weight row
// decode(): unpack to dp4a operands and per-chunk scales
// term():   contribution of the chunk to one activation row, given the SEGS
//           activation segments, the chunk's aux word and the activation scale
//           plane of that row.
template <int FMT>
struct Chunk;

template <>
struct Chunk<FQ_Q8_0> {
    uint4 q;
    float d;
    __device__ __forceinline__ void load(const uint8_t* row, int c, int k, size_t) {
        q = ld_weight16(row + (size_t)c * 16);
        d = h2f(ld_scale16(row + k + (c >> 1) * 2));
    }
    __device__ __forceinline__ void decode(int) {}
    __device__ __forceinline__ float term(const int4* a, uint32_t, const float* ad, int c) const {
        int dot = __dp4a((int)q.x, a[0].x, 0);
        dot = __dp4a((int)q.y, a[0].y, dot);
        dot = __dp4a((int)q.z, a[0].z, dot);
        dot = __dp4a((int)q.w, a[0].w, dot);
        return (float)dot * (ad[c >> 1] * d);
    }
};

template <>
struct Chunk<FQ_Q4_K> {
    uint4 hdr, q;
    uint32_t lo[4], hi[4];
    int sc0, sc1, mn0, mn1;
    float d, dmin;
    __device__ __forceinline__ void load(const uint8_t* row, int c, int, size_t ustride) {
        const uint8_t* b = row + (size_t)(c >> 3) * ustride;
        hdr = ldg_cached16(b);  // shared by the 8 lanes of this block
        q = ld_weight16(b + 16 + (c & 7) * 16);
    }
    __device__ __forceinline__ void unpack_scales(int p) {
        const __half2 dm = *reinterpret_cast<const __half2*>(&hdr.x);
        d = __low2float(dm);
        dmin = __high2float(dm);
        const uint32_t s0 = hdr.y, s1 = hdr.z, s2 = hdr.w;
        if (p < 2) {
            const int sh = 16 * p;
            sc0 = (s0 >> sh) & 63;
            sc1 = (s0 >> (sh + 8)) & 63;
            mn0 = (s1 >> sh) & 63;
            mn1 = (s1 >> (sh + 8)) & 63;
        } else {
            const int sh = 16 * (p - 2);
            sc0 = ((s2 >> sh) & 0xf) | (((s0 >> (sh + 6)) & 3) << 4);
            mn0 = ((s2 >> (sh + 4)) & 0xf) | (((s1 >> (sh + 6)) & 3) << 4);
            sc1 = ((s2 >> (sh + 8)) & 0xf) | (((s0 >> (sh + 14)) & 3) << 4);
            mn1 = ((s2 >> (sh + 12)) & 0xf) | (((s1 >> (sh + 14)) & 3) << 4);
        }
    }
    __device__ __forceinline__ void decode(int c) {
        unpack_scales((c & 7) >> 1);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            lo[j] = w[j] & 0x0f0f0f0fu;
            hi[j] = (w[j] >> 4) & 0x0f0f0f0fu;
        }
    }
    __device__ __forceinline__ float term(const int4* a, uint32_t aux, const float* ad, int c) const {
        const int isc = sc0 * dot16_u(lo, a[0]) + sc1 * dot16_u(hi, a[1]);
        const int imn = mn0 * (int)(int16_t)(aux & 0xffffu) + mn1 * (int)(int16_t)(aux >> 16);
        const float da = ad[c >> 3];
        return (d * da) * (float)isc - (dmin * da) * (float)imn;
    }
};

template <>
struct Chunk<FQ_Q5_K> {
    uint4 hdr, qh, q;
    uint32_t lo[4], hi[4];
    int sc0, sc1, mn0, mn1;
    float d, dmin;
    __device__ __forceinline__ void load(const uint8_t* row, int c, int, size_t ustride) {
        const uint8_t* b = row + (size_t)(c >> 3) * ustride;
        hdr = ldg_cached16(b);
        qh = ldg_cached16(b + 16 + (c & 1) * 16);  // fifth bits of elements h*16..h*16+15, all 8 sub-blocks
        q = ld_weight16(b + 48 + (c & 7) * 16);
    }
    __device__ __forceinline__ void decode(int c) {
        const int p = (c & 7) >> 1;
        const __half2 dm = *reinterpret_cast<const __half2*>(&hdr.x);
        d = __low2float(dm);
        dmin = __high2float(dm);
        const uint32_t s0 = hdr.y, s1 = hdr.z, s2 = hdr.w;
        if (p < 2) {
            const int sh = 16 * p;
            sc0 = (s0 >> sh) & 63;
            sc1 = (s0 >> (sh + 8)) & 63;
            mn0 = (s1 >> sh) & 63;
            mn1 = (s1 >> (sh + 8)) & 63;
        } else {
            const int sh = 16 * (p - 2);
            sc0 = ((s2 >> sh) & 0xf) | (((s0 >> (sh + 6)) & 3) << 4);
            mn0 = ((s2 >> (sh + 4)) & 0xf) | (((s1 >> (sh + 6)) & 3) << 4);
            sc1 = ((s2 >> (sh + 8)) & 0xf) | (((s0 >> (sh + 14)) & 3) << 4);
            mn1 = ((s2 >> (sh + 12)) & 0xf) | (((s1 >> (sh + 14)) & 3) << 4);
        }
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        const uint32_t hb[4] = {qh.x, qh.y, qh.z, qh.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            lo[j] = (w[j] & 0x0f0f0f0fu) | (((hb[j] >> (2 * p)) & 0x01010101u) << 4);
            hi[j] = ((w[j] >> 4) & 0x0f0f0f0fu) | (((hb[j] >> (2 * p + 1)) & 0x01010101u) << 4);
        }
    }
    __device__ __forceinline__ float term(const int4* a, uint32_t aux, const float* ad, int c) const {
        const int isc = sc0 * dot16_u(lo, a[0]) + sc1 * dot16_u(hi, a[1]);
        const int imn = mn0 * (int)(int16_t)(aux & 0xffffu) + mn1 * (int)(int16_t)(aux >> 16);
        const float da = ad[c >> 3];
        return (d * da) * (float)isc - (dmin * da) * (float)imn;
    }
};

// Q6_K (split rows: 208 payload bytes per block — ql[128], qh[64], sixteen i8 scales — then the f16 d plane).
// Chunk c of a block: 16 ql bytes whose low nibbles are 16 weights of 32-element section h32 and whose high nibbles
// are the same positions of section h32 + 2; each 16-weight run has its own scale (q6_k.zig:1239-1259, dot :1274-1330).
template <>
struct Chunk<FQ_Q6_K> {
    uint4 q, qh, scales;
    uint32_t lo[4], hi[4];
    int sc0, sc1;
    float d;
    __device__ __forceinline__ void load(const uint8_t* row, int c, int k, size_t) {
        const int cc = c & 7, c2 = cc >> 2, h32 = (cc >> 1) & 1, l0 = (cc & 1) * 16;
        const uint8_t* b = row + (size_t)(c >> 3) * 208;
        q = ld_weight16(b + c2 * 64 + h32 * 32 + l0);
        qh = ldg_cached16(b + 128 + c2 * 32 + l0);  // shared by the chunks of both sections
        scales = ldg_cached16(b + 192);
        d = h2f(ld_scale16(row + (size_t)(k >> 8) * 208 + (c >> 3) * 2));
    }
    __device__ __forceinline__ void decode(int c) {
        const int cc = c & 7, c2 = cc >> 2, h32 = (cc >> 1) & 1, half = cc & 1;
        const uint32_t sw = c2 ? scales.z : scales.x, sw2 = c2 ? scales.w : scales.y;  // scales [c2*8 .. +3] and [c2*8+4 .. +7]
        sc0 = (int)(int8_t)(sw >> (8 * (h32 * 2 + half)));
        sc1 = (int)(int8_t)(sw2 >> (8 * (h32 * 2 + half)));
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        const uint32_t hb[4] = {qh.x, qh.y, qh.z, qh.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t l6 = (w[j] & 0x0f0f0f0fu) | (((hb[j] >> (2 * h32)) & 0x03030303u) << 4);
            const uint32_t h6 = ((w[j] >> 4) & 0x0f0f0f0fu) | (((hb[j] >> (2 * h32 + 4)) & 0x03030303u) << 4);
            lo[j] = __vsub4(l6, 0x20202020u);  // 0..63 -> -32..31 per byte
            hi[j] = __vsub4(h6, 0x20202020u);
        }
    }
    __device__ __forceinline__ float term(const int4* a, uint32_t, const float* ad, int c) const {
        const int isum = sc0 * dot16_u(lo, a[0]) + sc1 * dot16_u(hi, a[1]);  // dp4a on signed bytes
        return (float)isum * (d * ad[c >> 3]);
    }
};

template <>
struct Chunk<FQ_TQ2_0> {
    uint4 q;
    float d;
    __device__ __forceinline__ void load(const uint8_t* row, int c, int k, size_t) {
        q = ld_weight16(row + (size_t)c * 16);
        d = h2f(ld_scale16(row + (k >> 2) + (c >> 2) * 2));
    }
    __device__ __forceinline__ void decode(int) {}
    __device__ __forceinline__ float term(const int4* a, uint32_t aux, const float* ad, int c) const {
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        int dot = 0;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            uint32_t x[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) x[j] = (w[j] >> (2 * n)) & 0x03030303u;
            dot += dot16_u(x, a[n]);
        }
        return (d * ad[c >> 2]) * (float)(dot - (int)aux);
    }
};

template <>
struct Chunk<FQ_TQ2_0_FOLDED> {
    uint4 q;
    float d;
    __device__ __forceinline__ void load(const uint8_t* row, int c, int k, size_t) {
        q = ld_weight16(row + (size_t)c * 16);
        d = h2f(ld_scale16(row + (k >> 1) + (c >> 3) * 2));
    }
    __device__ __forceinline__ void decode(int) {}
    __device__ __forceinline__ float term(const int4* a, uint32_t aux, const float* ad, int c) const {
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        uint32_t lo[4], hi[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            lo[j] = w[j] & 0x0f0f0f0fu;
            hi[j] = (w[j] >> 4) & 0x0f0f0f0fu;
        }
        const int dot = dot16_u(lo, a[0]) + dot16_u(hi, a[1]);
        return (d * ad[c >> 3]) * (float)(dot - (int)aux);
    }
};

template <>
struct Chunk<FQ_Q2_0> {
    uint4 q;
    float d;
    __device__ __forceinline__ void load(const uint8_t* row, int c, int k, size_t) {
        q = ld_weight16(row + (size_t)c * 16);
        d = h2f(ld_scale16(row + (k >> 2) + (c >> 1) * 2));
    }
    __device__ __forceinline__ void decode(int) {}
    __device__ __forceinline__ float term(const int4* a, uint32_t aux, const float* ad, int c) const {
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        int i0 = 0, i1 = 0;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            i0 = __dp4a((int)((w[0] >> (2 * n)) & 0x03030303u), a[n].x, i0);
            i0 = __dp4a((int)((w[1] >> (2 * n)) & 0x03030303u), a[n].y, i0);
            i1 = __dp4a((int)((w[2] >> (2 * n)) & 0x03030303u), a[n].z, i1);
            i1 = __dp4a((int)((w[3] >> (2 * n)) & 0x03030303u), a[n].w, i1);
        }
        i0 -= (int)(int16_t)(aux & 0xffffu);
        i1 -= (int)(int16_t)(aux >> 16);
        return d * ad[2 * c] * (float)i0 + d * ad[2 * c + 1] * (float)i1;
    }
};

// MODE 0: dense (one matrix, MB >= m rows, padded rows are zero); 1: grouped table (MoE), a group
// multiplies only its own m <= MB rows; 2: grouped with the fused gate/up pair.
template <int FMT, int MB, int LPR, int MODE>
__global__ void __launch_bounds__(kThreads) gemv_kernel(const GemvArgs A) {
    constexpr bool GATED = MODE == 2, GUARD = MODE >= 1;
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int R = 2;  // weight rows per lane group (gated: the gate row and the up row)
    constexpr ActLayout L = {FMT == FQ_Q8_0 ? 16 : (FMT == FQ_TQ2_0 || FMT == FQ_Q2_0) ? 64 : 32,
                             FMT == FQ_Q8_0 ? 1 : (FMT == FQ_TQ2_0 || FMT == FQ_Q2_0) ? 4 : 2,
                             (FMT == FQ_Q8_0 || FMT == FQ_Q2_0) ? 32 : 256};
    const int k = A.w.k, n = A.w.n;
    const ActSizes S = act_sizes(FMT, k);
    const int C = k / L.chunk_elems;

    // grouped forms: blockIdx.y strides over the table entries (a table may be longer than the grid's y limit)
    for (int entry = blockIdx.y;; entry += gridDim.y) {
    int mat = A.mat, m = A.m;
    const uint8_t* acts = A.acts;
    float* cbase = A.c;
    if (A.table != nullptr) {
        if (entry >= min(*A.n_desc, A.max_desc)) return;
        const GroupDesc d = A.table[entry];
        mat = d.mat;
        m = d.m;
        acts += (size_t)d.row0 * S.row;
        cbase += (size_t)d.row0 * A.ldc;
        if (entry != (int)blockIdx.y) __syncthreads();  // every thread is done with the previous entry's staged rows
    }

    // stage the m activation rows; the dense form zeroes the padded batch slots (they are multiplied), the
    // grouped forms never read them
    {
        const int units = m * (int)(S.row / 16), all = (GUARD ? m : MB) * (int)(S.row / 16);
        const uint4* src = reinterpret_cast<const uint4*>(acts);
        uint4* dst = reinterpret_cast<uint4*>(smem);
        for (int i = threadIdx.x; i < all; i += kThreads) dst[i] = i < units ? __ldg(src + i) : make_uint4(0, 0, 0, 0);
    }
    __syncthreads();

    constexpr int GPW = 32 / LPR;  // row groups per warp
    constexpr int RSTEP = GATED ? 1 : R;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gl = lane % LPR;
    const unsigned gmask = (LPR == 32) ? 0xffffffffu : (((1u << (LPR & 31)) - 1u) << (lane / LPR * LPR));
    const int group = (blockIdx.x * kWarps + warp) * GPW + lane / LPR;
    const int n_groups = gridDim.x * kWarps * GPW;
    const uint8_t* wbase = A.w.base + (size_t)mat * A.w.mat_stride;
    const uint8_t* wbase2 = GATED ? A.w2.base + (size_t)mat * A.w2.mat_stride : nullptr;
    constexpr int ub = FMT == FQ_Q4_K ? 144 : FMT == FQ_Q5_K ? 176 : 16;  // unit bytes (only K-quants can be tile-major)
    const size_t ustride = unit_stride(A.w, ub);

    for (int row0 = group * RSTEP; row0 < n; row0 += n_groups * RSTEP) {
        float acc[R][MB];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int b = 0; b < MB; ++b) acc[r][b] = 0.0f;
        const uint8_t* wr[R];
        if (GATED) {
            wr[0] = row_unit0(A.w, wbase, row0, ub);
            wr[1] = row_unit0(A.w2, wbase2, row0, ub);
        } else {
#pragma unroll
            for (int r = 0; r < R; ++r) wr[r] = row_unit0(A.w, wbase, min(row0 + r, n - 1), ub);
        }

#pragma unroll 2
        for (int c = gl; c < C; c += LPR) {
            Chunk<FMT> ch[R];
#pragma unroll
            for (int r = 0; r < R; ++r) ch[r].load(wr[r], c, k, ustride);
#pragma unroll
            for (int r = 0; r < R; ++r) ch[r].decode(c);
#pragma unroll
            for (int b = 0; b < MB; ++b) {
                if (!GUARD || b < m) {  // CTA-uniform: a short group (few tokens on this expert) pays for its own rows only
                    const uint8_t* rec = smem + (size_t)b * S.row;
                    int4 a[L.segs];
#pragma unroll
                    for (int s = 0; s < L.segs; ++s) a[s] = *reinterpret_cast<const int4*>(rec + ((size_t)s * C + c) * 16);
                    const uint32_t aux = *reinterpret_cast<const uint32_t*>(rec + S.aq + (size_t)c * 4);
                    const float* ad = reinterpret_cast<const float*>(rec + S.aq + S.aaux);
#pragma unroll
                    for (int r = 0; r < R; ++r) acc[r][b] += ch[r].term(a, aux, ad, c);
                }
            }
        }

#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int b = 0; b < MB; ++b) {
                if (!GUARD || b < m) {
                    float v = acc[r][b];
#pragma unroll
                    for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(gmask, v, o);
                    acc[r][b] = v;
                }
            }
        if (gl == 0) {
            if (GATED) {
#pragma unroll
                for (int b = 0; b < MB; ++b) {
                    if (b >= m) continue;
                    cbase[(size_t)b * A.ldc + row0] = gated_pair(A.gated_op, acc[0][b], acc[1][b]);
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    if (row0 + r >= n) continue;
#pragma unroll
                    for (int b = 0; b < MB; ++b) {
                        if (b >= m) continue;
                        float* out = cbase + (size_t)b * A.ldc + row0 + r;
                        *out = A.accumulate ? (*out + acc[r][b]) : acc[r][b];
                    }
                }
            }
        }
    }
    if (A.table == nullptr) return;
    }
}

template <int FMT, int MB, int LPR, int MODE>
cudaError_t launch_one(const GemvArgs& a, int sm_count, cudaStream_t st) {
    constexpr bool GATED = MODE == 2;
    const ActSizes S = act_sizes(FMT, a.w.k);
    const size_t smem = (size_t)MB * S.row;
    auto kern = gemv_kernel<FMT, MB, LPR, MODE>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    const int rows_per_group = GATED ? 1 : 2;
    const int groups_per_cta = kWarps * (32 / LPR);
    const long long groups = ((long long)a.w.n + rows_per_group - 1) / rows_per_group;
    long long ctas = (groups + groups_per_cta - 1) / groups_per_cta;
    long long ny = a.table ? (a.max_desc > 0 ? a.max_desc : 1) : 1;
    if (ny > g_gemv_grid_y_limit) ny = g_gemv_grid_y_limit;  // the kernel strides over longer tables
    // grouped launches spread the SM budget over the table entries: about eight CTAs per SM in total, so a
    // CTA stages its group's activations once and then walks many weight rows
    long long cap = (long long)sm_count * 8 / ny;
    if (cap < 1) cap = 1;
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    kern<<<dim3((unsigned)ctas, (unsigned)ny), kThreads, smem, st>>>(a);
    return cudaGetLastError();
}

template <int FMT, int MB>
cudaError_t launch_lpr(const GemvArgs& a, int sm_count, cudaStream_t st) {
    const ActLayout L = act_layout(FMT);
    const int C = a.w.k / L.chunk_elems;
    // lanes per row group: the choice wasting the fewest lane slots, ties to the wider
    int best = 32, best_cost = ((C + 31) / 32) * 32;
    for (int lpr : {16, 8}) {
        const int cost = ((C + lpr - 1) / lpr) * lpr;
        if (cost < best_cost) best = lpr, best_cost = cost;
    }
    const int mode = a.w2.base != nullptr ? 2 : a.table != nullptr ? 1 : 0;
#define FQ_LAUNCH_LPR(L)                                                    \
    (mode == 2 ? launch_one<FMT, MB, L, 2>(a, sm_count, st)                  \
               : mode == 1 ? launch_one<FMT, MB, L, 1>(a, sm_count, st) : launch_one<FMT, MB, L, 0>(a, sm_count, st))
    switch (best) {
        case 32: return FQ_LAUNCH_LPR(32);
        case 16: return FQ_LAUNCH_LPR(16);
        default: return FQ_LAUNCH_LPR(8);
    }
#undef FQ_LAUNCH_LPR
}

template <int FMT>
cudaError_t launch_mb(const GemvArgs& a, int sm_count, cudaStream_t st) {
    if (a.m <= 1) return launch_lpr<FMT, 1>(a, sm_count, st);
    if (a.m <= 2) return launch_lpr<FMT, 2>(a, sm_count, st);
    if (a.m <= 4) return launch_lpr<FMT, 4>(a, sm_count, st);
    if (a.m <= 8) return launch_lpr<FMT, 8>(a, sm_count, st);
    return launch_lpr<FMT, 16>(a, sm_count, st);
}

}  // namespace

size_t gemv_max_rows() { return 16; }
void set_gemv_grid_y_limit(int limit) { g_gemv_grid_y_limit = limit < 1 ? 65535 : (limit > 65535 ? 65535 : limit); }

// The kernel stages its (padded) activation rows in dynamic shared memory: pad(m) * act_sizes(fmt, k).row
// bytes must fit the 227 KiB a CTA may opt in to.
constexpr size_t kGemvSmemLimit = 227 * 1024;
int gemv_padded_rows(size_t m) { return m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : m <= 8 ? 8 : 16; }
int gemv_rows_that_fit(int fmt, size_t k) {
    const ActSizes S = act_sizes(fmt, k);
    if (S.row == 0) return 0;
    for (int mb = 16; mb >= 1; mb >>= 1)
        if ((size_t)mb * S.row <= kGemvSmemLimit) return mb;
    return 0;
}

cudaError_t launch_gemv(const GemvArgs& a, int sm_count, cudaStream_t st) {
    if (a.m < 1 || a.m > 16) return cudaErrorInvalidValue;
    if (gemv_padded_rows((size_t)a.m) > gemv_rows_that_fit(a.w.fmt, (size_t)a.w.k)) return cudaErrorInvalidValue;  // callers split or decline first
    switch (a.w.fmt) {
        case FQ_Q8_0: return launch_mb<FQ_Q8_0>(a, sm_count, st);
        case FQ_Q4_K: return launch_mb<FQ_Q4_K>(a, sm_count, st);
        case FQ_Q5_K: return launch_mb<FQ_Q5_K>(a, sm_count, st);
        case FQ_Q6_K: return launch_mb<FQ_Q6_K>(a, sm_count, st);
        case FQ_TQ2_0: return launch_mb<FQ_TQ2_0>(a, sm_count, st);
        case FQ_TQ2_0_FOLDED: return launch_mb<FQ_TQ2_0_FOLDED>(a, sm_count, st);
        case FQ_Q2_0: return launch_mb<FQ_Q2_0>(a, sm_count, st);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace fq
