// Row-per-lane decode GEMV for sm_100a with TMA-staged weight streaming.
//
// c[b, j] = sum_e a[b, e] * dequant(W)[j, e], b < m <= 16, for the dense decode
// shapes (K >= 2048; Q4_K / Q5_K up to 16 rows, Q8_0 up to 8, TQ2_0 planes up
// to 4). Same arithmetic as the reference's CPU kernels: int8 activations,
// exact integer block dots, and per block the f32 epilogue of
// q4_k.zig:895-913 / q5_k.zig:1093-1111 / q8_0.zig:1074-1089 /
// ternary.zig:377-386, evaluated without fusing; only the order in which block
// terms are added differs.
//
// Data movement. One persistent CTA per SM owns a contiguous range of weight
// rows and walks it in tiles of 32 rows; lane l of every warp owns row l of
// the tile, so no cross-lane reduction is needed and the block header is
// decoded once per 256 weights. The warps (16, or 8 for wider batches) split
// K: warp w takes the slabs (1-2 blocks per row) w, w+W, ... . A warp step
// brings one slab of 32 rows into a ring of shared-memory stages and
// completes on one mbarrier, by the cheapest copy the layout allows:
//   tile-major K-quants   one bulk copy of the contiguous 32 x 144/176 bytes
//   row-major K-quants    one 2-D tensor copy (32 rows x one unit)
//   split rows (Q8_0)     three tensor copies: two 32 x 128-byte payload boxes (128-byte swizzle) and
//                         the 32 x 16 scale bytes (per-lane bulk copies when no tensor map can be made)
//   split rows (TQ2_0)    one tensor copy: a 32 x 128-byte payload box (512 weights per row, 128-byte
//                         swizzle); the two f16 scales of a lane's row come straight from global memory
// Slots are an odd number of 16-byte units wide so the 128-bit shared loads
// of a quarter warp hit 32 distinct banks. Copies for the next slabs (also of
// the next tile) are in flight while a slab is consumed, which keeps ~144 KB
// per SM outstanding independent of register count -- the thing an HBM-bound
// kernel needs. The kernel launches with programmatic stream serialisation:
// its weight copies start before griddepcontrol.wait, so they overlap the
// tail of the previous kernel. Activations are quantised per CTA after that
// wait, while the first weight slabs are in flight, and are read as warp-wide
// broadcasts.
//
// Every wait on an mbarrier is bounded; a wait that gives up records
// FQ_ERR_TIMEOUT in the status word and the CTA returns.
#include <cuda.h>

#include <cstdlib>
#include <cstring>

#include "actquant.cuh"
#include "internal.h"

namespace fq {

namespace {

constexpr int kMaxStages = 4;
constexpr unsigned kWaitLimit = 1u << 20;

// Diagnostic build only (-DFQ_TIMELINE): thread 0 of every CTA stamps the phases of the last launch
// into shared memory (a global store here would sit in front of the barrier-init fence and distort
// what it measures) and copies them out when the CTA is done.
#ifdef FQ_TIMELINE
constexpr int kTimelineSlots = 16;
__device__ unsigned long long g_timeline[1024 * kTimelineSlots];
__shared__ unsigned long long s_timeline[kTimelineSlots];
__device__ __forceinline__ void stamp(int slot) {
    if (threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");
        s_timeline[slot] = t;
    }
}
__device__ __forceinline__ void stamp_flush() {
    if (threadIdx.x == 0 && blockIdx.x < 1024)
        for (int i = 0; i < kTimelineSlots; ++i) g_timeline[blockIdx.x * kTimelineSlots + i] = s_timeline[i];
}
#else
__device__ __forceinline__ void stamp(int) {}
__device__ __forceinline__ void stamp_flush() {}
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the barrier did not complete within the limit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (unsigned i = 0; i < kWaitLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// Bulk async copy global -> this CTA's shared memory; bytes and both
// addresses are multiples of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}
// The same copy marked evict-first in L2: decode weights are read once per token, so they should
// not push the activations and outputs of the surrounding kernels out of the cache.
__device__ __forceinline__ uint64_t evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_load_stream(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t pol) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar), "l"(pol)
                 : "memory");
}

// Shared-memory addresses are carried as 32-bit shared-window offsets; loads go through typed
// pointers so constant offsets fold into the instruction and the scheduler may batch them. The
// mbarrier wait's memory clobber keeps every load behind the wait that guards its stage.
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    return *reinterpret_cast<const uint4*>(__cvta_shared_to_generic(addr));
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
    return *reinterpret_cast<const float*>(__cvta_shared_to_generic(addr));
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) { return __dp4a((int)a, (int)b, c); }
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// two independent chains per 16 bytes: dp4a results are needed soon and the chain latency shows
__device__ __forceinline__ int dot16_ss(const uint32_t* w, const uint4& a, int acc) {
    const int x = dp4a_ss(w[1], a.y, dp4a_ss(w[0], a.x, acc));
    const int y = dp4a_ss(w[3], a.w, dp4a_ss(w[2], a.z, 0));
    return x + y;
}
__device__ __forceinline__ int dot16_us(const uint32_t* w, const uint4& a, int acc) {
    const int x = dp4a_us(w[1], a.y, dp4a_us(w[0], a.x, acc));
    const int y = dp4a_us(w[3], a.w, dp4a_us(w[2], a.z, 0));
    return x + y;
}
__device__ __forceinline__ int byte_of(uint32_t w, int i) { return (int)((w >> (8 * i)) & 0xffu); }

// K-quant header: d, dmin and the eight 6-bit (scale, min) pairs as bytes
// (reference backend/quant/q8k.zig:637-648, four pairs per word at a time).
struct KHeader {
    float d, dmin;
    uint32_t sc[2], mn[2];
    __device__ __forceinline__ void decode(const uint4& h) {
        const __half2 dm = *reinterpret_cast<const __half2*>(&h.x);
        d = __low2float(dm);
        dmin = __high2float(dm);
        sc[0] = h.y & 0x3f3f3f3fu;
        mn[0] = h.z & 0x3f3f3f3fu;
        sc[1] = (h.w & 0x0f0f0f0fu) | (((h.y >> 6) & 0x03030303u) << 4);
        mn[1] = ((h.w >> 4) & 0x0f0f0f0fu) | (((h.z >> 6) & 0x03030303u) << 4);
    }
};

// Per block epilogue shared by Q4_K and Q5_K, kept unfused like the CPU code.
__device__ __forceinline__ float kquant_term(const KHeader& H, float da, int isc, int imn) {
    return __fsub_rn(__fmul_rn(__fmul_rn(H.d, da), (float)isc), __fmul_rn(__fmul_rn(H.dmin, da), (float)imn));
}

__device__ __forceinline__ int min_term(const KHeader& H, uint32_t sums_addr) {
    const uint4 s0 = lds128(sums_addr), s1 = lds128(sums_addr + 16);
    int imn = byte_of(H.mn[0], 0) * (int)s0.x;
    imn += byte_of(H.mn[0], 1) * (int)s0.y;
    imn += byte_of(H.mn[0], 2) * (int)s0.z;
    imn += byte_of(H.mn[0], 3) * (int)s0.w;
    imn += byte_of(H.mn[1], 0) * (int)s1.x;
    imn += byte_of(H.mn[1], 1) * (int)s1.y;
    imn += byte_of(H.mn[1], 2) * (int)s1.z;
    imn += byte_of(H.mn[1], 3) * (int)s1.w;
    return imn;
}

// Shared-memory view of the MB activation records of this CTA.
struct ActView {
    uint32_t base;      // shared address of record 0
    uint32_t row;       // bytes per record
    uint32_t off_sums;  // Q8_K: int32 sub-block sums
    uint32_t off_ad;    // f32 scales
};

// ---- one 256-weight Q4_K block of this lane's row against MB activation rows
template <int MB>
__device__ __forceinline__ void block_q4_k(uint32_t p, const ActView& V, int kb, float (&acc)[MB]) {
    KHeader H;
    H.decode(lds128(p));
    int isc_lo[MB], isc_hi[MB];
#pragma unroll
    for (int b = 0; b < MB; ++b) isc_lo[b] = isc_hi[b] = 0;
#pragma unroll
    for (int pp = 0; pp < 4; ++pp) {
        const uint4 q0 = lds128(p + 16 + pp * 32), q1 = lds128(p + 32 + pp * 32);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        uint32_t lo[8], hi[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            lo[j] = w[j] & 0x0f0f0f0fu;
            hi[j] = w[j] & 0xf0f0f0f0u;  // 16 * nibble as an unsigned byte; the factor is shifted out below
        }
        const int sa = byte_of(H.sc[pp >> 1], (pp & 1) * 2), sb = byte_of(H.sc[pp >> 1], (pp & 1) * 2 + 1);
#pragma unroll
        for (int b = 0; b < MB; ++b) {
            const uint32_t a = V.base + b * V.row + kb * 256 + pp * 64;
            const uint4 a0 = lds128(a), a1 = lds128(a + 16), a2 = lds128(a + 32), a3 = lds128(a + 48);
            int dlo = dot16_ss(lo, a0, 0);
            dlo = dot16_ss(lo + 4, a1, dlo);
            int dhi = dot16_us(hi, a2, 0);
            dhi = dot16_us(hi + 4, a3, dhi);
            isc_lo[b] += sa * dlo;
            isc_hi[b] += sb * dhi;
        }
    }
#pragma unroll
    for (int b = 0; b < MB; ++b) {
        const uint32_t rec = V.base + b * V.row;
        const int imn = min_term(H, rec + V.off_sums + kb * 32);
        const float da = lds_f32(rec + V.off_ad + kb * 4);
        acc[b] = __fadd_rn(acc[b], kquant_term(H, da, isc_lo[b] + (isc_hi[b] >> 4), imn));
    }
}

// ---- Q5_K: as Q4_K plus the fifth bits (bit s of qh[i] belongs to sub-block s)
template <int MB>
__device__ __forceinline__ void block_q5_k(uint32_t p, const ActView& V, int kb, float (&acc)[MB]) {
    KHeader H;
    H.decode(lds128(p));
    const uint4 h0 = lds128(p + 16), h1 = lds128(p + 32);
    const uint32_t hb[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
    int isc[MB];
#pragma unroll
    for (int b = 0; b < MB; ++b) isc[b] = 0;
#pragma unroll
    for (int pp = 0; pp < 4; ++pp) {
        const uint4 q0 = lds128(p + 48 + pp * 32), q1 = lds128(p + 64 + pp * 32);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        uint32_t lo[8], hi[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            lo[j] = (w[j] & 0x0f0f0f0fu) | (((hb[j] >> (2 * pp)) & 0x01010101u) << 4);
            hi[j] = ((w[j] >> 4) & 0x0f0f0f0fu) | (((hb[j] >> (2 * pp + 1)) & 0x01010101u) << 4);
        }
        const int sa = byte_of(H.sc[pp >> 1], (pp & 1) * 2), sb = byte_of(H.sc[pp >> 1], (pp & 1) * 2 + 1);
#pragma unroll
        for (int b = 0; b < MB; ++b) {
            const uint32_t a = V.base + b * V.row + kb * 256 + pp * 64;
            const uint4 a0 = lds128(a), a1 = lds128(a + 16), a2 = lds128(a + 32), a3 = lds128(a + 48);
            int dlo = dot16_ss(lo, a0, 0);
            dlo = dot16_ss(lo + 4, a1, dlo);
            int dhi = dot16_ss(hi, a2, 0);
            dhi = dot16_ss(hi + 4, a3, dhi);
            isc[b] += sa * dlo + sb * dhi;
        }
    }
#pragma unroll
    for (int b = 0; b < MB; ++b) {
        const uint32_t rec = V.base + b * V.row;
        const int imn = min_term(H, rec + V.off_sums + kb * 32);
        const float da = lds_f32(rec + V.off_ad + kb * 4);
        acc[b] = __fadd_rn(acc[b], kquant_term(H, da, isc[b], imn));
    }
}

// ---- Q6_K: the 208 payload bytes of this lane's row at p (ql[128] | qh[64] | scales[16]); the block's f16 scale
// travels in a plane of its own and arrives as `dw`. Element 128 c + 32 s + l takes its low four bits from
// ql[64 c + 32 (s & 1) + l] (low nibble for sections 0-1, high for 2-3) and two more from bits 2s, 2s+1 of qh[32 c + l];
// levels carry an offset of 32 and every 16 elements have a signed scale (q6_k.zig:1239-1259). The integer total and
// the epilogue f32(total) * (d_w * d_a) are those of dotQ6_KQ8_K (q6_k.zig:617-631).
template <int MB>
__device__ __forceinline__ void block_q6_k(uint32_t p, float dw, const ActView& V, int kb, float (&acc)[MB]) {
    const uint4 scv = lds128(p + 192);
    const uint32_t scw[4] = {scv.x, scv.y, scv.z, scv.w};
    // sum over the 16 groups of scale * (dot of the unsigned levels 0..63) - 32 * scale * (sum of the group's activations):
    // the second part needs the record's sixteen int16 group sums and no re-centring of the levels
    int isum[MB];
#pragma unroll
    for (int b = 0; b < MB; ++b) {
        const uint32_t sums = V.base + b * V.row + V.off_sums + kb * 32;
        const uint4 s0 = lds128(sums), s1 = lds128(sums + 16);
        const uint32_t sw[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};  // groups 2j | 2j + 1 as int16 pairs
        int corr = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            // scales 2j and 2j + 1 are bytes (2j) & 3 and (2j + 1) & 3 of word j / 2
            const uint32_t two = scw[j >> 1] >> ((j & 1) * 16);
            corr = __dp2a_lo((int)sw[j], (int)two, corr);  // int16 x int8 pairs
        }
        isum[b] = -32 * corr;
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const uint4 la = lds128(p + 64 * c), lb = lds128(p + 64 * c + 16), lc = lds128(p + 64 * c + 32), ld = lds128(p + 64 * c + 48);
        const uint4 ha = lds128(p + 128 + 32 * c), hb = lds128(p + 128 + 32 * c + 16);
        const uint32_t wl0[8] = {la.x, la.y, la.z, la.w, lb.x, lb.y, lb.z, lb.w};
        const uint32_t wl1[8] = {lc.x, lc.y, lc.z, lc.w, ld.x, ld.y, ld.z, ld.w};
        const uint32_t wh[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
        uint32_t q[4][8];  // [section][word of four consecutive l]: levels 0..63
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            q[0][g] = (wl0[g] & 0x0f0f0f0fu) | ((wh[g] << 4) & 0x30303030u);
            q[1][g] = (wl1[g] & 0x0f0f0f0fu) | ((wh[g] << 2) & 0x30303030u);
            q[2][g] = ((wl0[g] >> 4) & 0x0f0f0f0fu) | (wh[g] & 0x30303030u);
            q[3][g] = ((wl1[g] >> 4) & 0x0f0f0f0fu) | ((wh[g] >> 2) & 0x30303030u);
        }
#pragma unroll
        for (int b = 0; b < MB; ++b) {
            const uint32_t a = V.base + b * V.row + kb * 256 + c * 128;
#pragma unroll
            for (int sec = 0; sec < 4; ++sec)
#pragma unroll
                for (int is = 0; is < 2; ++is) {
                    // scale of elements 128 c + 32 sec + 16 is ..: index 8 c + 2 sec + is
                    const int sc = (int)(int8_t)(scw[2 * c + (sec >> 1)] >> (8 * ((sec & 1) * 2 + is)));
                    isum[b] += sc * dot16_us(&q[sec][4 * is], lds128(a + 32 * sec + 16 * is), 0);
                }
        }
    }
#pragma unroll
    for (int b = 0; b < MB; ++b) {
        const float da = lds_f32(V.base + b * V.row + V.off_ad + kb * 4);
        acc[b] = __fadd_rn(acc[b], __fmul_rn((float)isum[b], __fmul_rn(dw, da)));
    }
}

// ---- Q8_0: one unit = 8 blocks of 32 weights; payload at p, the unit's eight
// f16 scales at ps. Per block f32(idot) * (d_a * d_w)  (q8_0.zig:1074-1089).
template <int MB>
__device__ __forceinline__ void unit_q8_0(uint32_t p, uint32_t ps, const ActView& V, int kb, float (&acc)[MB]) {
    const uint4 su = lds128(ps);
    const uint32_t sw[4] = {su.x, su.y, su.z, su.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint4 w0 = lds128(p + j * 32), w1 = lds128(p + j * 32 + 16);
        const uint32_t w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        const float dw = __half2float(__ushort_as_half((unsigned short)((sw[j >> 1] >> ((j & 1) * 16)) & 0xffffu)));
#pragma unroll
        for (int b = 0; b < MB; ++b) {
            const uint32_t rec = V.base + b * V.row;
            const uint32_t a = rec + kb * 256 + j * 32;
            const uint4 a0 = lds128(a), a1 = lds128(a + 16);
            int dot = dot16_ss(w, a0, 0);
            dot = dot16_ss(w + 4, a1, dot);
            const float da = lds_f32(rec + V.off_ad + (kb * 8 + j) * 4);
            acc[b] = __fadd_rn(acc[b], __fmul_rn((float)dot, __fmul_rn(da, dw)));
        }
    }
}

// ---- eight activation rows at a time: the block dots go through the warp-level int8 tensor-core
// instruction (mma.sync m16n8k32, u8 levels x s8 activations -> s32, exact), 16 weight rows x 8 tokens x 32
// weights at a time, instead of eight rounds of dp4a per row. The lane <-> (row, token) ownership is the
// instruction's fragment layout, with g = lane / 4 and t = lane % 4:
//   A (weights)      words of rows g and g + 8, elements 4t..4t+3 and 16+4t..16+4t+3 of the sub-block
//   B (activations)  token g, the same element columns
//   D (dots)         rows g and g + 8, tokens 2t and 2t + 1
// A 32-row tile is two such row groups; acc[4 * group + {0,1}] belongs to row 16*group + g, tokens 2t and
// 2t + 1, acc[4 * group + {2,3}] to row 16*group + 8 + g. Sub-block scales multiply the integer dots, the
// min term and the f32 epilogue are those of block_q4_k / block_q5_k, so values are identical to them.
__device__ __forceinline__ void mma_u8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) { return *reinterpret_cast<const uint32_t*>(__cvta_shared_to_generic(addr)); }

template <int FMT>
__device__ __forceinline__ void expert_block_mma(uint32_t tile_base, const ActView& V, int kb, int lane, float (&acc)[8]) {
    constexpr int UB = FMT == FQ_Q4_K ? 144 : 176;
    constexpr int QS = FMT == FQ_Q4_K ? 16 : 48;  // offset of the nibble payload inside a block
    const int g = lane >> 2, t = lane & 3;
    // headers of this lane's four rows: g, g + 8, g + 16, g + 24
    KHeader H[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) H[i].decode(lds128(tile_base + (uint32_t)(g + 8 * i) * UB));
    int isc[4][2], imn[4][2];
#pragma unroll
    for (int i = 0; i < 4; ++i) isc[i][0] = isc[i][1] = imn[i][0] = imn[i][1] = 0;
    uint32_t qh[4][2];  // Q5_K: fifth bits of elements 4t..4t+3 and 16+4t.. of the four rows, all eight sub-blocks
    if (FMT == FQ_Q5_K) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            qh[i][0] = lds32(tile_base + (uint32_t)(g + 8 * i) * UB + 16 + 4 * t);
            qh[i][1] = lds32(tile_base + (uint32_t)(g + 8 * i) * UB + 32 + 4 * t);
        }
    }
    const uint32_t arow = V.base + (uint32_t)g * V.row + (uint32_t)kb * 256 + 4 * t;  // token g, this lane's columns
#pragma unroll
    for (int pp = 0; pp < 4; ++pp) {
        // activations of sub-blocks 2pp (low nibbles) and 2pp + 1 (high nibbles)
        const uint32_t b_lo0 = lds32(arow + pp * 64), b_lo1 = lds32(arow + pp * 64 + 16);
        const uint32_t b_hi0 = lds32(arow + pp * 64 + 32), b_hi1 = lds32(arow + pp * 64 + 48);
#pragma unroll
        for (int grp = 0; grp < 2; ++grp) {
            const int ia = 2 * grp, ib = 2 * grp + 1;  // rows 16*grp + g and 16*grp + 8 + g
            const uint32_t pa = tile_base + (uint32_t)(g + 16 * grp) * UB + QS + pp * 32 + 4 * t;
            const uint32_t pb = pa + 8 * UB;
            const uint32_t w[4] = {lds32(pa), lds32(pb), lds32(pa + 16), lds32(pb + 16)};
            uint32_t lo[4], hi[4];
            int dlo[4], dhi[4];
            if (FMT == FQ_Q5_K) {
                const uint32_t h[4] = {qh[ia][0], qh[ib][0], qh[ia][1], qh[ib][1]};
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    lo[x] = (w[x] & 0x0f0f0f0fu) | (((h[x] >> (2 * pp)) & 0x01010101u) << 4);
                    hi[x] = ((w[x] >> 4) & 0x0f0f0f0fu) | (((h[x] >> (2 * pp + 1)) & 0x01010101u) << 4);
                }
                mma_u8s8(dlo, lo, b_lo0, b_lo1);
                mma_u8s8(dhi, hi, b_hi0, b_hi1);
            } else {
                // Q4_K: the high nibbles stay in place as 16 * level (a u8 below 256); the factor is shifted out of the dots
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    lo[x] = w[x] & 0x0f0f0f0fu;
                    hi[x] = w[x] & 0xf0f0f0f0u;
                }
                mma_u8s8(dlo, lo, b_lo0, b_lo1);
                mma_u8s8(dhi, hi, b_hi0, b_hi1);
#pragma unroll
                for (int x = 0; x < 4; ++x) dhi[x] >>= 4;  // exact: every product carried the factor 16
            }
            const int sa_a = byte_of(H[ia].sc[pp >> 1], (pp & 1) * 2), sb_a = byte_of(H[ia].sc[pp >> 1], (pp & 1) * 2 + 1);
            const int sa_b = byte_of(H[ib].sc[pp >> 1], (pp & 1) * 2), sb_b = byte_of(H[ib].sc[pp >> 1], (pp & 1) * 2 + 1);
            isc[ia][0] += sa_a * dlo[0] + sb_a * dhi[0];
            isc[ia][1] += sa_a * dlo[1] + sb_a * dhi[1];
            isc[ib][0] += sa_b * dlo[2] + sb_b * dhi[2];
            isc[ib][1] += sa_b * dlo[3] + sb_b * dhi[3];
        }
    }
    // min term and f32 epilogue per (row, token), as in block_q4_k. The eight sub-block sums of a token fit
    // int16 (|sum of 32 int8| <= 4064), so sum(mn[s] * bsum[s]) is four 2-way int16 x int8 dot instructions.
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const uint32_t rec = V.base + (uint32_t)(2 * t + c) * V.row;
        const float da = lds_f32(rec + V.off_ad + kb * 4);
        const uint4 s0 = lds128(rec + V.off_sums + kb * 32), s1 = lds128(rec + V.off_sums + kb * 32 + 16);
        const int bs01 = (int)__byte_perm(s0.x, s0.y, 0x5410), bs23 = (int)__byte_perm(s0.z, s0.w, 0x5410);
        const int bs45 = (int)__byte_perm(s1.x, s1.y, 0x5410), bs67 = (int)__byte_perm(s1.z, s1.w, 0x5410);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int mn_term = __dp2a_lo(bs01, (int)H[i].mn[0], 0);
            mn_term = __dp2a_hi(bs23, (int)H[i].mn[0], mn_term);
            mn_term = __dp2a_lo(bs45, (int)H[i].mn[1], mn_term);
            mn_term = __dp2a_hi(bs67, (int)H[i].mn[1], mn_term);
            const int grp = i >> 1, half = i & 1;  // rows g + 8*i = 16*grp + 8*half + g
            float& a = acc[4 * grp + 2 * half + c];
            a = __fadd_rn(a, kquant_term(H[i], da, isc[i][c], mn_term));
        }
    }
}

// The same unit when it was staged by tensor copies (RowsArgs.use_tmap == 2): per warp step the 32 rows x 256
// payload bytes arrive as two boxes of 32 x 128 bytes with the 128-byte swizzle (16-byte chunk c of row r sits
// at chunk c ^ (r % 8), so a quarter warp's 128-bit loads fall on distinct banks although rows are 128 bytes
// apart), followed by the 32 x 16 scale bytes. `base` is the 1024-byte aligned start of the stage.
constexpr int kQ8StageBytes = 9216;  // 2 x 4096 payload + 512 scales, padded to a multiple of 1024
template <int MB>
__device__ __forceinline__ void unit_q8_0_swz(uint32_t base, int lane, const ActView& V, int kb, float (&acc)[MB]) {
    const uint4 su = lds128(base + 8192 + lane * 16);
    const uint32_t sw[4] = {su.x, su.y, su.z, su.w};
    const uint32_t x = (uint32_t)(lane & 7);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t rowp = base + (uint32_t)(j >> 2) * 4096 + (uint32_t)lane * 128;
        const uint32_t c0 = (uint32_t)(j & 3) * 2;
        const uint4 w0 = lds128(rowp + ((c0 ^ x) << 4)), w1 = lds128(rowp + (((c0 + 1) ^ x) << 4));
        const uint32_t w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        const float dw = __half2float(__ushort_as_half((unsigned short)((sw[j >> 1] >> ((j & 1) * 16)) & 0xffffu)));
#pragma unroll
        for (int b = 0; b < MB; ++b) {
            const uint32_t rec = V.base + b * V.row;
            const uint32_t a = rec + kb * 256 + j * 32;
            const uint4 a0 = lds128(a), a1 = lds128(a + 16);
            int dot = dot16_ss(w, a0, 0);
            dot = dot16_ss(w + 4, a1, dot);
            const float da = lds_f32(rec + V.off_ad + (kb * 8 + j) * 4);
            acc[b] = __fadd_rn(acc[b], __fmul_rn((float)dot, __fmul_rn(da, dw)));
        }
    }
}

// ---- TQ2_0 (PTQTP planes): split rows [K/4 payload bytes][K/256 f16 scales]. A pipeline step is 512 weights of 32 rows:
// one box of 32 x 128 payload bytes with the 128-byte swizzle (as above); the two f16 scales of the lane's row come
// straight from global memory (`d2`, four bytes). Byte hg*32 + m of a 64-byte block holds elements hg*128 + n*32 + m in
// crumb n (dtype.zig:215-218), so crumb n of a 16-byte chunk pairs with 16 consecutive activations. The block term is
// (d * a.d) * f32(sum(code * a) - sum(a)) (ternary.zig:377-386).
constexpr int kTqStageBytes = 4096;
template <int MB>
__device__ __forceinline__ void unit_tq2_0_swz(uint32_t base, int lane, const ActView& V, int sl, uint32_t d2, float (&acc)[MB]) {
    const uint32_t x = (uint32_t)(lane & 7);
    const uint32_t rowp = base + (uint32_t)lane * 128;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int kb = sl * 2 + half;
        const float dw = __half2float(__ushort_as_half((unsigned short)((d2 >> (16 * half)) & 0xffffu)));
        // crumb n stays in place (a byte worth code * 4^n, unsigned): one mask per word instead of a shift and a mask;
        // the factor leaves each 16-weight integer sum by an exact shift
        int dot[MB];
#pragma unroll
        for (int b = 0; b < MB; ++b) dot[b] = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {  // chunk j of the block: half-group j / 2, bytes (j % 2) * 16 ..+15
            const uint4 wq = lds128(rowp + ((((uint32_t)(half * 4 + j)) ^ x) << 4));
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                // (the top crumb would make a byte of 128 or more, which the signed instruction cannot take: it is shifted down)
                const int sh = n == 3 ? 6 : 0;
                const uint32_t mask = n == 3 ? 0x03030303u : 0x03030303u << (2 * n);
                const uint32_t w[4] = {(wq.x >> sh) & mask, (wq.y >> sh) & mask, (wq.z >> sh) & mask, (wq.w >> sh) & mask};
#pragma unroll
                for (int b = 0; b < MB; ++b) {
                    const uint4 a = lds128(V.base + b * V.row + kb * 256 + (j >> 1) * 128 + n * 32 + (j & 1) * 16);
                    dot[b] += dot16_ss(w, a, 0) >> (n == 3 ? 0 : 2 * n);
                }
            }
        }
#pragma unroll
        for (int b = 0; b < MB; ++b) {
            const uint32_t rec = V.base + b * V.row;
            const float da = lds_f32(rec + V.off_ad + kb * 4);
            const uint4 s0 = lds128(rec + V.off_sums + kb * 32), s1 = lds128(rec + V.off_sums + kb * 32 + 16);
            const int asum = (int)s0.x + (int)s0.y + (int)s0.z + (int)s0.w + (int)s1.x + (int)s1.y + (int)s1.z + (int)s1.w;
            const int isum = dot[b] - asum;
            acc[b] = __fadd_rn(acc[b], __fmul_rn(__fmul_rn(dw, da), (float)isum));
        }
    }
}

// Geometry of one slab (what a lane fetches per pipeline step).
struct SlabGeom {
    int unit_bytes;    // payload bytes per 256 weights
    int scale_bytes;   // separate scale-plane bytes per 256 weights (0: scales travel inside the payload)
    int slot_bytes;    // shared-memory slot per lane, an odd number of 16-byte units
    int scale_off;     // offset of the scale bytes inside the slot
};
__host__ __device__ inline SlabGeom slab_geom(int fmt, int slab) {
    SlabGeom g;
    g.unit_bytes = fmt == FQ_Q4_K ? 144 : fmt == FQ_Q5_K ? 176 : fmt == FQ_Q6_K ? 208 : 256;
    g.scale_bytes = fmt == FQ_Q8_0 ? 16 : 0;
    g.scale_off = slab * g.unit_bytes;
    int bytes = slab * (g.unit_bytes + g.scale_bytes);
    if (((bytes / 16) & 1) == 0) bytes += 16;
    g.slot_bytes = bytes;
    return g;
}

// where the product of token `tok` and weight row `row` goes: c[tok][row], or, for stacked matrices that share
// the activations, the [matrix][token][row inside the matrix] layout of the shared-input batch
__device__ __forceinline__ size_t out_index(const RowsArgs& A, int tok, int row) {
    if (A.split_n == 0) return (size_t)tok * A.ldc + row;
    const int mat = row / A.split_n;
    return ((size_t)mat * A.m + tok) * A.split_n + (row - mat * A.split_n);
}

template <int FMT, int MB, bool FUSED, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, (WARPS == 8 && MB < 8) ? 2 : 1) decode_rows_kernel(const RowsArgs A, const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap tmap2) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int kWarps = WARPS, kThreads = WARPS * 32;  // the warps split K; 16 when a row has at least 16 units
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int k = A.w.k, n = A.w.n;
    constexpr bool Q8K = FMT != FQ_Q8_0;
    const NatSizes NS = nat_sizes(Q8K, k);
    const SlabGeom G = slab_geom(FMT, A.slab);
    constexpr bool TQ = FMT == FQ_TQ2_0;
    constexpr bool Q6 = FMT == FQ_Q6_K;  // payload units by tensor copy (one-unit slabs); the f16 block scales by plain loads
    const int units = TQ ? (k >> 9) : (k >> 8);              // pipeline units per row: 256 weights (TQ2_0: 512)
    const int nslabs = (units + A.slab - 1) / A.slab;        // slabs per row
    const int my_slabs = warp < nslabs ? (nslabs - warp + kWarps - 1) / kWarps : 0;

    // shared memory: barriers | activation records | reduction buffers | stage slots
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    uint8_t* acts = smem + 512;
    float* red = reinterpret_cast<float*>(acts + ((MB * NS.row + 127) & ~(size_t)127));
    uint8_t* slots = reinterpret_cast<uint8_t*>(red) + 2 * kWarps * MB * 32 * sizeof(float);
    // bytes between the stages of a warp; Q8_0 staged by tensor copies uses whole 1024-byte aligned stages
    const bool q8_boxes = FMT == FQ_Q8_0 && A.use_tmap == 2;
    const uint32_t stage_stride = TQ ? (uint32_t)kTqStageBytes : q8_boxes ? (uint32_t)kQ8StageBytes : (uint32_t)(32 * G.slot_bytes);
    const uint32_t slot0 = (TQ || q8_boxes) ? ((smem_u32(slots) + 1023u) & ~1023u) + (uint32_t)(warp * A.stages) * stage_stride
                                            : smem_u32(slots) + (uint32_t)((warp * A.stages) * 32 + lane) * G.slot_bytes;
    const uint32_t bar0 = smem_u32(bars) + warp * kMaxStages * 8;

    stamp(0);
    if (lane == 0)
        for (int s = 0; s < A.stages; ++s) mbar_init(bar0 + s * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncwarp();
    stamp(7);

    // this CTA's contiguous row range, balanced over the grid
    // (or, for a matrix with no more 32-row tiles than CTAs, exactly one storage tile each: one full-width
    // pipeline step per warp instead of two partial ones)
    int r_begin, r_end;
    if (A.rows_per_cta > 0) {
        r_begin = (int)blockIdx.x * A.rows_per_cta;
        r_end = min(n, r_begin + A.rows_per_cta);
    } else if (A.rows_per_cta < 0) {  // whole 32-row storage tiles, balanced over the grid: no piece straddles a tile
        const long long T = (n + 31) >> 5;
        r_begin = (int)(T * blockIdx.x / gridDim.x) << 5;
        r_end = min(n, (int)(T * (blockIdx.x + 1) / gridDim.x) << 5);
    } else {
        r_begin = (int)((long long)n * blockIdx.x / gridDim.x);
        r_end = (int)((long long)n * (blockIdx.x + 1) / gridDim.x);
    }
    // row tiles of this CTA: 32 rows from r_begin on (row-major), or the pieces of its range inside
    // each 32-row storage tile (tile-major: a piece is contiguous in HBM, a straddle is two pieces)
    const bool tiled = A.w.tile_rows != 0;
    const int first_tile = r_begin >> 5;
    const int ntiles = r_end <= r_begin ? 0 : tiled ? ((r_end - 1) >> 5) - first_tile + 1 : (r_end - r_begin + 31) / 32;
    auto tile_rows = [&](int tile, int& row0, int& nvalid) {
        if (tiled) {
            row0 = max(r_begin, (first_tile + tile) << 5);
            nvalid = min(r_end, (first_tile + tile + 1) << 5) - row0;
        } else {
            row0 = r_begin + tile * 32;
            nvalid = min(32, r_end - row0);
        }
    };
    const int total = ntiles * my_slabs;  // pipeline steps of this warp
    const uint8_t* wbase = A.w.base + (size_t)A.mat * A.w.mat_stride;
    const uint64_t l2_policy = A.l2_stream ? evict_first_policy() : 0;

    auto issue = [&](int it) {
        const int tile = it / my_slabs, sl = warp + kWarps * (it % my_slabs);
        const int stage = it % A.stages;
        int row0, nvalid;
        tile_rows(tile, row0, nvalid);
        const int nu = min(A.slab, units - sl * A.slab);  // units in this (possibly ragged) slab
        const uint32_t bar = bar0 + stage * 8;
        if (tiled) {
            // tile-major weights: unit `sl` of these rows is one contiguous run -> one bulk copy per warp step
            if (lane == 0) {
                const uint32_t bytes = (uint32_t)(nvalid * G.unit_bytes);
                mbar_arrive_expect_tx(bar, bytes);
                const uint8_t* src = wbase + (size_t)(row0 >> 5) * ((size_t)32 * A.w.row_stride) + (size_t)sl * 32 * G.unit_bytes +
                                     (size_t)(row0 & 31) * G.unit_bytes;
                if (A.l2_stream)
                    bulk_load_stream(slot0 + (uint32_t)stage * 32 * G.slot_bytes, src, bytes, bar, l2_policy);
                else
                    bulk_load(slot0 + (uint32_t)stage * 32 * G.slot_bytes, src, bytes, bar);
            }
            return;
        }
        if (TQ) {
            // TQ2_0 split rows: one swizzled payload box of 32 rows x 128 bytes (512 weights per row)
            if (lane == 0) {
                mbar_arrive_expect_tx(bar, (uint32_t)kTqStageBytes);
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                        slot0 + (uint32_t)stage * stage_stride),
                    "l"(&tmap), "r"(sl * 128), "r"(row0), "r"(bar)
                    : "memory");
            }
            return;
        }
        if (q8_boxes) {
            // Q8_0 split rows: two swizzled payload boxes (32 rows x 128 bytes) and the 32 x 16 scale bytes
            if (lane == 0) {
                mbar_arrive_expect_tx(bar, (uint32_t)(32 * 272));
                const uint32_t dst = slot0 + (uint32_t)stage * stage_stride;
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                    "l"(&tmap), "r"(sl * 256), "r"(row0), "r"(bar)
                    : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst + 4096),
                    "l"(&tmap), "r"(sl * 256 + 128), "r"(row0), "r"(bar)
                    : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst + 8192),
                    "l"(&tmap2), "r"(sl * 16), "r"(row0), "r"(bar)
                    : "memory");
            }
            return;
        }
        if (A.use_tmap) {
            // one 2-D tensor copy per warp step: 32 rows x one unit, landing densely (the unit size is an
            // odd number of 16-byte chunks, so the rows need no padding to stay bank-conflict free);
            // rows past the end of the matrix arrive as zeros
            if (lane == 0) {
                mbar_arrive_expect_tx(bar, (uint32_t)(32 * G.unit_bytes));
                const uint32_t dst = slot0 + (uint32_t)stage * 32 * G.slot_bytes;  // lane 0's slot = the stage base
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                    "l"(&tmap), "r"(sl * G.unit_bytes), "r"(row0), "r"(bar)
                    : "memory");
            }
            return;
        }
        if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)(nvalid * nu * (G.unit_bytes + G.scale_bytes)));
        __syncwarp();
        if (lane < nvalid) {
            const uint8_t* row = wbase + (size_t)(row0 + lane) * A.w.row_stride;
            const uint32_t dst = slot0 + (uint32_t)stage * 32 * G.slot_bytes;
            bulk_load(dst, row + (size_t)sl * A.slab * G.unit_bytes, (uint32_t)(nu * G.unit_bytes), bar);
            if (G.scale_bytes)
                bulk_load(dst + G.scale_off, row + (size_t)units * G.unit_bytes + (size_t)sl * A.slab * G.scale_bytes,
                          (uint32_t)(nu * G.scale_bytes), bar);
        }
    };

    // let the next kernel of the stream begin its own launch; it waits below before it reads or writes
    // anything this kernel (or an earlier one) may still be producing
    stamp(8);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    stamp(9);

    // start streaming weights before touching the activations
    const int prefetch = min(A.stages, total);
    for (int it = 0; it < prefetch; ++it) issue(it);

    // TQ2_0 and Q6_K keep their f16 block scales in a plane of their own behind the payload of a row; a lane reads the
    // scale bits of its row for a pipeline step with a plain load. Requested at the top of the step that needs them,
    // that load's whole DRAM latency is exposed once per step (profiled: 3.3 long-scoreboard stall cycles per issued instruction); so they
    // are requested two steps ahead and travel through two registers.
    auto plane_scales = [&](int step) -> uint32_t {
        const int tile = step / my_slabs, sl = warp + kWarps * (step % my_slabs);
        int row0, nvalid;
        tile_rows(tile, row0, nvalid);
        const uint8_t* row = wbase + (size_t)min(row0 + lane, n - 1) * A.w.row_stride;
        if (TQ) return __ldg(reinterpret_cast<const uint32_t*>(row + (size_t)(k >> 2)) + sl);
        return (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(row + (size_t)units * 208) + sl);
    };
    // the first two are requested here, with the first weight copies, ahead of the dependency wait (weights are immutable)
    uint32_t ps0 = 0, ps1 = 0;
    if (TQ || Q6) {
        if (total > 0) ps0 = plane_scales(0);
        if (total > 1) ps1 = plane_scales(1);
    }

    // everything before this point read only immutable weights; activations and outputs may belong
    // to the preceding kernel
    stamp(1);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    stamp(2);

    // activation records: quantise here (FUSED) or copy the pre-quantised records
    if (FUSED) {
        // warp w quantises activation blocks w, w+kWarps, ...: with one-unit slabs these are exactly the
        // blocks it consumes, so no CTA-wide barrier is needed before it starts on its weights
        const int nblk = k >> 8;
        const size_t a_stride = A.pre.op == FQ_PRE_SPLIT_SWIGLU ? (size_t)2 * k : (size_t)k;  // input values per row
        float pre_scale[MB];
#pragma unroll
        for (int b = 0; b < MB; ++b) pre_scale[b] = 0.0f;
        if (A.pre.op == FQ_PRE_RMS_NORM_MUL) {
            // the rows' sums of squares: block sums by the warps that will quantise those blocks, parked in the
            // (still unused) reduction buffer, then added in block order by every thread
            float* part = red;
            for (int i = 0; i < MB * ((nblk - warp + kWarps - 1) / kWarps); ++i) {
                const int blk = warp + (i / MB) * kWarps, b = i % MB;
                if (b >= A.m) continue;
                float v[8];
                load8(A.a_f32 + (size_t)b * a_stride + (size_t)blk * 256 + lane * 8, v);
                const float ss = block_sumsq(v);
                if (lane == 0) part[b * nblk + blk] = ss;
            }
            __syncthreads();
#pragma unroll
            for (int b = 0; b < MB; ++b)
                if (b < A.m) pre_scale[b] = rms_scale(part + b * nblk, nblk, A.pre.eps);
            __syncthreads();  // the buffer goes back to the tile loop
        }
        for (int i = 0; i < MB * ((nblk - warp + kWarps - 1) / kWarps); ++i) {
            const int blk = warp + (i / MB) * kWarps, b = i % MB;
            uint8_t* rec = acts + (size_t)b * NS.row;
            if (b < A.m) {
                if (A.pre.op == FQ_PRE_NONE) {
                    quantize_block_natural(A.a_f32 + (size_t)b * k, blk, FMT == FQ_Q6_K ? 2 : (Q8K ? 1 : 0), k, rec, lane);
                } else {
                    float v[8];
                    float scale = 0.0f;
#pragma unroll
                    for (int bb = 0; bb < MB; ++bb)
                        if (bb == b) scale = pre_scale[bb];
                    load_block_pre(A.pre, A.a_f32 + (size_t)b * a_stride, (size_t)k, blk, lane, scale, v);
                    quantize_values_natural(v, blk, FMT == FQ_Q6_K ? 2 : (Q8K ? 1 : 0), k, rec, lane);
                }
            } else {  // padded batch slots contribute zeros
                *reinterpret_cast<uint2*>(rec + (size_t)blk * 256 + lane * 8) = make_uint2(0, 0);
                if (Q8K) {
                    if (lane < 8) reinterpret_cast<int32_t*>(rec + NS.aq)[blk * 8 + lane] = 0;
                    if (lane == 0) reinterpret_cast<float*>(rec + NS.aq + NS.sums)[blk] = 0.0f;
                } else if (lane < 8) {
                    reinterpret_cast<float*>(rec + NS.aq)[blk * 8 + lane] = 0.0f;
                }
            }
        }
    } else {
        const int units_per_rec = (int)(NS.row / 16);
        const uint4* src = reinterpret_cast<const uint4*>(A.acts_nat);
        uint4* dst = reinterpret_cast<uint4*>(acts);
        for (int i = threadIdx.x; i < MB * units_per_rec; i += kThreads)
            dst[i] = (i / units_per_rec < A.m) ? __ldg(src + i) : make_uint4(0, 0, 0, 0);
    }
    if (FUSED && A.slab == 1 && !TQ)  // (a TQ2_0 step spans two activation blocks, quantised by two different warps)
        __syncwarp();
    else
        __syncthreads();

    stamp(3);
    const ActView V = {smem_u32(acts), (uint32_t)NS.row, (uint32_t)NS.aq, (uint32_t)(NS.aq + NS.sums)};
    bool ok = true;
    int it = 0;
    for (int tile = 0; tile < ntiles; ++tile) {
        // K-quant batches of 3..16 rows (MB = 8 or 16) multiply through the warp-level tensor-core instruction:
        // acc then holds the fragment layout of expert_block_mma, eight values per group of eight rows
        constexpr bool kMma = (FMT == FQ_Q4_K || FMT == FQ_Q5_K) && MB >= 8;
        float acc[MB];
#pragma unroll
        for (int b = 0; b < MB; ++b) acc[b] = 0.0f;
        for (int j = 0; j < my_slabs && ok; ++j, ++it) {
            const int sl = warp + kWarps * j;
            const int stage = it % A.stages;
            const uint32_t parity = (uint32_t)(it / A.stages) & 1u;
            // TQ2_0 / Q6_K: this lane's scale bits for this step were requested two steps ago (see plane_scales)
            const uint32_t step_scales = ps0;
            if (TQ || Q6) {
                ps0 = ps1;
                ps1 = it + 2 < total ? plane_scales(it + 2) : 0u;
            }
            const uint32_t tq_scales = step_scales;
            const float q6_dw = Q6 ? h2f((uint16_t)step_scales) : 0.0f;
            if (!mbar_wait(bar0 + stage * 8, parity)) {
                ok = false;
                break;
            }
            if (it == 0) stamp(4);
            const int nu = min(A.slab, units - sl * A.slab);
            const uint32_t p = slot0 + (uint32_t)stage * stage_stride;
            for (int u = 0; u < nu && !A.skip_compute; ++u) {
                const int kb = sl * A.slab + u;
                if (kMma) {
                    constexpr int UBK = FMT == FQ_Q4_K ? 144 : 176;
#pragma unroll
                    for (int tg = 0; tg < MB / 8; ++tg) {
                        const ActView Vt = {V.base + (uint32_t)(tg * 8) * V.row, V.row, V.off_sums, V.off_ad};
                        expert_block_mma<FMT == FQ_Q8_0 ? FQ_Q4_K : FMT>(p - (uint32_t)lane * G.slot_bytes + u * UBK * 32, Vt, kb, lane,
                                                                        *reinterpret_cast<float(*)[8]>(&acc[tg * 8 < MB ? tg * 8 : 0]));
                    }
                } else if (FMT == FQ_Q4_K) {
                    block_q4_k<MB>(p + u * 144, V, kb, acc);
                } else if (FMT == FQ_Q5_K) {
                    block_q5_k<MB>(p + u * 176, V, kb, acc);
                } else if (Q6) {
                    block_q6_k<MB>(p, q6_dw, V, kb, acc);
                }
                if (FMT == FQ_Q8_0) {
                    if (q8_boxes) unit_q8_0_swz<MB>(p, lane, V, kb, acc);
                    else unit_q8_0<MB>(p + u * 256, p + G.scale_off + u * 16, V, kb, acc);
                }
                if (TQ) unit_tq2_0_swz<MB>(p, lane, V, kb, tq_scales, acc);
            }
            __syncwarp();  // every lane is done with this stage before it is refilled
            if (it + A.stages < total) issue(it + A.stages);
        }
        // cross-warp sum of the K slices; two reduction buffers alternate so one CTA barrier per tile is enough
        if (tile == ntiles - 1) stamp(5);
        float* rbuf = red + (size_t)(tile & 1) * kWarps * MB * 32;
#pragma unroll
        for (int b = 0; b < MB; ++b) rbuf[(warp * MB + b) * 32 + lane] = acc[b];
        __syncthreads();
        for (int b = warp; b < MB; b += kWarps) {
            float s = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) s += rbuf[(w * MB + b) * 32 + lane];
            int row0, nvalid;
            tile_rows(tile, row0, nvalid);
            if (kMma) {
                // value b of a lane: token group b / 8, fragment slot i = b % 8 -> (row, token) of expert_block_mma
                const int i = b & 7;
                const int r = 16 * (i >> 2) + 8 * ((i >> 1) & 1) + (lane >> 2);
                const int tok = (b >> 3) * 8 + 2 * (lane & 3) + (i & 1);
                if (r < nvalid && tok < A.m) A.c[out_index(A, tok, row0 + r)] = s;
            } else if (lane < nvalid && b < A.m) {
                float* o = A.c + out_index(A, b, row0 + lane);
                *o = A.accumulate ? __fadd_rn(*o, s) : s;  // (sums of PTQTP planes: plane order is launch order)
            }
        }
    }
    stamp(6);
    stamp_flush();
    if (!ok) {
        if (lane == 0) *(volatile int*)A.status = FQ_ERR_TIMEOUT;
        // give copies still in flight a bounded chance to land before the CTA's shared memory is released
        for (int s = 0; s < A.stages; ++s) mbar_wait(bar0 + s * 8, 0);
    }
}

#ifdef FQ_TIMELINE
constexpr size_t kSmemLimit = 227 * 1024 - 256;  // the stamps live in static shared memory
#else
constexpr size_t kSmemLimit = 227 * 1024;
#endif
constexpr int kFusedMaxRows = 4;  // up to here each CTA quantises the activations itself

size_t smem_bytes(int fmt, int k, int mb, int slab, int stages, int warps) {
    const NatSizes NS = nat_sizes(fmt != FQ_Q8_0, (size_t)k);
    const SlabGeom G = slab_geom(fmt, slab);
    return 512 + ((mb * NS.row + 127) & ~(size_t)127) + (size_t)2 * warps * mb * 32 * sizeof(float) +
           (size_t)warps * stages * 32 * G.slot_bytes;
}

// 16 warps per CTA double the thread-level parallelism that hides shared-memory and dp4a latency;
// they need 16 units per row to split and the register budget of the small-batch variants.
int tq_warps(int k, int mb);
int pick_warps(int fmt, int k, int mb) {
    if (fmt == FQ_TQ2_0) return tq_warps(k, mb);
    static const int forced = getenv("FUCINA_B200_DECODE_WARPS") ? atoi(getenv("FUCINA_B200_DECODE_WARPS")) : 0;
    if (forced == 8) return 8;
    static const bool wide8 = getenv("FUCINA_B200_DECODE_WIDE8") ? atoi(getenv("FUCINA_B200_DECODE_WIDE8")) != 0 : true;
    const bool wide_ok = mb <= 2 || (mb == 8 && fmt != FQ_Q8_0 && fmt != FQ_Q6_K && wide8);  // the eight-row tensor-core variant also fits 16 warps
    if (k / 256 < 16 || !wide_ok) return 8;
    return smem_bytes(fmt, k, mb, 1, 2, 16) <= 227 * 1024 ? 16 : 8;  // the smallest 16-warp ring must fit
}

int pad_rows(size_t m) { return m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : 8; }
// Row tile of the dense kernel: K-quant batches of 3..16 rows run the tensor-core block product in groups of
// eight tokens; Q8_0 keeps dp4a up to eight rows.
constexpr int kMaxDecodeRows = 16;
int decode_pad_rows(int fmt, size_t m) {
    if (fmt == FQ_Q8_0 || fmt == FQ_TQ2_0 || fmt == FQ_Q6_K || m <= 2) return pad_rows(m);
    return m <= 8 ? 8 : 16;
}

// Two CTAs per SM (8 warps, 2 stages, at most half the SM's shared memory each) for tile-major
// weights. In-flight bytes per SM stay the same as one 16-warp CTA with a deeper ring, but a CTA of
// the NEXT launch (programmatic dependent launch) can take the place of a CTA that has finished while
// its neighbour is still working, so its first weight stages are already in shared memory when the
// predecessor drains: the per-launch ramp disappears from chains of decode products.
constexpr size_t kHalfSmemLimit = 113 * 1024;
bool half_sm_config(const DevWeights& w, int mb) {
    static const int env = getenv("FUCINA_B200_DECODE_HALF") ? atoi(getenv("FUCINA_B200_DECODE_HALF")) : 0;
    return env != 0 && w.tile_rows != 0 && smem_bytes(w.fmt, w.k, mb, 1, 2, 8) <= kHalfSmemLimit;
}

// deepest pipeline that fits: more bytes in flight per SM first, then fewer barriers per byte
bool pick_config(int fmt, int k, int mb, int* slab, int* stages) {
    const int warps = pick_warps(fmt, k, mb);
    static const int cand[][2] = {{1, 4}, {2, 2}, {1, 3}, {1, 2}};
    static int force_slab = -1, force_stages = -1;
    if (force_slab < 0) {
        const char* a = getenv("FUCINA_B200_DECODE_SLAB");
        const char* b = getenv("FUCINA_B200_DECODE_STAGES");
        force_slab = a ? atoi(a) : 0;
        force_stages = b ? atoi(b) : 0;
    }
    if (force_slab > 0 && force_stages > 0 && force_stages <= kMaxStages && smem_bytes(fmt, k, mb, force_slab, force_stages, warps) <= kSmemLimit) {
        *slab = force_slab, *stages = force_stages;
        return true;
    }
    for (auto& c : cand)
        if (smem_bytes(fmt, k, mb, c[0], c[1], warps) <= kSmemLimit) {
            *slab = c[0], *stages = c[1];
            return true;
        }
    return false;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no libcuda link dependency).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
        cudaGetLastError();
    }
    return fn;
}

// 2-D byte view of one weight matrix: inner dimension = the used bytes of a row, outer = rows;
// one box = one 256-weight unit of 32 consecutive rows.
bool make_weight_tmap(const DevWeights& w, int mat, int unit_bytes, CUtensorMap* out) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)(w.k / 256) * unit_bytes, (cuuint64_t)w.n};
    const cuuint64_t strides[1] = {(cuuint64_t)w.row_stride};
    const cuuint32_t box[2] = {(cuuint32_t)unit_bytes, 32};
    const cuuint32_t estr[2] = {1, 1};
    void* base = const_cast<uint8_t*>(w.base) + (size_t)mat * w.mat_stride;
    return fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Q8_0 split rows [K payload bytes][K/16 scale bytes]: a payload map (box 128 bytes x 32 rows, 128-byte swizzle)
// and a scale map over the second plane (box 16 bytes x 32 rows).
bool make_q8_tmaps(const DevWeights& w, int mat, CUtensorMap* payload, CUtensorMap* scales) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    uint8_t* base = const_cast<uint8_t*>(w.base) + (size_t)mat * w.mat_stride;
    if (((uintptr_t)base & 15) || (w.row_stride & 15)) return false;
    const cuuint32_t estr[2] = {1, 1};
    const cuuint64_t strides[1] = {(cuuint64_t)w.row_stride};
    const cuuint64_t pdims[2] = {(cuuint64_t)w.k, (cuuint64_t)w.n};
    const cuuint32_t pbox[2] = {128, 32};
    if (fn(payload, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, pdims, strides, pbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    const cuuint64_t sdims[2] = {(cuuint64_t)w.k / 16, (cuuint64_t)w.n};
    const cuuint32_t sbox[2] = {16, 32};
    return fn(scales, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base + w.k, sdims, strides, sbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// TQ2_0: payload map over the first plane (box 128 bytes = 512 weights x 32 rows, 128-byte swizzle)
bool make_tq_tmap(const DevWeights& w, int mat, CUtensorMap* payload) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    uint8_t* base = const_cast<uint8_t*>(w.base) + (size_t)mat * w.mat_stride;
    if (((uintptr_t)base & 15) || (w.row_stride & 15)) return false;
    const cuuint32_t estr[2] = {1, 1};
    const cuuint64_t strides[1] = {(cuuint64_t)w.row_stride};
    const cuuint64_t pdims[2] = {(cuuint64_t)w.k / 4, (cuuint64_t)w.n};
    const cuuint32_t pbox[2] = {128, 32};
    return fn(payload, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, pdims, strides, pbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
int tq_warps(int k, int mb) { return (k / 512 >= 16 && mb <= 2) ? 16 : 8; }
size_t smem_bytes_tq_boxes(int k, int mb, int stages, int warps) {
    const NatSizes NS = nat_sizes(true, (size_t)k);
    return 512 + ((mb * NS.row + 127) & ~(size_t)127) + (size_t)2 * warps * mb * 32 * sizeof(float) + 1024 + (size_t)warps * stages * kTqStageBytes;
}
size_t smem_bytes_q8_boxes(int k, int mb, int stages) {
    const NatSizes NS = nat_sizes(false, (size_t)k);
    return 512 + ((mb * NS.row + 127) & ~(size_t)127) + (size_t)2 * 8 * mb * 32 * sizeof(float) + 1024 + (size_t)8 * stages * kQ8StageBytes;
}

template <int FMT, int MB>
cudaError_t launch_fmt_mb(const RowsArgs& a, const CUtensorMap& tmap, const CUtensorMap& tmap2, bool fused, bool half, int grid, size_t smem,
                          cudaStream_t st) {
    constexpr bool kWide = MB <= 2 || (MB == 8 && FMT != FQ_Q8_0);  // the 16-warp form exists for these variants only
    const bool wide = kWide && !half && pick_warps(FMT, a.w.k, MB) == 16;
    void (*kern)(const RowsArgs, const CUtensorMap, const CUtensorMap) =
        wide ? (fused ? decode_rows_kernel<FMT, MB, true, kWide ? 16 : 8> : decode_rows_kernel<FMT, MB, false, kWide ? 16 : 8>)
             : (fused ? decode_rows_kernel<FMT, MB, true, 8> : decode_rows_kernel<FMT, MB, false, 8>);
    // opt in to the large dynamic shared memory once per instantiation, not per launch
    static bool granted[2][2] = {{false, false}, {false, false}};
    if (!granted[wide][fused]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit);
        if (e != cudaSuccess) return e;
        // all of the SM's configurable memory as shared memory, so two half-size CTAs fit side by side
        e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        granted[wide][fused] = true;
    }
    // Programmatic dependent launch: this grid may be scheduled while the previous kernel of the
    // stream drains. It only touches read-only weights and its own shared memory before
    // griddepcontrol.wait, so the launch latency and the first weight loads overlap the predecessor.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(wide ? 512 : 256);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    static const bool no_pdl = getenv("FUCINA_B200_NO_PDL") != nullptr;
    cfg.attrs = attr;
    cfg.numAttrs = no_pdl ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kern, a, tmap, tmap2);
}

template <int FMT>
cudaError_t launch_fmt(const RowsArgs& a, const CUtensorMap& tmap, const CUtensorMap& tmap2, int mb, bool fused, bool half, int grid, size_t smem,
                       cudaStream_t st) {
    switch (mb) {
        case 1: return launch_fmt_mb<FMT, 1>(a, tmap, tmap2, fused, half, grid, smem, st);
        case 2: return launch_fmt_mb<FMT, 2>(a, tmap, tmap2, fused, half, grid, smem, st);
        case 4: return launch_fmt_mb<FMT, 4>(a, tmap, tmap2, fused, half, grid, smem, st);
        case 16: return launch_fmt_mb<FMT, 16>(a, tmap, tmap2, fused, half, grid, smem, st);
        default: return launch_fmt_mb<FMT, 8>(a, tmap, tmap2, fused, half, grid, smem, st);
    }
}


// Q6_K has the dp4a block product only: batches of one, two, four and eight rows, 16 warps for the first two
template <int MB>
cudaError_t launch_q6_mb(const RowsArgs& a, const CUtensorMap& tmap, const CUtensorMap& tmap2, bool fused, int grid, size_t smem, cudaStream_t st) {
    constexpr bool kWide = MB <= 2;
    const bool wide = kWide && pick_warps(FQ_Q6_K, a.w.k, MB) == 16;
    void (*kern)(const RowsArgs, const CUtensorMap, const CUtensorMap) =
        wide ? (fused ? decode_rows_kernel<FQ_Q6_K, MB, true, kWide ? 16 : 8> : decode_rows_kernel<FQ_Q6_K, MB, false, kWide ? 16 : 8>)
             : (fused ? decode_rows_kernel<FQ_Q6_K, MB, true, 8> : decode_rows_kernel<FQ_Q6_K, MB, false, 8>);
    static bool granted[2][2] = {{false, false}, {false, false}};
    if (!granted[wide][fused]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        granted[wide][fused] = true;
    }
    return launch_pdl(kern, dim3((unsigned)grid), dim3(wide ? 512 : 256), smem, st, a, tmap, tmap2);
}
cudaError_t launch_fmt_q6(const RowsArgs& a, const CUtensorMap& tmap, const CUtensorMap& tmap2, int mb, bool fused, int grid, size_t smem, cudaStream_t st) {
    switch (mb) {
        case 1: return launch_q6_mb<1>(a, tmap, tmap2, fused, grid, smem, st);
        case 2: return launch_q6_mb<2>(a, tmap, tmap2, fused, grid, smem, st);
        case 4: return launch_q6_mb<4>(a, tmap, tmap2, fused, grid, smem, st);
        default: return launch_q6_mb<8>(a, tmap, tmap2, fused, grid, smem, st);
    }
}

// TQ2_0 has the dp4a block product only: batches of one, two and four rows
cudaError_t launch_fmt_tq(const RowsArgs& a, const CUtensorMap& tmap, const CUtensorMap& tmap2, int mb, bool fused, int grid, size_t smem, cudaStream_t st) {
    switch (mb) {
        case 1: return launch_fmt_mb<FQ_TQ2_0, 1>(a, tmap, tmap2, fused, false, grid, smem, st);
        case 2: return launch_fmt_mb<FQ_TQ2_0, 2>(a, tmap, tmap2, fused, false, grid, smem, st);
        default: return launch_fmt_mb<FQ_TQ2_0, 4>(a, tmap, tmap2, fused, false, grid, smem, st);
    }
}

// ---------------------------------------------------------------------------------------------
// Grouped form for MoE expert stacks at decode batch sizes: the same row-per-lane arithmetic over
// a device-built table of (expert, run of <= 8 activation rows) entries.
//
// A work item is (table entry, group of TPI 32-row tiles of the expert's matrix), dealt round-robin
// to one persistent CTA per SM. The 8 warps of the CTA are arranged as TPI tiles x (8 / TPI) K parts:
// with many items every warp owns a whole tile and walks all of K by itself (no cross-warp sum);
// with few items (a single token) the warps split K so that more SMs have work. Weights are
// row-major expert stacks, fetched with one 2-D tensor copy per warp step (32 rows x one 256-weight
// unit) into a per-warp ring; the copies of the next item are in flight while this one is consumed.
// The entry's activation rows are quantised by the CTA itself (Q8_K, the CPU kernels' quantiser)
// straight from f32: token rows through the sorted pair list for the gate/up product, pair rows for
// the down product. GATED multiplies the gate and the up matrix in the same pass and stores
// up * gate * sigmoid(gate).
constexpr int kExpertWarps = 8;

// One block of one row against the first M activation records, accumulators acc[0..M).
template <int FMT, int M>
__device__ __forceinline__ void expert_block(uint32_t p, const ActView& V, int unit, float* acc, float dw) {
    float(&a)[M] = *reinterpret_cast<float(*)[M]>(acc);
    if (FMT == FQ_Q4_K) block_q4_k<M>(p, V, unit, a);
    if (FMT == FQ_Q5_K) block_q5_k<M>(p, V, unit, a);
    if (FMT == FQ_Q6_K) block_q6_k<M>(p, dw, V, unit, a);  // `dw`: the block's f16 scale from the plane behind the row's payload
}
// Entries mostly hold fewer rows than the launch-wide bound MB (a token batch spreads over many
// experts), so the block product is instantiated for 1, 2, 4 and 8 rows and chosen per entry.
__host__ __device__ inline int expert_rows_step(int m) { return m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : 8; }
template <int FMT, int MB>
__device__ __forceinline__ void expert_block_m(int mstep, uint32_t p, const ActView& V, int unit, float* acc, float dw) {
    if (MB >= 8 && mstep == 8) return expert_block<FMT, MB >= 8 ? 8 : MB>(p, V, unit, acc, dw);
    if (MB >= 4 && mstep == 4) return expert_block<FMT, MB >= 4 ? 4 : MB>(p, V, unit, acc, dw);
    if (MB >= 2 && mstep == 2) return expert_block<FMT, MB >= 2 ? 2 : MB>(p, V, unit, acc, dw);
    expert_block<FMT, 1>(p, V, unit, acc, dw);
}

template <int FMT, int MB, bool GATED>
__global__ void __launch_bounds__(kExpertWarps * 32, (MB == 8 && FMT != FQ_Q6_K) ? 2 : 1)  // eight-row tables: two CTAs per SM (128 registers, no spills)
    expert_rows_kernel(const ExpertArgs A, const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap tmap2) {
    extern __shared__ __align__(128) uint8_t smem[];
    // The table, its length, the pair list and the activation rows come from the kernels before this one: nothing
    // global is read before the predecessor has completed (the launch itself overlaps its tail).
    pdl_wait_then_release();
    constexpr int NM = GATED ? 2 : 1;
    constexpr int UB = FMT == FQ_Q4_K ? 144 : FMT == FQ_Q5_K ? 176 : 208;  // Q6_K: the payload of a unit; its f16 scale by a plain load
    constexpr bool Q6 = FMT == FQ_Q6_K;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int k = A.w.k, n = A.w.n;
    const int mat_rows = A.w.n_mats > 1 ? (int)(A.w.mat_stride / A.w.row_stride) : n;
    const NatSizes NS = nat_sizes(true, k);
    const int units = k >> 8;
    const int tpi = A.tiles_per_item, ksplit = kExpertWarps / tpi;
    const int tsub = warp / ksplit, kpart = warp % ksplit;
    const int my_units = kpart < units ? (units - kpart + ksplit - 1) / ksplit : 0;
    const int spi = my_units * NM;  // pipeline steps of this warp per item
    const int tiles_per_mat = (n + 31) >> 5;
    const int items_per_desc = (tiles_per_mat + tpi - 1) / tpi;
    const int n_desc = min(*A.n_desc, A.max_desc);
    const int total_items = n_desc * items_per_desc;
    const int my_items = (int)blockIdx.x < total_items ? (total_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

    // shared memory: barriers | activation records | reduction buffer | per-warp stage ring
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    uint8_t* acts = smem + 512;
    float* red = reinterpret_cast<float*>(acts + ((MB * NS.row + 127) & ~(size_t)127));
    uint8_t* slots = reinterpret_cast<uint8_t*>(red) + (ksplit > 1 ? (size_t)kExpertWarps * NM * MB * 32 * sizeof(float) : 0);  // no K split, no buffer
    const uint32_t slot0 = smem_u32(slots) + (uint32_t)(warp * A.stages) * 32 * UB;
    const uint32_t bar0 = smem_u32(bars) + warp * kMaxStages * 8;
    if (lane == 0)
        for (int s = 0; s < A.stages; ++s) mbar_init(bar0 + s * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncwarp();

    // Step `it` of this warp: item it / spi, unit kpart + ksplit * (j / NM), matrix j % NM, j = it % spi.
    // A warp whose tile lies past the end of the matrix (last group of a matrix) has no copies in that
    // item, so ring slots and barrier phases are counted in copies actually issued, not in steps.
    auto item_of = [&](int item_local, int& d, int& tile) {
        const int item = blockIdx.x + item_local * gridDim.x;
        d = item / items_per_desc;
        tile = (item % items_per_desc) * tpi + tsub;
    };
    const int total = my_items * spi;
    int next_it = 0, issued = 0, consumed = 0;
    auto advance = [&]() {  // keep up to `stages` copies in flight
        while (issued < consumed + A.stages && next_it < total) {
            int d, tile;
            item_of(next_it / spi, d, tile);
            if (tile < tiles_per_mat) {
                if (lane == 0) {
                    const int j = next_it % spi, unit = kpart + ksplit * (j / NM);
                    const int stage = issued % A.stages;
                    const uint32_t bar = bar0 + stage * 8;
                    // row in the stacked matrix: experts are mat_rows rows apart (n for a dense stack, more for a row view of a wider one)
                    const int row = A.table[d].mat * mat_rows + tile * 32;
                    mbar_arrive_expect_tx(bar, (uint32_t)(32 * UB));
                    const CUtensorMap* tm = (GATED && (j % NM)) ? &tmap2 : &tmap;
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                            slot0 + (uint32_t)stage * 32 * UB),
                        "l"(tm), "r"(unit * UB), "r"(row), "r"(bar)
                        : "memory");
                }
                ++issued;
            }
            ++next_it;
        }
    };

    advance();

    const ActView V = {smem_u32(acts), (uint32_t)NS.row, (uint32_t)NS.aq, (uint32_t)(NS.aq + NS.sums)};
    bool ok = true;  // per warp; a warp that gave up still walks through every CTA barrier below
    // Q6_K: scale bits of this lane's row (its matrix by j % NM) for step j of item il, from the plane behind the payload
    auto plane_scale = [&](int il, int j) -> uint32_t {
        int d, tile;
        item_of(il, d, tile);
        const DevWeights& W = (GATED && (j % NM)) ? A.w2 : A.w;
        const int row = A.table[d].mat * mat_rows + min(tile * 32 + lane, n - 1);
        const int unit = kpart + ksplit * (j / NM);
        return (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(W.base + (size_t)row * W.row_stride + (size_t)units * 208) + unit);
    };
    uint32_t q6_next = 0;
    int q6_for = -1;  // the step q6_next was requested for
    for (int il = 0; il < my_items; ++il) {
        int d, tile;
        item_of(il, d, tile);
        const GroupDesc G = A.table[d];
        if (il) __syncthreads();  // everyone is done with the previous item's activation records
        // quantise this entry's rows: (row b, block blk) pairs over the warps; the slots up to the row count the
        // block product is instantiated for are zero
        const int nblk = k >> 8;
        // entries of three or more rows in an eight-row launch use the tensor-core block product (CTA-uniform choice)
        const bool kMma = !Q6 && MB == 8 && G.m > 2;
        const int mstep = kMma ? MB : min(MB, expert_rows_step(G.m));
        for (int i = warp; i < mstep * nblk; i += kExpertWarps) {
            const int b = i / nblk, blk = i % nblk;
            uint8_t* rec = acts + (size_t)b * NS.row;
            if (b < G.m) {
                const int pos = G.row0 + b;
                const size_t src_row = A.src_index ? (size_t)(A.src_index[pos] / A.top_k) : (size_t)pos;
                quantize_block_natural(A.src + src_row * k, blk, Q6 ? 2 : 1, k, rec, lane);
            } else {
                *reinterpret_cast<uint2*>(rec + (size_t)blk * 256 + lane * 8) = make_uint2(0, 0);
                if (lane < 8) reinterpret_cast<int32_t*>(rec + NS.aq)[blk * 8 + lane] = 0;
                if (lane == 0) reinterpret_cast<float*>(rec + NS.aq + NS.sums)[blk] = 0.0f;
            }
        }
        __syncthreads();

        float acc[NM][MB];
#pragma unroll
        for (int q = 0; q < NM; ++q)
#pragma unroll
            for (int b = 0; b < MB; ++b) acc[q][b] = 0.0f;
        const bool have_tile = tile < tiles_per_mat;
        if (have_tile) {
            for (int j = 0; j < spi; ++j) {
                if (!ok) break;
                const int unit = kpart + ksplit * (j / NM), stage = consumed % A.stages;
                // Q6_K: the f16 scale of this lane's row for this step, requested during the step before (or, for the
                // first step of an item, here); the next step's request goes out before this step's wait
                float dw = 0.0f;
                if (Q6) {
                    const uint32_t bits = (q6_for == il * spi + j) ? q6_next : plane_scale(il, j);
                    if (j + 1 < spi) {
                        q6_next = plane_scale(il, j + 1);
                        q6_for = il * spi + j + 1;
                    }
                    dw = h2f((uint16_t)bits);
                }
                if (!mbar_wait(bar0 + stage * 8, (uint32_t)(consumed / A.stages) & 1u)) {
                    ok = false;
                    break;
                }
                const uint32_t tile_base = slot0 + (uint32_t)stage * 32 * UB;
                const uint32_t p = tile_base + (uint32_t)lane * UB;
                if (kMma) {
                    if (!GATED || (j % NM) == 0)
                        expert_block_mma<Q6 ? FQ_Q5_K : FMT>(tile_base, V, unit, lane, reinterpret_cast<float(&)[8]>(acc[0]));
                    else
                        expert_block_mma<Q6 ? FQ_Q5_K : FMT>(tile_base, V, unit, lane, reinterpret_cast<float(&)[8]>(acc[NM - 1]));
                } else if (!GATED || (j % NM) == 0) {
                    expert_block_m<FMT, MB>(mstep, p, V, unit, acc[0], dw);
                } else {
                    expert_block_m<FMT, MB>(mstep, p, V, unit, acc[NM - 1], dw);
                }
                __syncwarp();  // every lane is done with this stage before it is refilled
                ++consumed;
                advance();
            }
        }

        // K parts of a tile live in consecutive warps: sum them (ksplit > 1), then apply the gate and store
        if (ksplit > 1) {
#pragma unroll
            for (int q = 0; q < NM; ++q)
#pragma unroll
                for (int b = 0; b < MB; ++b) red[((warp * NM + q) * MB + b) * 32 + lane] = acc[q][b];
            __syncthreads();
            if (kpart == 0) {
#pragma unroll
                for (int q = 0; q < NM; ++q)
#pragma unroll
                    for (int b = 0; b < MB; ++b) {
                        float sum = 0.0f;
                        for (int w2 = 0; w2 < ksplit; ++w2) sum += red[(((warp + w2) * NM + q) * MB + b) * 32 + lane];
                        acc[q][b] = sum;
                    }
            }
        }
        if (kMma) {
            // fragment layout: acc[4*grp + 2*half + c] = (row 16*grp + 8*half + lane/4, token 2*(lane%4) + c)
            if (kpart == 0 && have_tile) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int row = tile * 32 + 16 * (i >> 2) + 8 * ((i >> 1) & 1) + (lane >> 2);
                    const int b = 2 * (lane & 3) + (i & 1);
                    if (row >= n || b >= G.m) continue;
                    float v = acc[0][i < MB ? i : 0];
                    if (GATED) v = gated_pair(A.gated_op, v, acc[NM - 1][i < MB ? i : 0]);
                    A.out[(size_t)(G.row0 + b) * n + row] = v;
                }
            }
            continue;
        }
        const int row = tile * 32 + lane;
        if (kpart == 0 && have_tile && row < n) {
#pragma unroll
            for (int b = 0; b < MB; ++b) {
                if (b >= G.m) continue;
                float v = acc[0][b];
                if (GATED) v = gated_pair(A.gated_op, acc[0][b], acc[NM - 1][b]);
                A.out[(size_t)(G.row0 + b) * n + row] = v;
            }
        }
    }
    if (!ok) {
        if (lane == 0) *(volatile int*)A.status = FQ_ERR_TIMEOUT;
        // give copies still in flight a bounded chance to land before the CTA's shared memory is released
        for (int s = 0; s < A.stages; ++s) mbar_wait(bar0 + s * 8, (uint32_t)((consumed + s) / A.stages) & 1u);
    }
}

size_t expert_smem_bytes(int fmt, int k, int mb, int nm, int stages, bool k_split = true) {
    const NatSizes NS = nat_sizes(true, (size_t)k);
    const int ub = fmt == FQ_Q4_K ? 144 : fmt == FQ_Q5_K ? 176 : 208;
    return 512 + ((mb * NS.row + 127) & ~(size_t)127) + (k_split ? (size_t)kExpertWarps * nm * mb * 32 * sizeof(float) : 0) +
           (size_t)kExpertWarps * stages * 32 * ub;
}

template <int FMT, int MB, bool GATED>
cudaError_t launch_expert_t(const ExpertArgs& a, const CUtensorMap& t1, const CUtensorMap& t2, int grid, size_t smem, cudaStream_t st) {
    auto kern = expert_rows_kernel<FMT, MB, GATED>;
    static bool granted = false;
    if (!granted) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit);
        if (e != cudaSuccess) return e;
        // all of the SM's configurable memory as shared memory, so two CTAs of up to 113 KB fit side by side
        e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        granted = true;
    }
    // short tables (decode) chain by programmatic dependent launch; with every CTA slot of the part taken by one grid
    // the early launch of the next has nowhere to go and measured 2 % slower
    if (a.chain) return launch_pdl(kern, dim3(grid), dim3(kExpertWarps * 32), smem, st, a, t1, t2);
    kern<<<grid, kExpertWarps * 32, smem, st>>>(a, t1, t2);
    return cudaGetLastError();
}

template <int FMT, bool GATED>
cudaError_t launch_expert_mb(const ExpertArgs& a, int mb, const CUtensorMap& t1, const CUtensorMap& t2, int grid, size_t smem, cudaStream_t st) {
    switch (mb) {
        case 1: return launch_expert_t<FMT, 1, GATED>(a, t1, t2, grid, smem, st);
        case 2: return launch_expert_t<FMT, 2, GATED>(a, t1, t2, grid, smem, st);
        case 4: return launch_expert_t<FMT, 4, GATED>(a, t1, t2, grid, smem, st);
        default: return launch_expert_t<FMT, 8, GATED>(a, t1, t2, grid, smem, st);
    }
}

// 2-D byte view of a whole expert stack: [experts * n rows][row bytes], box = 32 rows x one unit
bool make_stack_tmap(const DevWeights& w, int unit_bytes, CUtensorMap* out) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t mat_rows = w.n_mats > 1 ? w.mat_stride / w.row_stride : (cuuint64_t)w.n;
    const cuuint64_t dims[2] = {(cuuint64_t)(w.k / 256) * unit_bytes, mat_rows * (cuuint64_t)(w.n_mats - 1) + (cuuint64_t)w.n};
    const cuuint64_t strides[1] = {(cuuint64_t)w.row_stride};
    const cuuint32_t box[2] = {(cuuint32_t)unit_bytes, 32};
    const cuuint32_t estr[2] = {1, 1};
    return fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(w.base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Self-test of the bounded-wait mechanism every pipeline in this file relies on: one warp waits, with the
// given iteration limit, on an mbarrier that nothing ever completes, records FQ_ERR_TIMEOUT in the status
// word exactly as the kernels above do, and returns normally. No copy is in flight and nothing else is touched.
__global__ void bounded_wait_probe_kernel(int* status, unsigned limit) {
    __shared__ __align__(8) uint64_t bar;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) mbar_init(b, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncwarp();
    bool done = false;
    for (unsigned i = 0; i < limit && !done; ++i) done = mbar_try_wait(b, 0);
    if (!done && threadIdx.x == 0) *(volatile int*)status = FQ_ERR_TIMEOUT;
}

}  // namespace

cudaError_t launch_bounded_wait_probe(int* status, unsigned limit, cudaStream_t st) {
    bounded_wait_probe_kernel<<<1, 32, 0, st>>>(status, limit);
    return cudaGetLastError();
}

bool decode_rows_eligible(const DevWeights& w, size_t m) {
    if (w.fmt == FQ_TQ2_0) {
        static const bool off = getenv("FUCINA_B200_NO_TQ_DECODE") != nullptr;
        if (off || m < 1 || m > (size_t)kFusedMaxRows || w.k % 512 != 0 || w.k < 2048 || w.n < 64 || w.tile_rows || !encode_tiled_fn()) return false;
        if (((uintptr_t)w.base & 15) || (w.row_stride & 15) || (w.mat_stride & 15)) return false;
        const int mb = pad_rows(m);
        return smem_bytes_tq_boxes(w.k, mb, 2, tq_warps(w.k, mb)) <= kSmemLimit;
    }
    if (w.fmt == FQ_Q6_K) {
        // split rows [payload | f16 scales], row-major; the payload is fetched by tensor copies (base and row stride rules)
        static const bool off = getenv("FUCINA_B200_NO_Q6_DECODE") != nullptr;
        if (off || m < 1 || m > 8 || w.k % 256 != 0 || w.k < 2048 || w.n < 64 || w.tile_rows || !encode_tiled_fn()) return false;
        if (((uintptr_t)w.base & 15) || (w.row_stride & 15) || (w.mat_stride & 15)) return false;
        return smem_bytes(w.fmt, w.k, pad_rows(m), 1, 2, pick_warps(w.fmt, w.k, pad_rows(m))) <= kSmemLimit;
    }
    if (w.fmt != FQ_Q4_K && w.fmt != FQ_Q5_K && w.fmt != FQ_Q8_0) return false;
    if (m < 1 || m > (size_t)(w.fmt == FQ_Q8_0 ? 8 : kMaxDecodeRows) || w.k % 256 != 0 || w.k < 2048 || w.n < 64) return false;
    int slab, stages;
    return pick_config(w.fmt, w.k, decode_pad_rows(w.fmt, m), &slab, &stages);
}

size_t decode_rows_scratch_bytes(const DevWeights& w, size_t m) {
    if ((int)m <= kFusedMaxRows) return 0;
    return nat_sizes(w.fmt != FQ_Q8_0, (size_t)w.k).row * m;
}

// the fused prologue parks m * k/256 block sums in the reduction buffer (at least 2 * 8 * 32 floats per padded row)
bool decode_rows_fuses_prologue(const DevWeights& w, size_t m) { return decode_rows_eligible(w, m) && (int)m <= kFusedMaxRows && w.k / 256 <= 512; }

cudaError_t launch_decode_rows(const DevWeights& w, int mat, const float* a_dev, uint8_t* scratch, float* c, int m, int ldc,
                               int sm_count, int* status, cudaStream_t st, int split_n, const PreArgs* pre, int accumulate) {
    const int mb = decode_pad_rows(w.fmt, (size_t)m);
    static const int skip = getenv("FUCINA_B200_DECODE_SKIP_COMPUTE") ? 1 : 0;  // diagnosis: copy pipeline only, outputs are garbage
    static const int l2_stream = getenv("FUCINA_B200_DECODE_L2_STREAM") ? atoi(getenv("FUCINA_B200_DECODE_L2_STREAM")) : 1;
    RowsArgs a{w, mat, a_dev, scratch, c, m, ldc, 1, 2, status, 0, skip, l2_stream, 0, split_n, pre ? *pre : PreArgs{FQ_PRE_NONE, nullptr, 0.0f}, accumulate};
    if (a.pre.op != FQ_PRE_NONE && !decode_rows_fuses_prologue(w, (size_t)m)) return cudaErrorInvalidValue;
    if (w.fmt == FQ_TQ2_0) {
        CUtensorMap tm, tm2;
        memset(&tm2, 0, sizeof tm2);
        if (!make_tq_tmap(w, mat, &tm)) return cudaErrorInvalidValue;
        const int warps = tq_warps(w.k, mb);
        a.slab = 1;
        a.use_tmap = 3;
        a.stages = smem_bytes_tq_boxes(w.k, mb, 3, warps) <= kSmemLimit ? 3 : 2;
        int grid_tq = sm_count;
        if (grid_tq > (w.n + 31) / 32) grid_tq = (w.n + 31) / 32;
        return launch_fmt_tq(a, tm, tm2, mb, true, grid_tq, smem_bytes_tq_boxes(w.k, mb, a.stages, warps), st);
    }
    if (w.fmt == FQ_Q6_K) {
        CUtensorMap tm, tm2;
        memset(&tm2, 0, sizeof tm2);
        if (!make_weight_tmap(w, mat, 208, &tm)) return cudaErrorInvalidValue;
        const int warps = pick_warps(w.fmt, w.k, mb);
        a.slab = 1;
        a.use_tmap = 1;
        a.stages = 2;
        while (a.stages < kMaxStages && smem_bytes(w.fmt, w.k, mb, 1, a.stages + 1, warps) <= kSmemLimit) ++a.stages;
        const bool fused_q6 = m <= kFusedMaxRows;
        if (!fused_q6) {
            cudaError_t e = launch_quantize_acts_natural(a_dev, m, w.k, 2, scratch, st);
            if (e != cudaSuccess) return e;
        }
        int grid_q6 = sm_count;
        if (grid_q6 > (w.n + 31) / 32) grid_q6 = (w.n + 31) / 32;
        return launch_fmt_q6(a, tm, tm2, mb, fused_q6, grid_q6, smem_bytes(w.fmt, w.k, mb, 1, a.stages, warps), st);
    }
    if (!pick_config(w.fmt, w.k, mb, &a.slab, &a.stages)) return cudaErrorInvalidValue;
    // K-quant units are an odd number of 16-byte chunks: one tensor copy per warp step instead of 32
    // per-lane bulk copies (small bulk copies are issue-rate bound in the copy engine)
    CUtensorMap tmap;
    memset(&tmap, 0, sizeof tmap);
    static const bool no_tmap = getenv("FUCINA_B200_DECODE_NO_TMAP") != nullptr;
    if (w.tile_rows) {
        a.slab = 1;  // tile-major runs are one unit wide
        // two stages of 16 x 4608 bytes keep ~144 KB per SM in flight; a deeper queue measured slower
        static const bool forced = getenv("FUCINA_B200_DECODE_STAGES") != nullptr;
        if (!forced && a.stages > 2) a.stages = 2;
    }
    if (w.fmt != FQ_Q8_0 && mb >= 8) a.slab = 1;  // the tensor-core block product reads one unit of 32 rows per stage
    if (!w.tile_rows && w.fmt != FQ_Q8_0 && a.slab == 1 && !no_tmap && make_weight_tmap(w, mat, slab_geom(w.fmt, 1).unit_bytes, &tmap)) a.use_tmap = 1;
    // Q8_0 rows are a payload plane and a scale plane: three tensor copies per warp step (two swizzled payload
    // boxes, one scale box) instead of 64 per-lane bulk copies
    CUtensorMap tmap2;
    memset(&tmap2, 0, sizeof tmap2);
    size_t smem_q8 = 0;
    if (w.fmt == FQ_Q8_0 && !no_tmap && w.k % 256 == 0 && make_q8_tmaps(w, mat, &tmap, &tmap2)) {
        smem_q8 = smem_bytes_q8_boxes(w.k, mb, 2);
        if (smem_q8 <= kSmemLimit) {
            a.use_tmap = 2;
            a.slab = 1;
            a.stages = 2;
        }
    }
    const bool fused = m <= kFusedMaxRows;
    if (!fused) {
        cudaError_t e = launch_quantize_acts_natural(a_dev, m, w.k, w.fmt != FQ_Q8_0, scratch, st);
        if (e != cudaSuccess) return e;
    }
    const bool half = half_sm_config(w, mb);
    if (half) a.stages = 2;
    int grid = half ? 2 * sm_count : sm_count;
    if (grid > (w.n + 7) / 8) grid = (w.n + 7) / 8;
    static const bool no_align = getenv("FUCINA_B200_DECODE_NO_ALIGN") != nullptr;
    if (w.tile_rows && !half && !no_align && (w.n + 31) / 32 <= sm_count) {
        grid = (w.n + 31) / 32;
        a.rows_per_cta = 32;
    }
    // larger tile-major matrices: whole storage tiles balanced over the grid. A CTA's range never straddles a tile, so
    // every pipeline step is one full 4608/5632-byte run (measured on B200: 32000 rows 14.7 -> 13.7 us, 11008 rows
    // 8.6 -> 7.7 us against an exact row split, whose straddling pieces each cost a full step)
    if (w.tile_rows && !half && !no_align && a.rows_per_cta == 0) a.rows_per_cta = -1;
    const size_t smem = a.use_tmap == 2 ? smem_q8 : smem_bytes(w.fmt, w.k, mb, a.slab, a.stages, half ? 8 : pick_warps(w.fmt, w.k, mb));
    switch (w.fmt) {
        case FQ_Q4_K: return launch_fmt<FQ_Q4_K>(a, tmap, tmap2, mb, fused, half, grid, smem, st);
        case FQ_Q5_K: return launch_fmt<FQ_Q5_K>(a, tmap, tmap2, mb, fused, half, grid, smem, st);
        default: return launch_fmt<FQ_Q8_0>(a, tmap, tmap2, mb, fused, half, grid, smem, st);
    }
}

#ifdef FQ_TIMELINE
// diagnostic build: copy the phase stamps of the last decode launch to the host
extern "C" __attribute__((visibility("default"))) int fq_debug_timeline(unsigned long long* out, int ctas) {
    return (int)cudaMemcpyFromSymbol(out, g_timeline, sizeof(unsigned long long) * kTimelineSlots * ctas);
}
#endif

// ---- grouped expert form (see expert_rows_kernel) --------------------------------------------
int expert_rows_max_group() { return 8; }

bool expert_rows_eligible(const DevWeights& w, const DevWeights* w2, int group_rows) {
    if (w.fmt != FQ_Q4_K && w.fmt != FQ_Q5_K && w.fmt != FQ_Q6_K) return false;
    if (w.tile_rows || w.k % 256 != 0 || w.k < 256 || group_rows < 1 || group_rows > 8) return false;
    if (w.n_mats > 1 && (w.mat_stride % w.row_stride != 0 || w.mat_stride < (size_t)w.n * w.row_stride)) return false;
    if (((uintptr_t)w.base & 15) || (w.row_stride & 15)) return false;  // tensor-map base and stride rules
    if (w2 && (w2->fmt != w.fmt || w2->k != w.k || w2->n != w.n || w2->tile_rows || w2->row_stride != w.row_stride || w2->mat_stride != w.mat_stride ||
               ((uintptr_t)w2->base & 15)))
        return false;
    static const bool off = getenv("FUCINA_B200_NO_EXPERT_ROWS") != nullptr;
    if (off || !encode_tiled_fn()) return false;
    return expert_smem_bytes(w.fmt, w.k, pad_rows((size_t)group_rows), w2 ? 2 : 1, 2) <= kSmemLimit;
}

cudaError_t launch_expert_rows(const DevWeights& w, const DevWeights* w2, const float* src, const int* src_index, int top_k, float* out,
                               const GroupDesc* table, const int* n_desc, int max_desc, int group_rows, int sm_count, int* status,
                               cudaStream_t st, int gated_op) {
    const int mb = pad_rows((size_t)group_rows), nm = w2 ? 2 : 1;
    const int ub = w.fmt == FQ_Q4_K ? 144 : w.fmt == FQ_Q5_K ? 176 : 208;
    int stages = kMaxStages;
    // tiles per item: whole tiles per warp when the table is long enough to fill the SMs, K split across
    // warps when it is short (a single token names top_k experts only)
    const int tiles_per_mat = (w.n + 31) / 32;
    int tpi = 8;
    while (tpi > 1 && (long long)max_desc * ((tiles_per_mat + tpi - 1) / tpi) < 2LL * sm_count) tpi >>= 1;
    const int units = w.k / 256;
    while (tpi < 8 && units < kExpertWarps / tpi) tpi <<= 1;  // no more K parts than units
    CUtensorMap t1, t2;
    memset(&t1, 0, sizeof t1);
    memset(&t2, 0, sizeof t2);
    if (!make_stack_tmap(w, ub, &t1) || (w2 && !make_stack_tmap(*w2, ub, &t2))) return cudaErrorInvalidValue;
    const bool k_split = tpi < kExpertWarps;  // the cross-warp reduction buffer exists only then
    while (stages > 2 && expert_smem_bytes(w.fmt, w.k, mb, nm, stages, k_split) > kSmemLimit) --stages;
    long long items = (long long)max_desc * ((tiles_per_mat + tpi - 1) / tpi);
    int grid = (int)(items < sm_count ? (items > 0 ? items : 1) : sm_count);
    // a short table (one token): one item per CTA and two half-size CTAs per SM instead of a second round
    if (items > sm_count && items <= 2LL * sm_count && expert_smem_bytes(w.fmt, w.k, mb, nm, 2, k_split) <= 113 * 1024) {
        grid = (int)items;
        stages = 2;
    }
    // eight-row tables run the warp-level tensor-core block product, which eight warps per SM leave latency-bound
    // (two warps per scheduler, issue slots half empty): two CTAs per SM with two-stage rings
    static const bool no_pair = getenv("FUCINA_B200_EXPERT_ONE_CTA") != nullptr;
    if (!no_pair && mb == 8 && w.fmt != FQ_Q6_K && items > sm_count && expert_smem_bytes(w.fmt, w.k, mb, nm, 2, k_split) <= 113 * 1024) {
        grid = (int)(items < 2LL * sm_count ? items : 2LL * sm_count);
        stages = 2;
    }
    ExpertArgs a{w, w2 ? *w2 : DevWeights{}, src, src_index, top_k, out, table, n_desc, max_desc, tpi, stages, status, gated_op, grid < 2 * sm_count ? 1 : 0};
    const size_t smem = expert_smem_bytes(w.fmt, w.k, mb, nm, stages, k_split);
    if (w.fmt == FQ_Q4_K)
        return w2 ? launch_expert_mb<FQ_Q4_K, true>(a, mb, t1, t2, grid, smem, st) : launch_expert_mb<FQ_Q4_K, false>(a, mb, t1, t2, grid, smem, st);
    if (w.fmt == FQ_Q6_K)
        return w2 ? launch_expert_mb<FQ_Q6_K, true>(a, mb, t1, t2, grid, smem, st) : launch_expert_mb<FQ_Q6_K, false>(a, mb, t1, t2, grid, smem, st);
    return w2 ? launch_expert_mb<FQ_Q5_K, true>(a, mb, t1, t2, grid, smem, st) : launch_expert_mb<FQ_Q5_K, false>(a, mb, t1, t2, grid, smem, st);
}

}  // namespace fq
