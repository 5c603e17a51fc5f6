// Device layout of int8-quantised activations as the decode kernels consume
// them ("gpu_formats" for the activation side).
//
// The CPU kernels of the reference quantise activation rows to Q8_K blocks
// (src/backend/quant/q8k.zig:268-313) or, for Q8_0 / Q2_0 weights, to Q8_0
// blocks (q8k.zig:49-69) before any integer dot runs
// (src/backend/native.zig:427-490). The values are reproduced exactly; only
// their placement changes: a decode kernel lane owns one 16-byte chunk of
// weight payload and needs the matching activations as 16-byte segments, so
// the int8 values of a row are stored permuted:
//
//     aq[(s * C + c) * 16 + i]   segment s of chunk c, byte i
//
// with C = K / chunk_elems chunks per row. Lane c then reads segment s at
// unit s*C + c: consecutive lanes hit consecutive 16-byte units (no shared
// memory bank conflicts), and the whole row is one flat copy into shared
// memory. Two side planes travel with it:
//     aaux[c]  one 32-bit word per chunk: the activation sums the format's
//              offset term needs (Q8_K bsums regrouped per chunk)
//     ad[b]    f32 scale per activation block (256 or 32 elements)
#pragma once
#include "common.cuh"

namespace fq {

struct ActLayout {
    int chunk_elems;  // weights covered by one 16-byte payload chunk
    int segs;         // 16-byte activation segments per chunk
    int act_block;    // activation scale granularity (256 = Q8_K, 32 = Q8_0)
};

__host__ __device__ inline ActLayout act_layout(int fmt) {
    switch (fmt) {
        case FQ_Q8_0: return {16, 1, 32};
        case FQ_Q4_K: return {32, 2, 256};
        case FQ_Q5_K: return {32, 2, 256};
        case FQ_Q6_K: return {32, 2, 256};
        case FQ_TQ2_0: return {64, 4, 256};
        case FQ_TQ2_0_FOLDED: return {32, 2, 256};
        case FQ_Q2_0: return {64, 4, 32};
        default: return {0, 0, 0};
    }
}

// Sizes of the three planes for one activation row.
struct ActSizes {
    size_t aq;    // bytes of int8 values (= K)
    size_t aaux;  // bytes of the per-chunk words
    size_t ad;    // bytes of the f32 scales
    size_t row;   // aq + aaux + ad, each 16-byte aligned
};
__host__ __device__ inline ActSizes act_sizes(int fmt, size_t k) {
    const ActLayout L = act_layout(fmt);
    ActSizes s;
    s.aq = k;
    s.aaux = ((k / L.chunk_elems) * 4 + 15) & ~(size_t)15;
    s.ad = ((k / L.act_block) * 4 + 15) & ~(size_t)15;
    s.row = s.aq + s.aaux + s.ad;
    return s;
}

// Element e of a row -> (chunk c, segment s, byte i).
__host__ __device__ inline void act_pos(int fmt, int e, int& c, int& s, int& i) {
    switch (fmt) {
        case FQ_Q4_K:
        case FQ_Q5_K: {
            // chunk = 16 nibble bytes of sub-block pair p, half h; low nibbles are
            // sub-block 2p (s = 0), high nibbles sub-block 2p+1 (s = 1)
            const int blk = e >> 8, sub = (e >> 5) & 7, h = (e >> 4) & 1;
            c = blk * 8 + (sub >> 1) * 2 + h;
            s = sub & 1;
            i = e & 15;
            return;
        }
        case FQ_Q6_K: {
            // chunk = 16 ql bytes: their low nibbles are 16 elements of section h32 (0 or 1) of a 128-element half
            // block, their high nibbles the same 16 positions of section h32 + 2 (q6_k.zig:1239-1259)
            const int blk = e >> 8, r = e & 255, c2 = r >> 7, sec = (r >> 5) & 3, l = r & 31;
            c = blk * 8 + c2 * 4 + (sec & 1) * 2 + (l >> 4);
            s = sec >> 1;
            i = l & 15;
            return;
        }
        case FQ_TQ2_0: {
            // byte m of half-group hg holds elements hg*128 + n*32 + m in crumb n
            const int blk = e >> 8, r = e & 255, hg = r >> 7, n = (r >> 5) & 3, h = (r >> 4) & 1;
            c = blk * 4 + hg * 2 + h;
            s = n;
            i = e & 15;
            return;
        }
        case FQ_TQ2_0_FOLDED:
            c = e >> 5;
            s = (e >> 4) & 1;
            i = e & 15;
            return;
        case FQ_Q2_0: {
            // byte b of a 16-byte chunk holds elements 4b..4b+3 in crumbs 0..3
            const int r = e & 63;
            c = e >> 6;
            s = r & 3;
            i = r >> 2;
            return;
        }
        default:  // FQ_Q8_0
            c = e >> 4;
            s = 0;
            i = e & 15;
            return;
    }
}

}  // namespace fq
