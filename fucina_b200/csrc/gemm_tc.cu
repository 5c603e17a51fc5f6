// Prefill-shaped quantized GEMM on the 5th-generation tensor cores.
//
// c[t, j] = sum_e bf16(a[t, e]) * bf16(dequant(W)[j, e]), f32 accumulate, for
// m > 16 token rows (reference role: fucina_mul_mm_mma_*, src/backend/cuda/
// kernels.cu:302-427, which rounds both operands to f16 and uses wmma). The
// dequantised weight follows the CPU decoders' formula (q4_k.zig:1954-1972,
// q5_k.zig:1154-1167, q8k.zig:95-114) evaluated with one fused multiply-add per
// weight and rounded to bf16: it equals the bf16 rounding of the reference's
// unfused f32 value except where that value lies within ~2^-20 (relative) of a
// bf16 rounding boundary, about one weight in two thousand, and then by one bf16
// ulp. Results differ from the f64 reference over bf16-rounded operands by that
// and by f32 accumulation.
//
// One persistent CTA per SM walks output tiles of 128 weight rows x TN tokens (TN = 256, or 128 for small
// batches and short expert runs) in K slabs of 64.
//   warp 0        copy-engine producer: TN x 64 bf16 token tiles (128-byte swizzle) into a 5-stage
//                 shared-memory ring
//   warp 14       copy-engine producer of the packed K-quant blocks of the tile's 128 rows (one
//                 256-weight unit = four slabs at a time) into a ring of its own (2 or 4 units), so
//                 weight fetches are not held back by the token ring's pace
//   warp 1        one thread issues tcgen05.mma (M=128 weight rows, N = the tile's tokens rounded up to
//                 16, K=16 per instruction, bf16 x bf16 -> f32): the A operand is read from TENSOR
//                 memory, the B operand through a shared-memory descriptor; the accumulator lives in
//                 256 TMEM columns (one of 256 tokens, or two of 128 that alternate between tiles so the
//                 epilogue of one tile runs under the MMAs of the next); tcgen05.commit releases a ring
//                 stage and signals the epilogue
//   warps 2..9    dequantise: two threads per weight row expand 64 weights of the current slab and
//                 store them with tcgen05.st into the A ring in tensor memory (32 columns per
//                 stage, next to the accumulator): the dequantised weights never touch shared
//                 memory, whose bandwidth the token tiles need
//   warps 10..13  epilogue: read the finished accumulator with tcgen05.ld and store f32 results
//                 (coalesced along n)
// A stage has one "full" barrier (copy-engine bytes + one arrival per dequantising warp) and one "empty"
// barrier (the MMAs' commit), so the issuing thread waits once and commits once per slab.
// Gated form (MoE gate/up pair, 128-token tiles): every tile makes two passes over K, gate weights into the
// first accumulator and up weights into the second; the epilogue of the gate pass parks gate * sigmoid(gate)
// in shared memory while the up pass multiplies, the epilogue of the up pass writes bf16(up * that).
// Every mbarrier wait is bounded and also watches a CTA-wide abort flag; a wait that gives up sets
// FQ_ERR_TIMEOUT in the status word, all roles fall through to the common exit, TMEM is freed.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdlib>
#include <cstring>

#include "internal.h"
#include "runtime.h"

namespace fq {

namespace {

#ifndef FQ_TC_DEQUANT_WARPS
#define FQ_TC_DEQUANT_WARPS 8  // 16 measured 4 % slower on dense and expert shapes alike: expansion is not the limit
#endif
constexpr int BM = 128;        // weight rows per tile (UMMA M)
// Tokens per tile (UMMA N) is a kernel parameter TN: 256 with one accumulator (dense prefill, long expert
// runs) or 128 with two accumulators that alternate between tiles, so the epilogue of one tile runs under
// the MMAs of the next (short expert runs, small batches). A ragged last tile multiplies only the tokens it
// has, rounded up to 16: the instruction's N is a run-time field.
constexpr int BK = 64;         // K elements per ring stage (128 bytes of bf16: one swizzle span)
// One ring of K slabs: stage s holds the token tile in shared memory and the dequantised weight slab in
// tensor memory (32 columns = 64 bf16 along K per lane). One "full" barrier per stage collects the copy
// engine's bytes and the eight dequantising warps, one "empty" barrier is signalled by the MMAs'
// commit: the single issuing thread waits once and commits once per slab, which is what bounds its rate.
constexpr int STAGES = 5;
// Ring of packed K-quant units (one unit = 256 weights of 128 rows = four K slabs), filled by a copy-engine
// producer of its own so that weight fetches run ahead of the token ring: as deep as shared memory allows.
constexpr int kMaxRawStages = 4;
constexpr int kGatedRawStages = 3;        // the gated form gives 64 KB of shared memory to the parked gate values
constexpr int kGateBytes = 128 * BM * 4;  // 128 tokens x 128 rows of f32
template <int TN>
struct RawRing {
    static constexpr int stages = TN == 128 ? 4 : 2;
};
constexpr int kAccCols = 256;  // tensor-memory columns of the f32 accumulator(s): one of 256 tokens or two of 128
// K-quant blocks are staged in shared memory by the copy engine (their 144/176 bytes are 16-byte
// multiples); Q8_0's split rows are read by the dequantising threads themselves.
template <int FMT>
struct Staged {
    static constexpr bool on = FMT == FQ_Q4_K || FMT == FQ_Q5_K;
    static constexpr int unit_bytes = FMT == FQ_Q4_K ? 144 : FMT == FQ_Q5_K ? 176 : 0;
    static constexpr int raw_bytes = BM * unit_bytes;
};
constexpr int kRawWarp = 2 + FQ_TC_DEQUANT_WARPS + 4;  // the warp after the epilogue warps: its lane 0 fetches packed weights
// Dequantising warps: a warp reaches one tensor-memory lane quarter (32 weight rows); eight warps cover the
// four quarters x the two 32-weight halves of a slab, and each further group of eight takes every
// kSlabSplit-th slab, so more slabs are expanded at once.
constexpr int kDequantWarps = FQ_TC_DEQUANT_WARPS;
constexpr int kSlabSplit = kDequantWarps / 8;
static_assert(kDequantWarps == 8 || kDequantWarps == 16, "8 or 16 dequantising warps");
constexpr int kEpilogueWarps = 4;  // one per tensor-memory lane quarter (eight, splitting the columns, measured no faster)
constexpr int kThreads = (3 + kDequantWarps + kEpilogueWarps) * 32;
constexpr unsigned kWaitLimit = 1u << 20;
#ifndef FQ_TC_SLEEP_NS
#define FQ_TC_SLEEP_NS 100
#endif
constexpr unsigned kProducerSleepNs = FQ_TC_SLEEP_NS;      // copy-engine producers waiting for a free ring stage
constexpr unsigned kEpilogueSleepNs = 2 * FQ_TC_SLEEP_NS;  // epilogue warps waiting for a finished accumulator
constexpr int TMEM_COLS = 512;  // columns 0..255: the f32 accumulator; from column 256: the A ring (STAGES x 32)
constexpr int A_COLS = BK / 2;  // tensor-memory columns of one A slab: two bf16 per 32-bit column
constexpr int A_COL0 = kAccCols;

struct TcArgs {
    DevWeights w;
    int mat;
    float* c;
    int m;    // tokens (dense) / rows of the sorted pair list (grouped)
    int ldc;
    int* status;
    // grouped form (MoE): a device-built list of output tiles, each naming its expert matrix, its
    // 128-row weight tile and the run of consecutive activation rows it multiplies
    const TcTile* table;
    const int* n_tiles_dev;
    int diag;  // diagnosis only (results are garbage): 1 = token tiles are not fetched, 2 = weights are not expanded
    // gated form (MoE gate/up pair, 128-token tiles): every tile multiplies the same rows of `w` (gate, first
    // accumulator) and `w2` (up, second accumulator); the epilogue writes bf16(up * silu(gate)) to g_out
    DevWeights w2;
    __nv_bfloat16* g_out;
    TcPeer peer;  // multi-GPU hooks (all null / zero on one GPU)
    int gated_op; // FQ_GATED_* of the gated form
    unsigned sleep_ns;  // pause between polls of the roles that wait off the critical path (see mbar_wait)
    // dense form, split-K tail: the tiles from `split_from` on (the last, partly filled wave of the persistent grid) are
    // cut along K into `split_parts` work items each, so that wave runs on every SM for 1/split_parts of a tile's time.
    // A part writes its f32 tile to partial[item - split_from][token][row]; splitk_reduce_kernel adds the parts in order.
    int split_from;   // = number of tiles when nothing is split
    int split_parts;  // a divisor of k / 256
    float* partial;
};

// One output tile: weight rows [rt*128, +128) of matrix `mat` times activation rows [tok0, tok0+ntok).
struct TileRef {
    int mat, rt, tok0, ntok;
    int u0, u1;  // the 256-weight units of K this work item multiplies (all of them unless it is a split-K part)
    int slot;    // -1, or the item's slot in TcArgs.partial
};
// Work item -> tile. Dense items below split_from are whole tiles; from there on, split_parts consecutive items share a tile.
template <int TN>
__device__ __forceinline__ TileRef tile_ref(const TcArgs& A, int item, int row_tiles, int units) {
    if (A.table) {
        const TcTile t = A.table[item];
        return {t.mat, t.rt, t.tok0, t.ntok, 0, units, -1};
    }
    int tile = item, u0 = 0, u1 = units, slot = -1;
    if (item >= A.split_from) {
        slot = item - A.split_from;
        tile = A.split_from + slot / A.split_parts;
        const int upp = units / A.split_parts;
        u0 = (slot % A.split_parts) * upp;
        u1 = u0 + upp;
    }
    const int tt = tile / row_tiles;  // consecutive CTAs share the token tile (L2 reuse) and take different weight rows
    return {A.mat, tile % row_tiles, tt * TN, min(TN, A.m - tt * TN), u0, u1, slot};
}

// Diagnostic build only (-DFQ_TIMELINE): the MMA thread of CTA 0 stamps, for the first slabs of its first tile,
// when it starts waiting for A, has A, has B, has issued the MMAs and has committed.
#ifdef FQ_TIMELINE
constexpr int kTlSlabs = 48;
__device__ unsigned long long g_tc_timeline[kTlSlabs * 5];
__device__ __forceinline__ unsigned long long tl_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");
    return t;
}
#define TL_STAMP(slab, what)                                                                          \
    do {                                                                                              \
        if (blockIdx.x == 0 && t == 0 && (slab) < kTlSlabs) g_tc_timeline[(slab) * 5 + (what)] = tl_now(); \
    } while (0)
// the first dequantising warp of CTA 0 stamps, for the slabs of its third tile: unit ready, slab loaded from
// shared memory, expanded, ring stage free, stored, barrier signalled
__device__ unsigned long long g_tc_timeline_dq[kTlSlabs * 6];
#define DQ_STAMP(slab, what)                                                                                             \
    do {                                                                                                                 \
        if (blockIdx.x == 0 && dq_tile == 2 && warp == 2 && lane == 0 && (slab) < kTlSlabs) g_tc_timeline_dq[(slab) * 6 + (what)] = tl_now(); \
    } while (0)
#else
#define TL_STAMP(slab, what) \
    do {                     \
    } while (0)
#define DQ_STAMP(slab, what) \
    do {                     \
    } while (0)
#endif

struct __align__(8) Barriers {
    uint64_t full[STAGES], empty[STAGES], raw_full[kMaxRawStages], raw_empty[kMaxRawStages], tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    volatile int abort_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// a flag another GPU writes: system-scope acquire, so the data it guards is visible once the value is seen
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
constexpr unsigned kPeerWaitLimit = 1u << 22;  // x ~0.2 us of sleep per poll: about a second
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// Bounded wait that also gives up when another role aborted. Returns false on abort/timeout.
// Roles that wait off the critical path (producers, epilogue) pass sleep_ns: a hot polling loop issues an
// instruction every few cycles and takes issue slots and the integer pipe from the dequantising warps.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, Barriers* B, int* status, unsigned sleep_ns = 0) {
    for (unsigned i = 0; i < kWaitLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (B->abort_flag) return false;
        if (sleep_ns) __nanosleep(sleep_ns);
    }
    B->abort_flag = 1;
    *(volatile int*)status = FQ_ERR_TIMEOUT;  // mapped host word: a plain store, device atomics on host memory are not portable
    return false;
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows of 128 bytes, 8-row groups
// 1024 bytes apart (stride byte offset), tile base 1024-byte aligned.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);       // start address
    d |= (uint64_t)1 << 16;                             // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                   // stride byte offset
    d |= (uint64_t)1 << 46;                             // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                             // SWIZZLE_128B
    return d;
}
// Instruction descriptor, kind::f16: D = f32, A = B = bf16, both K-major, M = 128, N = n_tokens (a multiple of 16, 16..256).
__device__ __forceinline__ uint32_t umma_idesc(int n_tokens) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n_tokens >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
// One MMA with A read from tensor memory (lane = row, 32-bit column = two consecutive bf16 along K) and B
// through a shared-memory descriptor.
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 consecutive 32-bit columns of this warp's tensor-memory lanes (asynchronous: tcgen05.wait::ld follows)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&acc)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(acc[0]), "=r"(acc[1]), "=r"(acc[2]), "=r"(acc[3]), "=r"(acc[4]), "=r"(acc[5]), "=r"(acc[6]), "=r"(acc[7]),
          "=r"(acc[8]), "=r"(acc[9]), "=r"(acc[10]), "=r"(acc[11]), "=r"(acc[12]), "=r"(acc[13]), "=r"(acc[14]), "=r"(acc[15]),
          "=r"(acc[16]), "=r"(acc[17]), "=r"(acc[18]), "=r"(acc[19]), "=r"(acc[20]), "=r"(acc[21]), "=r"(acc[22]), "=r"(acc[23]),
          "=r"(acc[24]), "=r"(acc[25]), "=r"(acc[26]), "=r"(acc[27]), "=r"(acc[28]), "=r"(acc[29]), "=r"(acc[30]), "=r"(acc[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// ---- packed weights of one 64-element K slab of one row: loaded one slab ahead, expanded later ----
template <int FMT>
struct Raw;

// Four byte-sized levels q0..q3 of one word -> bf16(a * (B + q) + c), packed two per word. Byte i is
// permuted straight into the mantissa of the f32 constant B, so no integer-to-float conversion is
// issued, and the multiply-adds run two per instruction. Levels below 128 (K-quants) use B = 128.0f
// (0x43000000 | q << 16 == 128 + q: mantissa bits 16..22); full bytes (Q8_0) use B = 32768.0f
// (0x47000000 | q << 8 == 32768 + q: mantissa bits 8..15).
template <bool FULL_BYTE>
__device__ __forceinline__ void expand_bytes(uint32_t v, float2 a2, float2 c2, uint32_t& out01, uint32_t& out23) {
    constexpr uint32_t base = FULL_BYTE ? 0x47000000u : 0x43000000u;
    constexpr uint32_t s0 = FULL_BYTE ? 0x7404 : 0x7044, s1 = FULL_BYTE ? 0x7414 : 0x7144, s2 = FULL_BYTE ? 0x7424 : 0x7244,
                       s3 = FULL_BYTE ? 0x7434 : 0x7344;
    const float2 x01 = make_float2(__uint_as_float(__byte_perm(v, base, s0)), __uint_as_float(__byte_perm(v, base, s1)));
    const float2 x23 = make_float2(__uint_as_float(__byte_perm(v, base, s2)), __uint_as_float(__byte_perm(v, base, s3)));
    const float2 w01 = __ffma2_rn(a2, x01, c2), w23 = __ffma2_rn(a2, x23, c2);
    out01 = pack_bf16(w01.x, w01.y);
    out23 = pack_bf16(w23.x, w23.y);
}

__device__ __forceinline__ void scale_min(const uint4& hdr, int s, int& sc, int& mn) {
    // K-quant 6-bit pair s from the 12 scale bytes in hdr.y/z/w (reference backend/quant/q8k.zig:637-648)
    const uint32_t s0 = hdr.y, s1 = hdr.z, s2 = hdr.w;
    if (s < 4) {
        sc = (s0 >> (8 * s)) & 63;
        mn = (s1 >> (8 * s)) & 63;
    } else {
        const int j = 8 * (s - 4);
        sc = ((s2 >> j) & 0xf) | (((s0 >> (j + 6)) & 3) << 4);
        mn = ((s2 >> (j + 4)) & 0xf) | (((s1 >> (j + 6)) & 3) << 4);
    }
}

template <>
struct Raw<FQ_Q4_K> {
    uint4 hdr, q0, q1;
    __device__ __forceinline__ void load(const DevWeights& w, const uint8_t* unit0, size_t ustride, int ks, int) {
        const uint8_t* b = unit0 + (size_t)(ks >> 2) * ustride;
        const int p = ks & 3;
        hdr = __ldg(reinterpret_cast<const uint4*>(b));
        q0 = __ldg(reinterpret_cast<const uint4*>(b + 16 + p * 32));
        q1 = __ldg(reinterpret_cast<const uint4*>(b + 32 + p * 32));
        if (p == 0 && (ks >> 2) + 1 < (w.k >> 8)) {  // pull the next block of this row towards the SM while this one is consumed
            asm volatile("prefetch.global.L2 [%0];" ::"l"(b + ustride));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(b + ustride + 128));
        }
    }
    // slab p (0..3) of the block staged at shared address `blk`
    __device__ __forceinline__ void load_header(uint32_t blk) { hdr = lds128(blk); }
    __device__ __forceinline__ void load_slab(uint32_t blk, int p) {
        q0 = lds128(blk + 16 + p * 32);
        q1 = lds128(blk + 32 + p * 32);
    }
    // w = d*sc*q - dmin*mn (q4_k.zig:1954-1972), rounded to bf16. No integer-to-float conversion:
    // the nibble is dropped into the mantissa of 128.0f (f32 0x43000000 | q << 16 == 128 + q exactly)
    // and one fused multiply-add per weight applies w = dsc * (128 + q) - (off + 128 * dsc).
    __device__ __forceinline__ void expand(int ks, int h, uint32_t out[16]) const {
        const int s = 2 * (ks & 3) + h;
        const __half2 dm = *reinterpret_cast<const __half2*>(&hdr.x);
        int sc, mn;
        scale_min(hdr, s, sc, mn);
        const float dsc = __fmul_rn(__low2float(dm), (float)sc), off = __fmul_rn(__high2float(dm), (float)mn);
        const float2 a2 = make_float2(dsc, dsc);
        const float cc = __fmaf_rn(dsc, -128.0f, -off);
        const float2 c2 = make_float2(cc, cc);
        const uint32_t wq[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t v = (h ? (wq[j] >> 4) : wq[j]) & 0x0f0f0f0fu;
            expand_bytes<false>(v, a2, c2, out[2 * j], out[2 * j + 1]);
        }
    }
};

template <>
struct Raw<FQ_Q5_K> {
    uint4 hdr, h0, h1, q0, q1;
    __device__ __forceinline__ void load(const DevWeights& w, const uint8_t* unit0, size_t ustride, int ks, int) {
        const uint8_t* b = unit0 + (size_t)(ks >> 2) * ustride;
        const int p = ks & 3;
        hdr = __ldg(reinterpret_cast<const uint4*>(b));
        h0 = __ldg(reinterpret_cast<const uint4*>(b + 16));
        h1 = __ldg(reinterpret_cast<const uint4*>(b + 32));
        q0 = __ldg(reinterpret_cast<const uint4*>(b + 48 + p * 32));
        q1 = __ldg(reinterpret_cast<const uint4*>(b + 64 + p * 32));
        if (p == 0 && (ks >> 2) + 1 < (w.k >> 8)) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(b + ustride));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(b + ustride + 128));
        }
    }
    __device__ __forceinline__ void load_header(uint32_t blk) {
        hdr = lds128(blk);
        h0 = lds128(blk + 16);
        h1 = lds128(blk + 32);
    }
    __device__ __forceinline__ void load_slab(uint32_t blk, int p) {
        q0 = lds128(blk + 48 + p * 32);
        q1 = lds128(blk + 64 + p * 32);
    }
    // as Q4_K with q = nibble + 16 * bit s of qh[i] (q5_k.zig:1154-1167, :1259-1264)
    __device__ __forceinline__ void expand(int ks, int h, uint32_t out[16]) const {
        const int s = 2 * (ks & 3) + h;
        const __half2 dm = *reinterpret_cast<const __half2*>(&hdr.x);
        int sc, mn;
        scale_min(hdr, s, sc, mn);
        const float dsc = __fmul_rn(__low2float(dm), (float)sc), off = __fmul_rn(__high2float(dm), (float)mn);
        const float2 a2 = make_float2(dsc, dsc);
        const float cc = __fmaf_rn(dsc, -128.0f, -off);
        const float2 c2 = make_float2(cc, cc);
        const uint32_t wq[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const uint32_t hb[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t nib = (h ? (wq[j] >> 4) : wq[j]) & 0x0f0f0f0fu;
            const uint32_t v = nib + ((hb[j] >> s) & 0x01010101u) * 16u;  // five-bit levels, one per byte
            expand_bytes<false>(v, a2, c2, out[2 * j], out[2 * j + 1]);
        }
    }
};

template <>
struct Raw<FQ_Q8_0> {
    uint4 q0, q1;
    float d;
    // row = [qs: K int8][d: K/32 f16]; one 32-weight block per (slab, half)
    __device__ __forceinline__ void load(const DevWeights& w, const uint8_t* unit0, size_t, int ks, int h) {
        const int blk = ks * 2 + h;
        q0 = __ldg(reinterpret_cast<const uint4*>(unit0 + (size_t)blk * 32));
        q1 = __ldg(reinterpret_cast<const uint4*>(unit0 + (size_t)blk * 32 + 16));
        d = h2f(__ldg(reinterpret_cast<const uint16_t*>(unit0 + w.k) + blk));
    }
    // f32(q) * d (q8k.zig:95-114), exactly: u = q + 128 goes into the mantissa of 32768.0f and
    // w = d * (32768 + u) - d * 32896 in one fused multiply-add (the constant term is exact in f32)
    __device__ __forceinline__ void load_header(uint32_t) {}
    __device__ __forceinline__ void load_slab(uint32_t, int) {}
    __device__ __forceinline__ void expand(int, int, uint32_t out[16]) const {
        const uint32_t wq[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const float2 a2 = make_float2(d, d);
        const float cc = __fmul_rn(d, -32896.0f);
        const float2 c2 = make_float2(cc, cc);
#pragma unroll
        for (int j = 0; j < 8; ++j) expand_bytes<true>(wq[j] ^ 0x80808080u, a2, c2, out[2 * j], out[2 * j + 1]);
    }
};

template <>
struct Raw<FQ_Q6_K> {
    uint4 q0, q1, h0, h1;
    float dsc0, dsc1;
    int nib, shift;
    // row = [per block: ql[128] qh[64] scales[16]][d: K/256 f16]. The 32 weights of (slab, half) are section
    // sec = 2*(slab & 1) + half of the 128-element half block c2 = (slab & 3) >> 1: low (sec < 2) or high nibbles of
    // ql[c2*64 + (sec & 1)*32 ..+32) with bits 2*sec, 2*sec+1 of qh[c2*32 ..+32) on top (q6_k.zig:1239-1259).
    __device__ __forceinline__ void load(const DevWeights& w, const uint8_t* unit0, size_t, int ks, int h) {
        const int blk = ks >> 2, p = ks & 3, c2 = p >> 1, sec = (p & 1) * 2 + h;
        const uint8_t* b = unit0 + (size_t)blk * 208;
        q0 = __ldg(reinterpret_cast<const uint4*>(b + c2 * 64 + h * 32));
        q1 = __ldg(reinterpret_cast<const uint4*>(b + c2 * 64 + h * 32 + 16));
        h0 = __ldg(reinterpret_cast<const uint4*>(b + 128 + c2 * 32));
        h1 = __ldg(reinterpret_cast<const uint4*>(b + 128 + c2 * 32 + 16));
        const uint16_t sc = __ldg(reinterpret_cast<const uint16_t*>(b + 192 + c2 * 8 + sec * 2));
        const float d = h2f(__ldg(reinterpret_cast<const uint16_t*>(unit0 + (size_t)(w.k >> 8) * 208) + blk));
        dsc0 = __fmul_rn(d, (float)(int8_t)(sc & 0xff));
        dsc1 = __fmul_rn(d, (float)(int8_t)(sc >> 8));
        nib = p & 1;
        shift = 2 * sec;
    }
    __device__ __forceinline__ void load_header(uint32_t) {}
    __device__ __forceinline__ void load_slab(uint32_t, int) {}
    // d * f32(scale) * f32(q6 - 32) (q6_k.zig:1159-1167), exactly: the level goes into the mantissa of 128.0f,
    // (128 + q6) - 160 is exact, and one rounded multiply by d*scale follows as in the reference
    __device__ __forceinline__ void expand(int, int, uint32_t out[16]) const {
        const uint32_t wq[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const uint32_t hb[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
        const float2 one = make_float2(1.0f, 1.0f), c160 = make_float2(-160.0f, -160.0f), zero = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t v = ((nib ? (wq[j] >> 4) : wq[j]) & 0x0f0f0f0fu) | (((hb[j] >> shift) & 0x03030303u) << 4);
            const float dsc = j < 4 ? dsc0 : dsc1;
            const float2 a2 = make_float2(dsc, dsc);
            const float2 x01 = make_float2(__uint_as_float(__byte_perm(v, 0x43000000u, 0x7044)), __uint_as_float(__byte_perm(v, 0x43000000u, 0x7144)));
            const float2 x23 = make_float2(__uint_as_float(__byte_perm(v, 0x43000000u, 0x7244)), __uint_as_float(__byte_perm(v, 0x43000000u, 0x7344)));
            const float2 w01 = __ffma2_rn(a2, __ffma2_rn(one, x01, c160), zero), w23 = __ffma2_rn(a2, __ffma2_rn(one, x23, c160), zero);
            out[2 * j] = pack_bf16(w01.x, w01.y);
            out[2 * j + 1] = pack_bf16(w23.x, w23.y);
        }
    }
};

template <>
struct Raw<FQ_TQ2_0> {
    uint4 q0, q1;
    float d;
    int shift;
    // row = [crumbs: K/4 bytes][d: K/256 f16]. Byte hg*32 + m of a 64-byte block holds elements
    // hg*128 + n*32 + m in crumb n (dtype.zig:215-218), so the 32 weights of one (slab, half) are crumb
    // n of 32 consecutive bytes.
    __device__ __forceinline__ void load(const DevWeights& w, const uint8_t* unit0, size_t, int ks, int h) {
        const int blk = ks >> 2, sub = (ks & 3) * 2 + h;  // eight 32-weight groups per block
        const uint8_t* p = unit0 + (size_t)blk * 64 + (sub >> 2) * 32;
        q0 = __ldg(reinterpret_cast<const uint4*>(p));
        q1 = __ldg(reinterpret_cast<const uint4*>(p + 16));
        d = h2f(__ldg(reinterpret_cast<const uint16_t*>(unit0 + (w.k >> 2)) + blk));
        shift = 2 * (sub & 3);
    }
    __device__ __forceinline__ void load_header(uint32_t) {}
    __device__ __forceinline__ void load_slab(uint32_t, int) {}
    // d * (code - 1), exactly (ternary.zig:850-876): d * (128 + code) - 129 * d in one fused multiply-add
    __device__ __forceinline__ void expand(int, int, uint32_t out[16]) const {
        const uint32_t wq[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const float2 a2 = make_float2(d, d);
        const float cc = __fmul_rn(d, -129.0f);
        const float2 c2 = make_float2(cc, cc);
#pragma unroll
        for (int j = 0; j < 8; ++j) expand_bytes<false>((wq[j] >> shift) & 0x03030303u, a2, c2, out[2 * j], out[2 * j + 1]);
    }
};

template <>
struct Raw<FQ_TQ2_0_FOLDED> {
    uint4 q;
    float d;
    // row = [nibbles: K/2 bytes][d: K/256 f16]. Sub-block s of a block is 16 bytes: low nibbles = its elements
    // 0..15, high nibbles = elements 16..31; value d * (cu - 4) (types.zig:177-180, ternary.zig:850-876).
    __device__ __forceinline__ void load(const DevWeights& w, const uint8_t* unit0, size_t, int ks, int h) {
        const int blk = ks >> 2, sub = (ks & 3) * 2 + h;
        q = __ldg(reinterpret_cast<const uint4*>(unit0 + (size_t)blk * 128 + sub * 16));
        d = h2f(__ldg(reinterpret_cast<const uint16_t*>(unit0 + (w.k >> 1)) + blk));
    }
    __device__ __forceinline__ void load_header(uint32_t) {}
    __device__ __forceinline__ void load_slab(uint32_t, int) {}
    __device__ __forceinline__ void expand(int, int, uint32_t out[16]) const {
        const uint32_t wq[4] = {q.x, q.y, q.z, q.w};
        const float2 a2 = make_float2(d, d);
        const float cc = __fmul_rn(d, -132.0f);  // d * (128 + cu) - 132 * d = d * (cu - 4), exact
        const float2 c2 = make_float2(cc, cc);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            expand_bytes<false>(wq[j] & 0x0f0f0f0fu, a2, c2, out[2 * j], out[2 * j + 1]);
            expand_bytes<false>((wq[j] >> 4) & 0x0f0f0f0fu, a2, c2, out[8 + 2 * j], out[8 + 2 * j + 1]);
        }
    }
};

template <>
struct Raw<FQ_Q2_0> {
    uint2 q;
    float d;
    // row = [crumbs: K/4 bytes][d: K/128 f16]. Element j of a 128-element group is crumb j % 4 of byte j / 4;
    // value d * (q - 1) (cold.zig:285-301).
    __device__ __forceinline__ void load(const DevWeights& w, const uint8_t* unit0, size_t, int ks, int h) {
        const int e0 = ks * 64 + h * 32;
        q = __ldg(reinterpret_cast<const uint2*>(unit0 + (e0 >> 2)));
        d = h2f(__ldg(reinterpret_cast<const uint16_t*>(unit0 + (w.k >> 2)) + (e0 >> 7)));
    }
    __device__ __forceinline__ void load_header(uint32_t) {}
    __device__ __forceinline__ void load_slab(uint32_t, int) {}
    // A byte holds four consecutive elements as crumbs 0..3. The byte is replicated into the four byte lanes of
    // a word and masked so that lane n keeps crumb n IN PLACE (bits 2n, 2n+1): dropped into the mantissa of
    // 128.0f this reads 128 + code * 4^n, and the scale d / 4^n with the offset -(128 / 4^n + 1) * d (all exact)
    // gives d * (code - 1). Crumb 3 would reach the exponent bit, so it is shifted down and treated like crumb 0.
    __device__ __forceinline__ void expand(int, int, uint32_t out[16]) const {
        const float2 a01 = make_float2(d, __fmul_rn(d, 0.25f)), a23 = make_float2(__fmul_rn(d, 0.0625f), d);
        const float2 c01 = make_float2(__fmul_rn(d, -129.0f), __fmul_rn(d, -33.0f));
        const float2 c23 = make_float2(__fmul_rn(d, -9.0f), __fmul_rn(d, -129.0f));
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t r = __byte_perm(j < 4 ? q.x : q.y, 0, 0x1111 * (j & 3));  // the byte in all four lanes
            const uint32_t m012 = r & 0x00300c03u, m3 = (r >> 6) & 0x03u;
            const float2 x01 = make_float2(__uint_as_float(__byte_perm(m012, 0x43000000u, 0x7044)),
                                           __uint_as_float(__byte_perm(m012, 0x43000000u, 0x7144)));
            const float2 x23 = make_float2(__uint_as_float(__byte_perm(m012, 0x43000000u, 0x7244)),
                                           __uint_as_float(__byte_perm(m3, 0x43000000u, 0x7044)));
            const float2 w01 = __ffma2_rn(a01, x01, c01), w23 = __ffma2_rn(a23, x23, c23);
            out[2 * j] = pack_bf16(w01.x, w01.y);
            out[2 * j + 1] = pack_bf16(w23.x, w23.y);
        }
    }
};

template <int FMT, int TN, bool GATED>
__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(const TcArgs A, const __grid_constant__ CUtensorMap tmap_tokens,
                                                              const __grid_constant__ CUtensorMap tmap_weights,
                                                              const __grid_constant__ CUtensorMap tmap_weights2) {
    static_assert(!GATED || TN == 128, "the gated form needs both accumulators of one tile");
    constexpr int PASSES = GATED ? 2 : 1;  // passes over K per tile: gate weights, then up weights
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte aligned rings: [B stages][packed-weight stages][barriers]; the dequantised A slabs live in tensor memory
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int B_BYTES = TN * BK * 2;   // one token tile of a K slab: 32 KB or 16 KB
    constexpr int NACC = kAccCols / TN;    // accumulators alternating between tiles
    constexpr int RAW_STAGES = GATED ? kGatedRawStages : RawRing<TN>::stages;
    uint8_t* sB = smem;
    uint8_t* sRaw = sB + STAGES * B_BYTES;
    // gated form: f32 gate * sigmoid(gate) of the tile, [token][row], parked between the two epilogues of a tile
    float* sG = reinterpret_cast<float*>(sRaw + RAW_STAGES * Staged<FMT>::raw_bytes);
    Barriers* B = reinterpret_cast<Barriers*>(reinterpret_cast<uint8_t*>(sG) + (GATED ? kGateBytes : 0));
    static_assert(A_COL0 + STAGES * A_COLS <= TMEM_COLS, "A ring does not fit the tensor memory");
    constexpr bool kStaged = Staged<FMT>::on;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = A.w.n, k = A.w.k, m = A.m;
    const int mat_rows = A.w.n_mats > 1 ? (int)(A.w.mat_stride / A.w.row_stride) : n;  // rows between stacked matrices (n when dense)
    const int kslabs = k / BK, units = k >> 8;
    const int row_tiles = (n + BM - 1) / BM, tok_tiles = (m + TN - 1) / TN;
    const int n_tiles = A.table ? *A.n_tiles_dev : A.split_from + (row_tiles * tok_tiles - A.split_from) * A.split_parts;  // work items

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&B->full[s]), 8 + 1);  // one arrival per warp that expands the slab + the producer's expect_tx arrival
            mbar_init(smem_u32(&B->empty[s]), 1);
        }
        for (int s = 0; s < kMaxRawStages; ++s) {
            mbar_init(smem_u32(&B->raw_full[s]), 1);
            mbar_init(smem_u32(&B->raw_empty[s]), kDequantWarps);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&B->tmem_full[a]), 1);
            mbar_init(smem_u32(&B->tmem_empty[a]), kEpilogueWarps);
        }
        B->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        // TMEM allocation by one full warp; the base address lands in shared memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&B->tmem_base)), "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = B->tmem_base;

    if (warp == 0) {
        // ---------------- copy-engine producer: token tiles ----------------
        if (lane == 0) {
            int gb = 0;
            bool ok = true;
            // expert parallelism: the token rows of this GPU's panel are written by other ranks; every source
            // posts a flag once its rows are visible. Bounded: a flag that never comes aborts the CTA.
            for (int i = 0; i < A.peer.n_wait && ok; ++i) {
                unsigned spins = 0;
                while (ld_acquire_sys(A.peer.wait_flags + i) < A.peer.wait_value) {
                    if (B->abort_flag || ++spins > kPeerWaitLimit) {
                        ok = false;
                        break;
                    }
                    __nanosleep(200);
                }
            }
            if (!ok) {
                B->abort_flag = 1;
                *(volatile int*)A.status = FQ_ERR_TIMEOUT;
            }
            for (int tile = blockIdx.x; tile < n_tiles && ok && !B->abort_flag; tile += gridDim.x) {
                const TileRef T = tile_ref<TN>(A, tile, row_tiles, units);
                for (int u = T.u0; u < (PASSES - 1) * units + T.u1 && ok; ++u) {
                    for (int p = 0; p < 4; ++p, ++gb) {
                        const int s = gb % STAGES;
                        if (!mbar_wait(smem_u32(&B->empty[s]), ((gb / STAGES) & 1) ^ 1, B, A.status, A.sleep_ns)) {
                            ok = false;
                            break;
                        }
                        const uint32_t bar = smem_u32(&B->full[s]);
                        if (A.diag == 1) {
                            mbar_arrive(bar);
                            continue;
                        }
                        mbar_arrive_expect_tx(bar, B_BYTES);
                        asm volatile(
                            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                                smem_u32(sB + s * B_BYTES)),
                            "l"(&tmap_tokens), "r"(((u % units) * 4 + p) * BK), "r"(T.tok0), "r"(bar)
                            : "memory");
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int g = 0, t = 0;
            for (int tile = blockIdx.x; tile < n_tiles && !B->abort_flag; tile += gridDim.x, ++t) {
                // the epilogue of the tile that used this accumulator before must have drained it
                // (gated form: the gate pass of a tile fills the first accumulator, the up pass the second)
                const int ai = t % NACC;
                if (!GATED && !mbar_wait(smem_u32(&B->tmem_empty[ai]), ((t / NACC) & 1) ^ 1, B, A.status)) break;
                const TileRef T = tile_ref<TN>(A, tile, row_tiles, units);
                const uint32_t idesc = umma_idesc(min(TN, (T.ntok + 15) & ~15));
                const int ks0 = GATED ? 0 : 4 * T.u0, ks1 = GATED ? kslabs : 4 * T.u1;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                bool ok = true;
                for (int ps = 0; ps < PASSES && ok; ++ps) {
                const int aj = GATED ? ps : ai;
                if (GATED && !mbar_wait(smem_u32(&B->tmem_empty[aj]), (t & 1) ^ 1, B, A.status)) {
                    ok = false;
                    break;
                }
                if (GATED) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem + (uint32_t)(aj * TN);
                for (int ks = ks0; ks < ks1; ++ks, ++g) {
                    const int sa = g % STAGES, sb = sa;
                    TL_STAMP(ks, 0);
                    if (!mbar_wait(smem_u32(&B->full[sa]), (g / STAGES) & 1, B, A.status)) {
                        ok = false;
                        break;
                    }
                    TL_STAMP(ks, 2);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t ta = tmem + (uint32_t)(A_COL0 + sa * A_COLS);
                    const uint64_t db = umma_desc(smem_u32(sB + sb * B_BYTES));
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk)  // 16 elements along K per instruction: 8 columns of A, 32 bytes of B
                        umma_bf16_ts(acc, ta + 8 * kk, db + 2 * kk, idesc, ((ks - ks0) | kk) ? 1u : 0u);
                    TL_STAMP(ks, 3);
                    umma_commit(smem_u32(&B->empty[sa]));  // the stage is free once these MMAs have read it
                    TL_STAMP(ks, 4);
                }
                if (ok) umma_commit(smem_u32(&B->tmem_full[aj]));
                }
                if (!ok) break;
            }
        }
    } else if (warp < 2 + kDequantWarps) {
        // ---------------- dequantise ----------------
        // a warp reaches the tensor-memory lanes 32 * (warp % 4) .. +31 only: that fixes its rows; the two warps
        // of a lane quarter take the two 32-weight halves of the 64-element slab
        const int r = 32 * (warp & 3) + lane;  // weight row inside the tile = tensor-memory lane
        const int h = ((warp - 2) >> 2) & 1;
        const int par = (warp - 2) >> 3;  // this warp expands the slabs ks with ks % kSlabSplit == par
        constexpr int ub = FMT == FQ_Q4_K ? 144 : FMT == FQ_Q5_K ? 176 : 256;
        const size_t ustride = unit_stride(A.w, ub);
        int gbase = 0, gu = 0;  // slabs of the tiles before this one; units consumed
        int dq_tile = 0;        // tiles this CTA has started (diagnostic stamps only)
        bool ok = true;
        // one slab of this row goes to A stage (ga % STAGES) in tensor memory: lane r, 16 columns from h * 16
        // (awaiting the store only after the next slab's expansion was measured slightly slower)
        auto publish = [&](const uint32_t (&v)[16], int ga) -> bool {
            const int s = ga % STAGES;
            if (!mbar_wait(smem_u32(&B->empty[s]), ((ga / STAGES) & 1) ^ 1, B, A.status)) return false;
            DQ_STAMP(ga - gbase, 3);
            __syncwarp();  // the store below is a warp-wide (.aligned) instruction
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(A_COL0 + s * A_COLS + h * 16);
            asm volatile(
                "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
                "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
                "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
                : "memory");
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            DQ_STAMP(ga - gbase, 4);
            __syncwarp();  // every lane's store has completed: one arrival for the warp (arrivals on one barrier serialise)
            if (lane == 0) mbar_arrive(smem_u32(&B->full[s]));
            DQ_STAMP(ga - gbase, 5);
            return true;
        };
        for (int tile = blockIdx.x; tile < n_tiles && ok && !B->abort_flag; tile += gridDim.x) {
            const TileRef T = tile_ref<TN>(A, tile, row_tiles, units);
            for (int ps = 0; ps < PASSES && ok; ++ps) {
            const DevWeights& W = (GATED && ps) ? A.w2 : A.w;
            if (kStaged) {
                for (int u = T.u0; u < T.u1 && ok; ++u, ++gu) {
                    const int rs = gu % RAW_STAGES;
                    if (!mbar_wait(smem_u32(&B->raw_full[rs]), (gu / RAW_STAGES) & 1, B, A.status)) {
                        ok = false;
                        break;
                    }
                    // this row's block: lanes are 144/176 bytes apart, an odd number of 16-byte chunks, so the
                    // 128-bit shared loads of a quarter warp fall on distinct banks
                    const uint32_t blk = smem_u32(sRaw + rs * Staged<FMT>::raw_bytes) + (uint32_t)r * Staged<FMT>::unit_bytes;
                    Raw<FMT> raw;
                    raw.load_header(blk);
#pragma unroll
                    for (int p0 = 0; p0 < 4; p0 += kSlabSplit) {
                        const int p = p0 + par;
                        DQ_STAMP(4 * u + p, 0);
                        raw.load_slab(blk, p);
                        DQ_STAMP(4 * u + p, 1);
                        uint32_t v[16];
                        if (A.diag == 2) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) v[i] = 0x3c003c00u;
                        } else {
                            raw.expand(p, h, v);
                        }
                        DQ_STAMP(4 * u + p, 2);
                        if (!(ok = publish(v, gbase + 4 * (u - T.u0) + p))) break;
                    }
                    // the loads above have returned (their values went into the stores): the unit may be overwritten
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&B->raw_empty[rs]));
                }
            } else {
                const uint8_t* wbase = W.base + (size_t)T.mat * W.mat_stride;
                const int row = min(T.rt * BM + r, n - 1);
                const uint8_t* unit0 = row_unit0(W, wbase, row, ub);
                Raw<FMT> next;
                const int ks0 = 4 * T.u0, ks1 = 4 * T.u1;
                next.load(W, unit0, ustride, ks0 + par, h);
                for (int ks = ks0 + par; ks < ks1; ks += kSlabSplit) {
                    const Raw<FMT> cur = next;
                    if (ks + kSlabSplit < ks1) next.load(W, unit0, ustride, ks + kSlabSplit, h);  // one slab ahead: the loads fly while this slab is expanded
                    uint32_t v[16];
                    cur.expand(ks, h, v);
                    if (!(ok = publish(v, gbase + ks - ks0))) break;
                }
            }
            gbase += 4 * (T.u1 - T.u0);
            }
            ++dq_tile;
        }
    } else if (warp == kRawWarp) {
        // ---------------- copy-engine producer: packed weight units (K-quants) ----------------
        // its own thread, so the weight ring runs ahead of the token ring by as many units as it holds
        if (kStaged && lane == 0) {
            constexpr int ub = Staged<FMT>::unit_bytes;
            int gu = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok && !B->abort_flag; tile += gridDim.x) {
                const TileRef T = tile_ref<TN>(A, tile, row_tiles, units);
                for (int ps = 0; ps < PASSES && ok; ++ps) {
                const DevWeights& W = (GATED && ps) ? A.w2 : A.w;
                const CUtensorMap* tmw = (GATED && ps) ? &tmap_weights2 : &tmap_weights;
                for (int u = T.u0; u < T.u1; ++u, ++gu) {
                    const int rs = gu % RAW_STAGES;
                    if (!mbar_wait(smem_u32(&B->raw_empty[rs]), ((gu / RAW_STAGES) & 1) ^ 1, B, A.status, A.sleep_ns)) {
                        ok = false;
                        break;
                    }
                    const uint32_t bar = smem_u32(&B->raw_full[rs]);
                    const uint32_t dst = smem_u32(sRaw + rs * Staged<FMT>::raw_bytes);
                    if (W.tile_rows) {
                        // tile-major storage: unit u of 32 consecutive rows is one contiguous run
                        const int n_store = (n + 31) >> 5;
                        const int valid = min(BM / 32, n_store - T.rt * (BM / 32));
                        mbar_arrive_expect_tx(bar, (uint32_t)(valid * 32 * ub));
                        const uint8_t* wbase = W.base + (size_t)T.mat * W.mat_stride;
                        for (int j = 0; j < valid; ++j)
                            bulk_load(dst + j * 32 * ub, wbase + (size_t)(T.rt * (BM / 32) + j) * ((size_t)32 * W.row_stride) + (size_t)u * 32 * ub,
                                      32 * ub, bar);
                    } else {
                        // row-major storage: a box of 128 rows x one unit; rows past the end of the tensor arrive as zeros
                        mbar_arrive_expect_tx(bar, (uint32_t)(BM * ub));
                        asm volatile(
                            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                            "l"(tmw), "r"(u * ub), "r"(T.mat * mat_rows + T.rt * BM), "r"(bar)
                            : "memory");
                    }
                }
                }
            }
        }
    } else {
        // ---------------- epilogue: accumulator lane = weight row, column = token ----------------
        int t = 0;
        for (int tile = blockIdx.x; tile < n_tiles && !B->abort_flag; tile += gridDim.x, ++t) {
            const TileRef T = tile_ref<TN>(A, tile, row_tiles, units);
            const int rt = T.rt;
            const int q = warp & 3;                       // TMEM lane quarter this warp may read
            const int out_row = rt * BM + q * 32 + lane;  // weight row = output column
            // a split-K part stores its whole f32 tile, [token][row], into its slot of the partial buffer
            float* const dst = T.slot >= 0 ? A.partial + (size_t)T.slot * TN * BM + q * 32 + lane : A.c + (size_t)T.tok0 * A.ldc + out_row;
            const size_t dst_ld = T.slot >= 0 ? (size_t)BM : (size_t)A.ldc;
            bool ok = true;
            for (int ps = 0; ps < PASSES; ++ps) {
                const int ai = GATED ? ps : t % NACC;
                if (!mbar_wait(smem_u32(&B->tmem_full[ai]), (GATED ? t : t / NACC) & 1, B, A.status, 2 * A.sleep_ns)) {
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int c0 = 0; c0 < TN; c0 += 32) {
                    if (c0 >= T.ntok) break;  // warp-uniform: columns past the tile's tokens were not multiplied
                    uint32_t acc[32];
                    tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(ai * TN + c0), acc);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (GATED) {
                        // g = up * (gate * 1/(1+exp(-gate))) in f32 (backend/ops.zig:150-190), rounded once to bf16.
                        // The gate pass parks gate * sigmoid(gate) in shared memory (each thread re-reads only what
                        // it wrote) while the MMAs of the up pass run; the up pass finishes the product.
                        float* mine = sG + (size_t)c0 * BM + q * 32 + lane;
                        // swiglu, the common op, keeps a loop of its own: the five-way switch inside the unrolled loop
                        // made this epilogue long enough to stall the up pass behind it
                        if (ps == 0) {
                            if (A.gated_op == FQ_GATED_SWIGLU) {
#pragma unroll
                                for (int j = 0; j < 32; ++j) {
                                    const float gv = __uint_as_float(acc[j]);
                                    const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-gv)));
                                    mine[j * BM] = __fmul_rn(gv, sig);
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; ++j) mine[j * BM] = gated_activation(A.gated_op, __uint_as_float(acc[j]));
                            }
                        } else if (out_row < n) {
                            if (A.gated_op == FQ_GATED_SWIGLU) {
#pragma unroll
                                for (int j = 0; j < 32; ++j) {
                                    if (c0 + j < T.ntok)
                                        A.g_out[(size_t)(T.tok0 + c0 + j) * A.ldc + out_row] =
                                            __float2bfloat16_rn(__fmul_rn(__uint_as_float(acc[j]), mine[j * BM]));
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; ++j) {
                                    if (c0 + j < T.ntok)
                                        A.g_out[(size_t)(T.tok0 + c0 + j) * A.ldc + out_row] =
                                            __float2bfloat16_rn(__fmul_rn(gated_source(A.gated_op, __uint_as_float(acc[j])), mine[j * BM]));
                                }
                            }
                        }
                    } else if (out_row < n) {
                        if (A.peer.row_meta) {
                            // every row goes to the panel of the rank that owns its token: lanes hold consecutive
                            // columns of one row, so a warp writes 128 contiguous bytes per row (plain peer stores)
#pragma unroll 8
                            for (int j = 0; j < 32; ++j) {
                                if (c0 + j < T.ntok) {
                                    const int2 mt = __ldg(A.peer.row_meta + T.tok0 + c0 + j);
                                    A.peer.dst_base[mt.x & (kMaxPeers - 1)][(size_t)mt.y * A.ldc + out_row] = __uint_as_float(acc[j]);
                                }
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (c0 + j < T.ntok) dst[(size_t)(c0 + j) * dst_ld] = __uint_as_float(acc[j]);
                            }
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&B->tmem_empty[ai]));
            }
            if (!ok) break;
        }
        if (A.peer.row_meta) __threadfence_system();  // this thread's peer stores are visible system-wide before the CTA reports
    }

    // common exit: everyone meets here (also after an abort), then the allocating warp frees TMEM
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (A.peer.n_signal && threadIdx.x == 32) {
        // the last CTA to finish tells the peers that every result row of this product is in their panels
        __threadfence_system();
        if (atomicAdd(A.peer.done_counter, 1) == (int)gridDim.x - 1) {
            __threadfence_system();
            for (int i = 0; i < A.peer.n_signal; ++i)
                asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(A.peer.signal_flag[i]), "r"(A.peer.signal_value) : "memory");
        }
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// Adds the split-K parts of the tail tiles in part order: c[token][row] = partial[0] + partial[1] + ...
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, float* __restrict__ c, int ldc, int n, int m, int row_tiles,
                                     int split_from, int parts, int tail_tiles, int tn) {
    const size_t per_tile = (size_t)tn * BM, total = (size_t)tail_tiles * per_tile;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(idx / per_tile);
        const int rem = (int)(idx % per_tile), tok = rem / BM, row = rem % BM;
        const int tile = split_from + r, gtok = (tile / row_tiles) * tn + tok, grow = (tile % row_tiles) * BM + row;
        if (gtok >= m || grow >= n) continue;
        const float* p = partial + ((size_t)r * parts * tn + tok) * BM + row;
        float sum = p[0];
        for (int i = 1; i < parts; ++i) sum = __fadd_rn(sum, p[(size_t)i * per_tile]);
        c[(size_t)gtok * ldc + grow] = sum;
    }
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n) {
    for (size_t i = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) * 4; i < n; i += (size_t)gridDim.x * blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(src + i);
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&lo);
        o.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst + i) = o;
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
        cudaGetLastError();
    }
    return fn;
}

template <int FMT, int TN, bool GATED = false>
cudaError_t launch_tc_tn(const TcArgs& a, const CUtensorMap& tmap, const CUtensorMap& tmap_w, const CUtensorMap& tmap_w2, int grid, cudaStream_t st) {
    const size_t smem = (size_t)STAGES * TN * BK * 2 + (size_t)(GATED ? kGatedRawStages : RawRing<TN>::stages) * Staged<FMT>::raw_bytes +
                        (GATED ? kGateBytes : 0) + sizeof(Barriers) + 1024;
    static bool granted = false;
    if (!granted) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<FMT, TN, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        granted = true;
    }
    gemm_tc_kernel<FMT, TN, GATED><<<grid, kThreads, smem, st>>>(a, tmap, tmap_w, tmap_w2);
    return cudaGetLastError();
}
template <int FMT>
cudaError_t launch_tc(const TcArgs& a, const CUtensorMap& tmap, const CUtensorMap& tmap_w, int grid, int tile_tokens, cudaStream_t st) {
    return tile_tokens == 128 ? launch_tc_tn<FMT, 128>(a, tmap, tmap_w, tmap_w, grid, st) : launch_tc_tn<FMT, 256>(a, tmap, tmap_w, tmap_w, grid, st);
}

#ifdef FQ_TIMELINE
extern "C" __attribute__((visibility("default"))) int fq_debug_tc_timeline(unsigned long long* out) {
    return (int)cudaMemcpyFromSymbol(out, g_tc_timeline, sizeof(unsigned long long) * kTlSlabs * 5);
}
extern "C" __attribute__((visibility("default"))) int fq_debug_tc_timeline_dq(unsigned long long* out) {
    return (int)cudaMemcpyFromSymbol(out, g_tc_timeline_dq, sizeof(unsigned long long) * kTlSlabs * 6);
}
#endif

}  // namespace

bool tensor_path_serves(const DevWeights& w) {
    return (w.fmt == FQ_Q4_K || w.fmt == FQ_Q5_K || w.fmt == FQ_Q6_K || w.fmt == FQ_Q8_0 || w.fmt == FQ_TQ2_0 || w.fmt == FQ_TQ2_0_FOLDED ||
            w.fmt == FQ_Q2_0) &&
           w.k % 256 == 0 && encode_fn() != nullptr;
}

// Launch over bf16 activation rows [rows][k]: dense tiles of matrix `mat` (table == nullptr) or a
// device-built tile list (grouped MoE form; `max_tiles` bounds the list for the grid size, and
// `tile_tokens`, 128 or 256, is the token width its entries were cut to).
// Tensor map over packed K-quant rows stored row-major (expert stacks, small matrices): all stacked matrices as
// one 2-D byte array, one box = one 256-weight unit of 128 rows. Other layouts and formats need none (zeroed map).
static int encode_packed_rows(EncodeTiledFn enc, const DevWeights& w, CUtensorMap* out) {
    memset(out, 0, sizeof *out);
    if (!((w.fmt == FQ_Q4_K || w.fmt == FQ_Q5_K) && !w.tile_rows)) return FQ_OK;
    const int ub = w.fmt == FQ_Q4_K ? 144 : 176;
    if (w.n_mats > 1 && (w.mat_stride % w.row_stride != 0 || w.mat_stride < (size_t)w.n * w.row_stride))
        return fail(FQ_DECLINED_ARGS, "stacked matrices are not a whole number of rows apart");
    if (((uintptr_t)w.base & 15) || (w.row_stride & 15)) return fail(FQ_DECLINED_ARGS, "packed rows are not 16-byte aligned");
    const cuuint64_t mat_rows = w.n_mats > 1 ? w.mat_stride / w.row_stride : (cuuint64_t)w.n;
    const cuuint64_t wdims[2] = {(cuuint64_t)(w.k / 256) * ub, mat_rows * (cuuint64_t)(w.n_mats - 1) + (cuuint64_t)w.n};
    const cuuint64_t wstrides[1] = {(cuuint64_t)w.row_stride};
    const cuuint32_t wbox[2] = {(cuuint32_t)ub, BM};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(w.base), wdims, wstrides, wbox, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return fail(FQ_DECLINED_ARGS, "tensor map for the packed weights could not be encoded");
    return FQ_OK;
}

// `up` and `g_out` select the gated form (grouped, 128-token tiles): w is the gate stack, the result is
// bf16(up * silu(gate)) in g_out instead of f32 products in c_dev.
static int launch_tc_rows(Ctx* ctx, const DevWeights& w, int mat, const __nv_bfloat16* abf, size_t rows, float* c_dev, size_t ldc,
                          const TcTile* table, const int* n_tiles_dev, int max_tiles, int tile_tokens, cudaStream_t st,
                          const DevWeights* up = nullptr, __nv_bfloat16* g_out = nullptr, const TcPeer* peer = nullptr, int gated_op = 0) {
    const int BN = tile_tokens;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return fail(FQ_DECLINED_ARGS, "cuTensorMapEncodeTiled unavailable");
    CUtensorMap tmap;
    memset(&tmap, 0, sizeof tmap);
    const cuuint64_t dims[2] = {(cuuint64_t)w.k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)w.k * 2};
    const cuuint32_t box[2] = {BK, (cuuint32_t)BN};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(abf), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return fail(FQ_DECLINED_ARGS, "tensor map for the activations could not be encoded");
    CUtensorMap tmap_w, tmap_w2;
    if (int rc = encode_packed_rows(enc, w, &tmap_w)) return rc;
    if (int rc = encode_packed_rows(enc, up ? *up : w, &tmap_w2)) return rc;
    static const int diag = getenv("FUCINA_B200_TC_DIAG") ? atoi(getenv("FUCINA_B200_TC_DIAG")) : 0;
    static const unsigned sleep_ns = getenv("FUCINA_B200_TC_SLEEP_NS") ? (unsigned)atoi(getenv("FUCINA_B200_TC_SLEEP_NS")) : kProducerSleepNs;
    const int tiles = table ? max_tiles : ((w.n + BM - 1) / BM) * (int)((rows + BN - 1) / BN);
    const int grid = tiles < ctx->sm_count ? (tiles > 0 ? tiles : 1) : ctx->sm_count;
    TcArgs a{w, mat, c_dev, (int)rows, (int)ldc, ctx->status_dev, table, n_tiles_dev, diag, up ? *up : w, g_out, peer ? *peer : TcPeer{}, gated_op, sleep_ns,
             tiles, 1, nullptr};
    // Dense products of several waves whose last wave fills at most half the SMs: that wave's tiles are cut along K
    // into as many parts as fit the grid (a power of two, at least two 256-weight units each), see TcArgs.
    static const bool no_split = getenv("FUCINA_B200_TC_NO_SPLITK") != nullptr;
    const int tail = tiles % grid, units = w.k / 256;
    int parts = 1;
    if (!table && !up && !no_split && tile_tokens == 256 && tiles > grid && tail > 0)
        while (parts * 2 * tail <= grid && units % (parts * 2) == 0 && units / (parts * 2) >= 2) parts *= 2;
    float* partial = nullptr;
    if (parts > 1) {
        partial = (float*)dev_alloc_on((size_t)tail * parts * 256 * BM * sizeof(float), st);
        if (partial) a.split_from = tiles - tail, a.split_parts = parts, a.partial = partial;
        else parts = 1;
    }
    struct FreePartial {
        float* p;
        cudaStream_t st;
        ~FreePartial() { if (p) dev_free_on(p, st); }
    } free_partial{partial, st};
    cudaError_t e;
    if (up) {  // gated form: the formats expert stacks come in
        switch (w.fmt) {
            case FQ_Q4_K: e = launch_tc_tn<FQ_Q4_K, 128, true>(a, tmap, tmap_w, tmap_w2, grid, st); break;
            case FQ_Q5_K: e = launch_tc_tn<FQ_Q5_K, 128, true>(a, tmap, tmap_w, tmap_w2, grid, st); break;
            case FQ_Q6_K: e = launch_tc_tn<FQ_Q6_K, 128, true>(a, tmap, tmap_w, tmap_w2, grid, st); break;
            default: e = launch_tc_tn<FQ_Q8_0, 128, true>(a, tmap, tmap_w, tmap_w2, grid, st); break;
        }
        g_trace.launches++;
        return e == cudaSuccess ? FQ_OK : cuda_fail(e, "tensor-core GEMM launch");
    }
    switch (w.fmt) {
        case FQ_Q4_K: e = launch_tc<FQ_Q4_K>(a, tmap, tmap_w, grid, tile_tokens, st); break;
        case FQ_Q5_K: e = launch_tc<FQ_Q5_K>(a, tmap, tmap_w, grid, tile_tokens, st); break;
        case FQ_Q6_K: e = launch_tc<FQ_Q6_K>(a, tmap, tmap_w, grid, tile_tokens, st); break;
        case FQ_TQ2_0: e = launch_tc<FQ_TQ2_0>(a, tmap, tmap_w, grid, tile_tokens, st); break;
        case FQ_TQ2_0_FOLDED: e = launch_tc<FQ_TQ2_0_FOLDED>(a, tmap, tmap_w, grid, tile_tokens, st); break;
        case FQ_Q2_0: e = launch_tc<FQ_Q2_0>(a, tmap, tmap_w, grid, tile_tokens, st); break;
        default: e = launch_tc<FQ_Q8_0>(a, tmap, tmap_w, grid, tile_tokens, st); break;
    }
    g_trace.launches++;
    if (e == cudaSuccess && parts > 1) {
        splitk_reduce_kernel<<<ctx->sm_count * 4, 256, 0, st>>>(partial, c_dev, (int)ldc, w.n, (int)rows, (w.n + BM - 1) / BM, a.split_from, parts, tail, 256);
        e = cudaGetLastError();
        g_trace.launches++;
    }
    return e == cudaSuccess ? FQ_OK : cuda_fail(e, "tensor-core GEMM launch");
}

int gemm_tensor_grouped_dev(Ctx* ctx, const DevWeights& w, const void* a_bf16, size_t rows, float* c_dev, size_t ldc,
                            const TcTile* table, const int* n_tiles_dev, int max_tiles, int tile_tokens, cudaStream_t st,
                            const TcPeer* peer) {
    if (tile_tokens != 128 && tile_tokens != 256) return fail(FQ_DECLINED_ARGS, "token tiles are 128 or 256 rows");
    if (!tensor_path_serves(w)) return fail(FQ_DECLINED_ARGS, "tensor-core path needs a served format with k %% 256 == 0");
    return launch_tc_rows(ctx, w, 0, (const __nv_bfloat16*)a_bf16, rows, c_dev, ldc, table, n_tiles_dev, max_tiles, tile_tokens, st,
                          nullptr, nullptr, peer);
}

// Gate and up products of one expert layer in one pass with the SwiGLU applied in the epilogue:
// g[row, j] = bf16(up[row, j] * silu(gate[row, j])) over the tile list (128-token tiles).
int gemm_tensor_grouped_gated_dev(Ctx* ctx, const DevWeights& gate, const DevWeights& up, const void* a_bf16, size_t rows, void* g_bf16,
                                  size_t ldc, const TcTile* table, const int* n_tiles_dev, int max_tiles, cudaStream_t st,
                                  const TcPeer* peer, int gated_op) {
    if (!tensor_path_serves(gate) || (gate.fmt != FQ_Q4_K && gate.fmt != FQ_Q5_K && gate.fmt != FQ_Q6_K && gate.fmt != FQ_Q8_0))
        return fail(FQ_DECLINED_ARGS, "the gated tensor-core form serves Q4_K, Q5_K, Q6_K and Q8_0 with k %% 256 == 0");
    if (up.fmt != gate.fmt || up.n != gate.n || up.k != gate.k || up.n_mats != gate.n_mats || up.tile_rows != gate.tile_rows ||
        up.row_stride != gate.row_stride || up.mat_stride != gate.mat_stride)
        return fail(FQ_DECLINED_ARGS, "gate and up stacks differ in shape or layout");
    return launch_tc_rows(ctx, gate, 0, (const __nv_bfloat16*)a_bf16, rows, nullptr, ldc, table, n_tiles_dev, max_tiles, 128, st, &up,
                          (__nv_bfloat16*)g_bf16, peer, gated_op);
}

__global__ void add_f32_kernel(float* __restrict__ c, const float* __restrict__ t, size_t n) {
    for (size_t i = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) * 4; i < n; i += (size_t)gridDim.x * blockDim.x * 4) {
        float4 a = *reinterpret_cast<const float4*>(c + i);
        const float4 b = *reinterpret_cast<const float4*>(t + i);
        a.x = __fadd_rn(a.x, b.x), a.y = __fadd_rn(a.y, b.y), a.z = __fadd_rn(a.z, b.z), a.w = __fadd_rn(a.w, b.w);
        *reinterpret_cast<float4*>(c + i) = a;
    }
}
// c += t over n floats (n % 4 == 0, both 16-byte aligned): the plane sum of a multi-plane ternary product
cudaError_t launch_add_f32(float* c, const float* t, size_t n, cudaStream_t st) {
    int blocks = (int)((n / 4 + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    add_f32_kernel<<<blocks, 256, 0, st>>>(c, t, n);
    return cudaGetLastError();
}

cudaError_t launch_f32_to_bf16(const float* src, void* dst, size_t n, cudaStream_t st) {
    int blocks = (int)((n / 4 + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    f32_to_bf16_kernel<<<blocks, 256, 0, st>>>(src, (__nv_bfloat16*)dst, n);
    return cudaGetLastError();
}

int gemm_tensor_dev(Ctx* ctx, const DevWeights& w, int mat, const float* a_dev, float* c_dev, size_t m, size_t ldc, cudaStream_t st) {
    if (!format_info(w.fmt).block_elems) return fail(FQ_DECLINED_ARGS, "format %d has no tensor-core kernel", w.fmt);
    if (w.k % 256 != 0 || m < 1 || m > (size_t)1 << 24) return fail(FQ_DECLINED_ARGS, "tensor-core path needs k %% 256 == 0");
    // bf16 copy of the activations: [m][k], read by TMA with a 128-byte swizzle
    __nv_bfloat16* abf = (__nv_bfloat16*)dev_alloc_on(m * (size_t)w.k * 2, st);
    if (!abf) return fail(FQ_DECLINED_BUDGET, "bf16 activation scratch allocation failed");
    launch_f32_to_bf16(a_dev, abf, m * (size_t)w.k, st);
    g_trace.launches++;
    // up to 128 tokens: one tile column of 128 with alternating accumulators; above that 256-token tiles
    const int rc = launch_tc_rows(ctx, w, mat, abf, m, c_dev, ldc, nullptr, nullptr, 0, m <= 128 ? 128 : 256, st);
    dev_free_on(abf, st);  // stream-ordered reuse: no host wait
    return rc;
}

}  // namespace fq
