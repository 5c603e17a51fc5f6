// Streaming attention forward: online-softmax grouped attention over an f16 or f32 KV cache.
//
// The reference provider has one kernel for it (src/backend/cuda/kernels.cu:574-681 `fucina_attn_fwd_{f16,f32}`, host
// side src/backend/cuda.zig:2601-2736): one warp per query row walks the whole key range. Same contract here --
// q [q_seq][heads][d] f32, k/v [kv_seq][kv_heads][d], per-head kv map, query row i at absolute position
// source_offset + i, causal with an optional sliding window or bidirectional, optional {row max, sum exp} stats --
// but the key range of a (row, head) is cut into splits that run on different SMs (a decode step has one query row and
// thousands of keys), each split walked by four warps, and a second kernel merges the splits' (max, sum, accumulator)
// triples. The K and V rows of a step are staged in shared memory by cp.async and shared by the query heads that map
// to the kv head. Everything is f32 arithmetic in a fixed order: results do not depend on the grid.
//
// Bound: HBM (K and V bytes are read once per kv head and query row).
#include <cuda_fp16.h>

#include <cstdlib>

#include "internal.h"
#include "runtime.h"

namespace fq {

namespace {

constexpr int kAttnWarps = 4;
constexpr int kAttnMaxD = 256;
constexpr float kNegBig = -3.4e38f;

struct AttnArgs {
    const float* q;
    const void* k;
    const void* v;
    float* out;
    float* stats;        // [heads][q_seq][2] or nullptr
    const int* kvmap;    // [heads]
    float* part;         // [q_seq][heads][splits][d + 2] when splits > 1
    int q_seq, kv_seq, heads, kv_heads, d;
    int source_offset, window, causal;
    float scale;
    int splits, split_len;  // split s covers keys [s * split_len, (s + 1) * split_len)
};

// ---- shared-memory tiles ------------------------------------------------------------------------------------------
// A warp step covers 32 keys of one kv head: the K and V rows of those keys are copied into shared memory by
// cp.async (16 bytes per lane per instruction, whole rows: coalesced), rows past the range arrive as zeros. The tile is
// then used by every query head that maps to this kv head (up to kGroup at a time), so K and V leave HBM and L2 once
// per kv head, not once per head.
constexpr int kGroup = 4;  // query heads multiplied per pass over the keys (a kv head with more takes further passes)
template <typename KVT>
struct Tile {
    static constexpr int vec = 16 / (int)sizeof(KVT);              // values per 16-byte chunk: 8 (f16) or 4 (f32)
    static __host__ __device__ int kstride(int d) { return d + vec; }  // K row stride in values: an odd number of 16-byte chunks
    static __host__ __device__ size_t warp_bytes(int d) { return (size_t)32 * (kstride(d) + d) * sizeof(KVT) + kGroup * 32 * sizeof(float); }
};
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}
// one 16-byte chunk of a tile row as floats
__device__ __forceinline__ void chunk_f32(const __half* p, float (&f)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = __half22float2(h[i]);
        f[2 * i] = x.x, f[2 * i + 1] = x.y;
    }
}
__device__ __forceinline__ void chunk_f32(const float* p, float (&f)[4]) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    f[0] = x.x, f[1] = x.y, f[2] = x.z, f[3] = x.w;
}
// four consecutive values of a V tile row (8 or 16 bytes)
__device__ __forceinline__ float4 load4(const __half* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }

// grid (splits, kv_heads, q_seq); blockDim.x / 32 warps: warp w takes the 32-key steps w, w + warps, ... of the split
template <typename KVT>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_split_kernel(const AttnArgs A) {
    extern __shared__ __align__(16) uint8_t attn_smem[];
    constexpr int VEC = Tile<KVT>::vec;
    __shared__ int sh_heads[kGroup];
    __shared__ int sh_ng, sh_more;
    __shared__ float sh_m[kAttnWarps][kGroup], sh_l[kAttnWarps][kGroup];
    const int nw = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s = blockIdx.x, kvh = blockIdx.y, qi = blockIdx.z;
    const int d = A.d, kstr = Tile<KVT>::kstride(d);
    float* sh_q = reinterpret_cast<float*>(attn_smem);  // [kGroup][d], pre-scaled
    uint8_t* wbase = attn_smem + (size_t)kGroup * d * sizeof(float) + (size_t)w * Tile<KVT>::warp_bytes(d);
    KVT* Ks = reinterpret_cast<KVT*>(wbase);
    KVT* Vs = Ks + (size_t)32 * kstr;
    float* sh_p = reinterpret_cast<float*>(Vs + (size_t)32 * d);  // [kGroup][32]
    const KVT* K = reinterpret_cast<const KVT*>(A.k);
    const KVT* V = reinterpret_cast<const KVT*>(A.v);

    // this row's key range (kernels.cu:600-602), cut to the split
    const int p_abs = A.source_offset + qi;
    int end = A.causal ? min(p_abs + 1, A.kv_seq) : A.kv_seq;
    int start = (A.causal && A.window > 0 && p_abs + 1 > A.window) ? (p_abs + 1 - A.window) : 0;
    start = max(start, s * A.split_len);
    end = min(end, (s + 1) * A.split_len);

    constexpr int ND = kAttnMaxD / 128;  // lane holds the four dims from (lane + 32 * t) * 4
    for (int base = 0;; base += kGroup) {
        // the heads that map to this kv head, in head order: ranks [base, base + kGroup) this pass
        if (w == 0) {
            int seen = 0;
            for (int h0 = 0; h0 < A.heads; h0 += 32) {
                const int h = h0 + lane;
                const bool hit = h < A.heads && A.kvmap[h] == kvh;
                const unsigned mask = __ballot_sync(0xffffffffu, hit);
                const int rank = seen + __popc(mask & ((1u << lane) - 1u));
                if (hit && rank >= base && rank < base + kGroup) sh_heads[rank - base] = h;
                seen += __popc(mask);
            }
            if (lane == 0) {
                sh_ng = max(0, min(kGroup, seen - base));
                sh_more = seen > base + kGroup;
            }
        }
        __syncthreads();
        const int ng = sh_ng;
        if (ng == 0) return;
        for (int t = threadIdx.x; t < ng * d; t += blockDim.x) {
            const int g = t / d, i = t - g * d;
            sh_q[t] = A.q[((size_t)qi * A.heads + sh_heads[g]) * d + i] * A.scale;
        }
        __syncthreads();

        float acc[kGroup][ND][4];
        float m_run[kGroup], l_run[kGroup];
#pragma unroll
        for (int g = 0; g < kGroup; ++g) {
            m_run[g] = kNegBig, l_run[g] = 0.0f;
#pragma unroll
            for (int t = 0; t < ND; ++t) acc[g][t][0] = acc[g][t][1] = acc[g][t][2] = acc[g][t][3] = 0.0f;
        }

        for (int j0 = start + w * 32; j0 < end; j0 += nw * 32) {
            // stage the 32 K rows and the 32 V rows of this step
            const int cpr = d / VEC;  // 16-byte chunks per row
            for (int c = lane; c < 32 * cpr; c += 32) {
                const int row = c / cpr, col = c - row * cpr;
                const int j = j0 + row;
                const bool ok = j < end;
                const size_t off = ((size_t)(ok ? j : j0) * A.kv_heads + kvh) * d + (size_t)col * VEC;
                cp_async16((uint32_t)__cvta_generic_to_shared(Ks + (size_t)row * kstr + col * VEC), K + off, ok ? 16 : 0);
                cp_async16((uint32_t)__cvta_generic_to_shared(Vs + (size_t)row * d + col * VEC), V + off, ok ? 16 : 0);
            }
            cp_async_wait_all();
            __syncwarp();

            // scores: lane = key, every head of the group against the lane's K row
            float sc[kGroup];
#pragma unroll
            for (int g = 0; g < kGroup; ++g) sc[g] = 0.0f;
            const KVT* krow = Ks + (size_t)lane * kstr;
            for (int t = 0; t < d; t += VEC) {
                float kf[VEC];
                chunk_f32(krow + t, kf);
#pragma unroll
                for (int g = 0; g < kGroup; ++g) {
                    if (g < ng) {
                        const float* qg = sh_q + g * d + t;
#pragma unroll
                        for (int i = 0; i < VEC; i += 4) {
                            const float4 qq = *reinterpret_cast<const float4*>(qg + i);  // broadcast read
                            sc[g] = fmaf(qq.x, kf[i], sc[g]);
                            sc[g] = fmaf(qq.y, kf[i + 1], sc[g]);
                            sc[g] = fmaf(qq.z, kf[i + 2], sc[g]);
                            sc[g] = fmaf(qq.w, kf[i + 3], sc[g]);
                        }
                    }
                }
            }
            const bool live = j0 + lane < end;
            float rescale[kGroup];
#pragma unroll
            for (int g = 0; g < kGroup; ++g) {
                if (g < ng) {
                    const float sg = live ? sc[g] : kNegBig;
                    float m_tile = sg;
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, off));
                    const float m_new = fmaxf(m_run[g], m_tile);
                    const float p = live ? expf(sg - m_new) : 0.0f;
                    rescale[g] = (m_run[g] > -3.0e38f) ? expf(m_run[g] - m_new) : 0.0f;
                    float p_sum = p;
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) p_sum += __shfl_xor_sync(0xffffffffu, p_sum, off);
                    l_run[g] = l_run[g] * rescale[g] + p_sum;
                    m_run[g] = m_new;
                    sh_p[g * 32 + lane] = p;
                } else {
                    rescale[g] = 0.0f;
                }
            }
            __syncwarp();

            // values: lane = four dims, the 32 V rows one after the other (rows past the range are zero with p = 0)
#pragma unroll
            for (int t = 0; t < ND; ++t) {
                const int dim = (lane + 32 * t) * 4;
#pragma unroll
                for (int g = 0; g < kGroup; ++g) {
                    acc[g][t][0] *= rescale[g], acc[g][t][1] *= rescale[g], acc[g][t][2] *= rescale[g], acc[g][t][3] *= rescale[g];
                }
                if (dim < d) {
#pragma unroll 8
                    for (int jj = 0; jj < 32; ++jj) {
                        const float4 vv = load4(Vs + (size_t)jj * d + dim);
#pragma unroll
                        for (int g = 0; g < kGroup; ++g) {
                            if (g < ng) {
                                const float pj = sh_p[g * 32 + jj];
                                acc[g][t][0] = fmaf(pj, vv.x, acc[g][t][0]);
                                acc[g][t][1] = fmaf(pj, vv.y, acc[g][t][1]);
                                acc[g][t][2] = fmaf(pj, vv.z, acc[g][t][2]);
                                acc[g][t][3] = fmaf(pj, vv.w, acc[g][t][3]);
                            }
                        }
                    }
                }
            }
            __syncwarp();  // the tile is free for the next step's copies
        }

        // merge the warps in warp order; a warp's accumulators go where its tiles were
        float* my_acc = reinterpret_cast<float*>(wbase);  // [kGroup][d]
        if (lane == 0) {
#pragma unroll
            for (int g = 0; g < kGroup; ++g) sh_m[w][g] = m_run[g], sh_l[w][g] = l_run[g];
        }
#pragma unroll
        for (int g = 0; g < kGroup; ++g)
#pragma unroll
            for (int t = 0; t < ND; ++t) {
                const int dim = (lane + 32 * t) * 4;
                if (g < ng && dim < d) *reinterpret_cast<float4*>(my_acc + g * d + dim) = make_float4(acc[g][t][0], acc[g][t][1], acc[g][t][2], acc[g][t][3]);
            }
        __syncthreads();
        for (int t = threadIdx.x; t < ng * d; t += blockDim.x) {
            const int g = t / d, dim = t - g * d, h = sh_heads[g];
            float m = kNegBig;
            for (int i = 0; i < nw; ++i) m = fmaxf(m, sh_m[i][g]);
            float l = 0.0f, a = 0.0f;
            for (int i = 0; i < nw; ++i) {
                const float f = sh_m[i][g] > -3.0e38f ? expf(sh_m[i][g] - m) : 0.0f;
                l += sh_l[i][g] * f;
                a += reinterpret_cast<const float*>(attn_smem + (size_t)kGroup * d * sizeof(float) + (size_t)i * Tile<KVT>::warp_bytes(d))[g * d + dim] * f;
            }
            if (A.splits > 1) {
                float* part = A.part + (((size_t)qi * A.heads + h) * A.splits + s) * (d + 2);
                part[2 + dim] = a;
                if (dim == 0) part[0] = m, part[1] = l;
            } else {
                A.out[((size_t)qi * A.heads + h) * d + dim] = a * (l > 0.0f ? 1.0f / l : 0.0f);
                if (dim == 0 && A.stats) {
                    const size_t sb = ((size_t)h * A.q_seq + qi) * 2;
                    A.stats[sb] = m, A.stats[sb + 1] = l;
                }
            }
        }
        if (!sh_more) return;
        __syncthreads();  // the next pass overwrites the head list, the query rows and the tiles
    }
}

// ---- f16 KV, d <= 128: the same step on the warp-level tensor-core instruction ------------------------------------
// The scalar form above spends about 4500 warp instructions on a step (32 keys x up to four heads); with
// mma.sync.m16n8k16 it is a few hundred, which is what a decode step needs to follow the memory system. Rows of the
// 16-row operand = the heads of the group (rows 4..15 are zero). Scores: A = the query rows as f16 high + low parts
// (two instructions, so the f32 query is not rounded), B = the K tile read by ldmatrix. Values: A = the probabilities
// as f16 (the accumulator layout of two 8-key score tiles is the operand layout of one 16-key step), B = the V tile
// read by ldmatrix.trans. Both tiles have rows padded by 16 bytes so the 8 row addresses of an ldmatrix phase fall on
// distinct banks. Fragment layouts (g = lane / 4, t = lane % 4): A a0 = (row g, k 2t..2t+1), a2 = (row g, k 2t+8..);
// B b0 = (k 2t..2t+1, n g), b1 = (k 2t+8.., n g); C c0, c1 = (row g, n 2t, 2t+1).
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// rows 8..15 of the A operand are zero (a1 = a3 = 0); their accumulator halves c2, c3 are dead (a shared pair of dead
// registers would chain every instruction behind the previous one: measured slower)
__device__ __forceinline__ void mma_rows8(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float x, float y) {
    const __half2 h = __floats2half2_rn(x, y);
    return *reinterpret_cast<const uint32_t*>(&h);
}
constexpr int kMmaMaxD = 128;
__host__ __device__ inline size_t mma_warp_bytes(int d) { return (size_t)2 * 32 * (d + 8) * sizeof(__half); }

__global__ void __launch_bounds__(kAttnWarps * 32) attn_split_mma_kernel(const AttnArgs A) {
    extern __shared__ __align__(16) uint8_t attn_smem[];
    __shared__ int sh_heads[kGroup];
    __shared__ int sh_ng, sh_more;
    __shared__ float sh_m[kAttnWarps][kGroup], sh_l[kAttnWarps][kGroup];
    const int nw = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int s = blockIdx.x, kvh = blockIdx.y, qi = blockIdx.z;
    const int d = A.d, str = d + 8, ksteps = d >> 4, ntiles = d >> 3;
    // two tile buffers per warp: the copies of the next step fly while this one is multiplied
    uint8_t* wbase = attn_smem + (size_t)w * 2 * mma_warp_bytes(d);
    const uint32_t buf_addr = (uint32_t)__cvta_generic_to_shared(wbase);
    const uint32_t buf_bytes = (uint32_t)mma_warp_bytes(d);
    const __half* K = reinterpret_cast<const __half*>(A.k);
    const __half* V = reinterpret_cast<const __half*>(A.v);

    const int p_abs = A.source_offset + qi;
    int end = A.causal ? min(p_abs + 1, A.kv_seq) : A.kv_seq;
    int start = (A.causal && A.window > 0 && p_abs + 1 > A.window) ? (p_abs + 1 - A.window) : 0;
    start = max(start, s * A.split_len);
    end = min(end, (s + 1) * A.split_len);

    constexpr int KS = kMmaMaxD / 16, NT = kMmaMaxD / 8;
    for (int base = 0;; base += kGroup) {
        if (w == 0) {
            int seen = 0;
            for (int h0 = 0; h0 < A.heads; h0 += 32) {
                const int h = h0 + lane;
                const bool hit = h < A.heads && A.kvmap[h] == kvh;
                const unsigned mask = __ballot_sync(0xffffffffu, hit);
                const int rank = seen + __popc(mask & ((1u << lane) - 1u));
                if (hit && rank >= base && rank < base + kGroup) sh_heads[rank - base] = h;
                seen += __popc(mask);
            }
            if (lane == 0) {
                sh_ng = max(0, min(kGroup, seen - base));
                sh_more = seen > base + kGroup;
            }
        }
        __syncthreads();
        const int ng = sh_ng;
        if (ng == 0) return;

        // query fragments: row g = head g of the group, pre-scaled, split into f16 high and low parts
        uint32_t qh[KS][2], ql[KS][2];
        {
            const bool row = g < ng;
            const float* qrow = A.q + ((size_t)qi * A.heads + (row ? sh_heads[g] : 0)) * d;
#pragma unroll
            for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    float x = 0.0f, y = 0.0f;
                    if (row && kk < ksteps) {
                        const float2 v = *reinterpret_cast<const float2*>(qrow + 16 * kk + 8 * half + 2 * t);
                        x = v.x * A.scale, y = v.y * A.scale;
                    }
                    const __half2 hi = __floats2half2_rn(x, y);
                    const float2 hf = __half22float2(hi);
                    qh[kk][half] = *reinterpret_cast<const uint32_t*>(&hi);
                    ql[kk][half] = pack_h2(x - hf.x, y - hf.y);
                }
            }
        }

        float o[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
        float m_run = kNegBig, l_run = 0.0f;  // of row g (the four lanes of a row agree)

        // two rows per pass: lane = (row parity, 16-byte chunk); d <= 128 is at most sixteen chunks per row
        auto issue = [&](int j0, int buf) {
            const int col = lane & 15, rpar = lane >> 4;
            if (col * 8 < d) {
                const uint32_t ka = buf_addr + (uint32_t)buf * buf_bytes, va = ka + (uint32_t)(32 * str) * 2;
                const size_t rstride = (size_t)A.kv_heads * d;
                const size_t off0 = ((size_t)j0 * A.kv_heads + kvh) * d + (size_t)col * 8;
                const uint32_t soff = (uint32_t)(col * 8) * 2;
#pragma unroll 4
                for (int r2 = 0; r2 < 32; r2 += 2) {
                    const int row = r2 + rpar;
                    const bool ok = j0 + row < end;
                    const size_t off = off0 + (ok ? (size_t)row * rstride : 0);
                    cp_async16(ka + (uint32_t)(row * str) * 2 + soff, K + off, ok ? 16 : 0);
                    cp_async16(va + (uint32_t)(row * str) * 2 + soff, V + off, ok ? 16 : 0);
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        const int first = start + w * 32;
        if (first < end) issue(first, 0);
        int it = 0;
        for (int j0 = first; j0 < end; j0 += nw * 32, ++it) {
            const int jn = j0 + nw * 32;
            if (jn < end) {
                issue(jn, (it + 1) & 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");  // everything but the copies just issued has landed
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            __syncwarp();
            const uint32_t ks_addr = buf_addr + (uint32_t)(it & 1) * buf_bytes, vs_addr = ks_addr + (uint32_t)(32 * str) * 2;

            // scores of the 32 keys: four 8-key tiles
            float sc[4][4];
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) sc[nb][0] = sc[nb][1] = sc[nb][2] = sc[nb][3] = 0.0f;
            const int mi = lane >> 3, mr = lane & 7;
#pragma unroll
            for (int kk = 0; kk < KS; ++kk) {
                if (kk < ksteps) {
#pragma unroll
                    for (int nbp = 0; nbp < 2; ++nbp) {
                        // matrices: (keys 16nbp..+7, dims lo), (same keys, dims hi), (keys 16nbp+8.., lo), (.., hi)
                        uint32_t r[4];
                        ldsm_x4(ks_addr + (uint32_t)(((2 * nbp + (mi >> 1)) * 8 + mr) * str + 16 * kk + (mi & 1) * 8) * 2, r);
                        mma_rows8(sc[2 * nbp], qh[kk][0], qh[kk][1], r[0], r[1]);
                        mma_rows8(sc[2 * nbp], ql[kk][0], ql[kk][1], r[0], r[1]);
                        mma_rows8(sc[2 * nbp + 1], qh[kk][0], qh[kk][1], r[2], r[3]);
                        mma_rows8(sc[2 * nbp + 1], ql[kk][0], ql[kk][1], r[2], r[3]);
                    }
                }
            }
            // online softmax of row g over the 32 keys: this lane holds keys 8nb + 2t, +1
            float m_tile = kNegBig;
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) {
                const int key = j0 + 8 * nb + 2 * t;
                if (key >= end) sc[nb][0] = kNegBig;
                if (key + 1 >= end) sc[nb][1] = kNegBig;
                m_tile = fmaxf(m_tile, fmaxf(sc[nb][0], sc[nb][1]));
            }
            m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 1));
            m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 2));
            const float m_new = fmaxf(m_run, m_tile);
            const float rescale = (m_run > -3.0e38f) ? expf(m_run - m_new) : 0.0f;
            float p_sum = 0.0f;
            uint32_t pa[2][2];  // probabilities as the A operand of the two 16-key steps
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) {
                const float p0 = sc[nb][0] > -3.0e38f ? expf(sc[nb][0] - m_new) : 0.0f;
                const float p1 = sc[nb][1] > -3.0e38f ? expf(sc[nb][1] - m_new) : 0.0f;
                p_sum += p0 + p1;
                pa[nb >> 1][nb & 1] = pack_h2(p0, p1);
            }
            p_sum += __shfl_xor_sync(0xffffffffu, p_sum, 1);
            p_sum += __shfl_xor_sync(0xffffffffu, p_sum, 2);
            l_run = l_run * rescale + p_sum;
            m_run = m_new;

            // values: out[row g][dims] += P[row g][32 keys] . V[32 keys][dims]
            const int vr = (mi & 1) * 8 + mr, vc = (mi >> 1) * 8;  // this lane's row address inside an ldmatrix.trans of 16 keys x 16 dims
#pragma unroll
            for (int ntp = 0; ntp < NT / 2; ++ntp) {
                if (2 * ntp < ntiles) {
                    o[2 * ntp][0] *= rescale, o[2 * ntp][1] *= rescale;
                    o[2 * ntp + 1][0] *= rescale, o[2 * ntp + 1][1] *= rescale;
#pragma unroll
                    for (int kb = 0; kb < 2; ++kb) {
                        // matrices: (keys 16kb..+7, dims 16ntp..+7), (keys +8, same dims), (keys 16kb.., dims +8), (keys +8, dims +8)
                        uint32_t r[4];
                        ldsm_x4_t(vs_addr + (uint32_t)((16 * kb + vr) * str + 16 * ntp + vc) * 2, r);
                        mma_rows8(o[2 * ntp], pa[kb][0], pa[kb][1], r[0], r[1]);
                        mma_rows8(o[2 * ntp + 1], pa[kb][0], pa[kb][1], r[2], r[3]);
                    }
                }
            }
            __syncwarp();  // the tiles are free for the next step's copies
        }

        // merge the warps in warp order; a warp's accumulators go where its tiles were
        float* my_acc = reinterpret_cast<float*>(wbase);  // [kGroup][d]
        if (g < ng) {
            if (t == 0) sh_m[w][g] = m_run, sh_l[w][g] = l_run;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
                if (nt < ntiles) *reinterpret_cast<float2*>(my_acc + g * d + 8 * nt + 2 * t) = make_float2(o[nt][0], o[nt][1]);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < ng * d; i += blockDim.x) {
            const int gg = i / d, dim = i - gg * d, h = sh_heads[gg];
            float m = kNegBig;
            for (int x = 0; x < nw; ++x) m = fmaxf(m, sh_m[x][gg]);
            float l = 0.0f, a = 0.0f;
            for (int x = 0; x < nw; ++x) {
                const float f = sh_m[x][gg] > -3.0e38f ? expf(sh_m[x][gg] - m) : 0.0f;
                l += sh_l[x][gg] * f;
                a += reinterpret_cast<const float*>(attn_smem + (size_t)x * 2 * mma_warp_bytes(d))[gg * d + dim] * f;
            }
            if (A.splits > 1) {
                float* part = A.part + (((size_t)qi * A.heads + h) * A.splits + s) * (d + 2);
                part[2 + dim] = a;
                if (dim == 0) part[0] = m, part[1] = l;
            } else {
                A.out[((size_t)qi * A.heads + h) * d + dim] = a * (l > 0.0f ? 1.0f / l : 0.0f);
                if (dim == 0 && A.stats) {
                    const size_t sb = ((size_t)h * A.q_seq + qi) * 2;
                    A.stats[sb] = m, A.stats[sb + 1] = l;
                }
            }
        }
        if (!sh_more) return;
        __syncthreads();
    }
}

// one CTA per (head, row): the splits' triples merged. The splits' maxima and sums are staged in shared memory; each of
// the four warps then adds every fourth split (lane = four dims, 16-byte loads, all of a warp's loads independent) and
// the warps' sums are added in warp order: a fixed order, whatever the grid of the first kernel was.
constexpr int kAttnMaxSplits = 1024;
__global__ void __launch_bounds__(128) attn_merge_kernel(const AttnArgs A) {
    __shared__ float sm_m[kAttnMaxSplits], sm_f[kAttnMaxSplits], sm_ls[kAttnMaxSplits];
    __shared__ __align__(16) float sm_acc[4][kAttnMaxD];
    __shared__ float sm_l;
    const int h = blockIdx.x, qi = blockIdx.y, d = A.d, n = A.splits;
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t stride = (size_t)d + 2;
    const float* part = A.part + ((size_t)qi * A.heads + h) * n * stride;
    for (int s = threadIdx.x; s < n; s += blockDim.x) sm_m[s] = part[(size_t)s * stride], sm_ls[s] = part[(size_t)s * stride + 1];
    __syncthreads();
    float m = kNegBig;
    for (int s = 0; s < n; ++s) m = fmaxf(m, sm_m[s]);
    for (int s = threadIdx.x; s < n; s += blockDim.x) sm_f[s] = sm_m[s] > -3.0e38f ? expf(sm_m[s] - m) : 0.0f;
    __syncthreads();
    if (threadIdx.x == 0) {
        float l = 0.0f;
        for (int s = 0; s < n; ++s) l += sm_ls[s] * sm_f[s];
        sm_l = l;
    }
    for (int d0 = 0; d0 < d; d0 += 128) {
        const int dim = d0 + lane * 4;
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        if (dim < d) {
#pragma unroll 4
            for (int s = w; s < n; s += 4) {
                const float2 lo = *reinterpret_cast<const float2*>(part + (size_t)s * stride + 2 + dim);  // (d + 2) floats per split: 8-byte aligned
                const float2 hi = *reinterpret_cast<const float2*>(part + (size_t)s * stride + 4 + dim);
                const float f = sm_f[s];
                a0 = fmaf(lo.x, f, a0), a1 = fmaf(lo.y, f, a1), a2 = fmaf(hi.x, f, a2), a3 = fmaf(hi.y, f, a3);
            }
            *reinterpret_cast<float4*>(&sm_acc[w][dim]) = make_float4(a0, a1, a2, a3);
        }
    }
    __syncthreads();
    const float l = sm_l, inv_l = l > 0.0f ? 1.0f / l : 0.0f;
    for (int dim = threadIdx.x; dim < d; dim += blockDim.x)
        A.out[((size_t)qi * A.heads + h) * d + dim] = (((sm_acc[0][dim] + sm_acc[1][dim]) + sm_acc[2][dim]) + sm_acc[3][dim]) * inv_l;
    if (A.stats && threadIdx.x == 0) {
        const size_t sb = ((size_t)h * A.q_seq + qi) * 2;
        A.stats[sb] = m, A.stats[sb + 1] = l;
    }
}

int check_attn(size_t q_seq, size_t kv_seq, size_t heads, size_t kv_heads, size_t d, int kv_is_f16) {
    if (q_seq == 0 || kv_seq == 0 || heads == 0 || kv_heads == 0 || d == 0) return fail(FQ_DECLINED_ARGS, "empty attention problem");
    if (d > (size_t)kAttnMaxD || heads > 512) return fail(FQ_DECLINED_ARGS, "d <= 256 and heads <= 512 (backend/cuda.zig:617-625)");
    if (d % (kv_is_f16 ? 8 : 4) != 0) return fail(FQ_DECLINED_ARGS, "d=%zu: rows of K and V are read 16 bytes at a time", d);
    if (q_seq > 65535 || kv_heads > 65535 || kv_seq > (size_t)INT32_MAX) return fail(FQ_DECLINED_ARGS, "attention problem too large for one launch");
    return FQ_OK;
}

}  // namespace
}  // namespace fq

using namespace fq;

extern "C" {

int fq_attn_fwd_dev(const float* q_dev, const void* k_dev, const void* v_dev, int kv_is_f16, float* out_dev, float* stats_dev,
                    const int32_t* kv_head_for_head_dev, size_t q_seq, size_t kv_seq, size_t heads, size_t kv_heads, size_t d,
                    size_t source_offset, float scale, size_t window, int causal, void* stream) {
    if (!q_dev || !k_dev || !v_dev || !out_dev || !kv_head_for_head_dev) return fail(FQ_DECLINED_ARGS, "null pointer");
    if (int rc = check_attn(q_seq, kv_seq, heads, kv_heads, d, kv_is_f16)) return rc;
    if (((uintptr_t)k_dev | (uintptr_t)v_dev | (uintptr_t)q_dev | (uintptr_t)out_dev) & 15) return fail(FQ_DECLINED_ARGS, "q, k, v and out must be 16-byte aligned");
    if (!gpu_enabled()) return fail(FQ_DECLINED_GATE, "disabled by FUCINA_GPU=0");
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    g_trace.calls++;
    cudaStream_t st = stream ? (cudaStream_t)stream : ctx->stream;
    // shared memory: the group's query rows + per warp a K tile, a V tile and the probabilities; as many of the four
    // warps as fit (f32 KV with d = 256 needs 65 KB per warp)
    static const bool no_mma = getenv("FUCINA_B200_ATTN_NO_MMA") != nullptr;
    const bool use_mma = kv_is_f16 && !no_mma && d <= (size_t)kMmaMaxD && d % 16 == 0;
    const size_t wbytes = use_mma ? mma_warp_bytes((int)d) : kv_is_f16 ? Tile<__half>::warp_bytes((int)d) : Tile<float>::warp_bytes((int)d);
    const size_t qbytes = use_mma ? 0 : (size_t)kGroup * d * sizeof(float);
    int nw = use_mma ? 2 : kAttnWarps;  // the tensor-core form double-buffers its tiles: two warps of 35 KB, three CTAs per SM
    const size_t per_warp = use_mma ? 2 * wbytes : wbytes;
    while (nw > 1 && qbytes + nw * per_warp > (size_t)200 * 1024) nw >>= 1;
    const size_t smem = qbytes + nw * per_warp;
    const int ctas_per_sm = (int)((size_t)220 * 1024 / (smem + 1024)) < 1 ? 1 : (int)((size_t)220 * 1024 / (smem + 1024));
    // splits: one wave of CTAs (what the shared memory lets an SM hold), at least one 32-key step per warp each
    const size_t rows = q_seq * kv_heads;
    size_t splits = ((size_t)ctas_per_sm * ctx->sm_count + rows - 1) / rows;
    const size_t step_keys = (size_t)nw * 32;
    const size_t max_splits = (kv_seq + step_keys - 1) / step_keys;
    if (splits > max_splits) splits = max_splits;
    if (splits > (size_t)kAttnMaxSplits) splits = kAttnMaxSplits;
    if (splits < 1) splits = 1;
    size_t split_len = ((kv_seq + splits - 1) / splits + step_keys - 1) / step_keys * step_keys;
    splits = (kv_seq + split_len - 1) / split_len;
    if (window > kv_seq) window = kv_seq;  // any window >= kv_seq is plain causal (backend/cuda.zig:2621-2625)
    float* part = nullptr;
    if (splits > 1) {
        part = (float*)dev_alloc_on(q_seq * heads * splits * (d + 2) * sizeof(float), st);
        if (!part) return fail(FQ_DECLINED_BUDGET, "attention scratch allocation failed");
    }
    AttnArgs a{q_dev, k_dev, v_dev, out_dev, stats_dev, kv_head_for_head_dev, part, (int)q_seq, (int)kv_seq, (int)heads, (int)kv_heads, (int)d,
               (int)source_offset, (int)window, causal ? 1 : 0, scale, (int)splits, (int)split_len};
    const dim3 grid((unsigned)splits, (unsigned)kv_heads, (unsigned)q_seq);
    static bool granted = false;
    cudaError_t e = cudaSuccess;
    if (!granted) {
        e = cudaFuncSetAttribute(attn_split_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_split_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_split_kernel<__half>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_split_kernel<float>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_split_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_split_mma_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) {
            dev_free_on(part, st);
            return cuda_fail(e, "attention kernel attributes");
        }
        granted = true;
    }
    if (use_mma) attn_split_mma_kernel<<<grid, nw * 32, smem, st>>>(a);
    else if (kv_is_f16) attn_split_kernel<__half><<<grid, nw * 32, smem, st>>>(a);
    else attn_split_kernel<float><<<grid, nw * 32, smem, st>>>(a);
    e = cudaGetLastError();
    g_trace.launches++;
    if (e == cudaSuccess && splits > 1) {
        attn_merge_kernel<<<dim3((unsigned)heads, (unsigned)q_seq), 128, 0, st>>>(a);
        e = cudaGetLastError();
        g_trace.launches++;
    }
    dev_free_on(part, st);
    return e == cudaSuccess ? FQ_OK : cuda_fail(e, "attention launch");
}

// Host buffers, blocking: the argument list of attnFwdHostImpl (backend/cuda.zig:2626-2736).
int fq_attn_fwd(const float* q, const void* k, const void* v, int kv_is_f16, float* out, float* stats, const int32_t* kv_head_for_head,
                size_t q_seq, size_t kv_seq, size_t heads, size_t kv_heads, size_t d, size_t source_offset, float scale, size_t window,
                int causal) {
    if (!q || !k || !v || !out || !kv_head_for_head) return fail(FQ_DECLINED_ARGS, "null pointer");
    if (int rc = check_attn(q_seq, kv_seq, heads, kv_heads, d, kv_is_f16)) return rc;
    for (size_t h = 0; h < heads; ++h)
        if (kv_head_for_head[h] < 0 || (size_t)kv_head_for_head[h] >= kv_heads) return fail(FQ_DECLINED_ARGS, "kv head map entry %zu out of range", h);
    if (!gpu_enabled()) return fail(FQ_DECLINED_GATE, "disabled by FUCINA_GPU=0");
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    const size_t qb = q_seq * heads * d * 4, kvb = kv_seq * kv_heads * d * (kv_is_f16 ? 2 : 4), sb = stats ? heads * q_seq * 2 * 4 : 0;
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    uint8_t* dev = (uint8_t*)dev_alloc(up(qb) * 2 + up(kvb) * 2 + up(heads * 4) + up(sb) + 256);
    if (!dev) return fail(FQ_DECLINED_BUDGET, "attention buffers could not be allocated");
    uint8_t* dq = dev;
    uint8_t* dk = dq + up(qb);
    uint8_t* dv = dk + up(kvb);
    uint8_t* dout = dv + up(kvb);
    uint8_t* dmap = dout + up(qb);
    uint8_t* dstats = dmap + up(heads * 4);
    int rc = FQ_OK;
    cudaError_t e = cudaMemcpyAsync(dq, q, qb, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dk, k, kvb, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dv, v, kvb, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dmap, kv_head_for_head, heads * 4, cudaMemcpyHostToDevice, ctx->stream);
    g_trace.h2d_bytes += qb + 2 * kvb + heads * 4;
    if (e != cudaSuccess) rc = cuda_fail(e, "attention upload");
    if (rc == FQ_OK)
        rc = fq_attn_fwd_dev((const float*)dq, dk, dv, kv_is_f16, (float*)dout, stats ? (float*)dstats : nullptr, (const int32_t*)dmap, q_seq, kv_seq, heads,
                             kv_heads, d, source_offset, scale, window, causal, ctx->stream);
    if (rc == FQ_OK) {
        e = cudaMemcpyAsync(out, dout, qb, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess && stats) e = cudaMemcpyAsync(stats, dstats, sb, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        g_trace.d2h_bytes += qb + sb;
        if (e != cudaSuccess) rc = cuda_fail(e, "attention download");
    } else {
        cudaStreamSynchronize(ctx->stream);
    }
    dev_free(dev);
    return rc;
}

}  // extern "C"
