// MoE expert layer on the device: router top-k, route plan, grouped expert
// products with fused SwiGLU, weighted combine. Tokens stay in HBM across all
// three expert products; the reference's GPU arm instead makes two PCIe round
// trips per layer with CPU gather / activation / scatter phases between them
// (src/llm/gemma/moe.zig:696-901, docs/GPU-OFFLOAD.md:191-203).
//
// Per (token, slot) pair p with expert e (reference src/exec/moe.zig:890-920,
// :1334-1401, src/exec/moe_chain.zig:236-330):
//   qx   = Q8_K(x[token])                       (Q8_0 blocks for Q8_0 experts)
//   g    = swiglu(W_gate[e].qx, W_up[e].qx)
//   qg   = Q8_K(g)
//   down = W_down[e].qg
//   out[token] = sum over the token's slots, in slot order, of w[p] * down
#include <cuda_bf16.h>

#include <vector>

#include "acts.cuh"
#include "internal.h"
#include "multi.h"
#include "runtime.h"

namespace fq {

namespace {

constexpr int kGroupRows = 16;  // activation rows one grouped-GEMV table entry covers

// Counting sort of pairs by expert plus the grouped-GEMV table, one CTA.
// Positions inside an expert's run are handed out by atomics: a pair's result
// does not depend on its position, so the layer output is unaffected.
//
// An expert shard (Shard.skip_foreign) serves experts [base, base + n_expert) of a larger layer:
// pairs routed elsewhere get inv = -1, take no position, and contribute nothing to the combine.
struct Shard {
    int base;
    int skip_foreign;
};
__device__ __forceinline__ int local_expert(int e, int n_expert, Shard sh) {
    e -= sh.base;
    if (e >= 0 && e < n_expert) return e;
    return sh.skip_foreign ? -1 : min(max(e, 0), n_expert - 1);
}

// One CTA: counting sort of the routed pairs by expert (order / inv), the table of row groups for the
// integer kernels and, when tile_tokens != 0, the tile lists of the grouped tensor-core GEMMs: per expert
// run ceil(count / tile_tokens) token tiles times the row tiles of the gate/up product (rt_gu) and of the
// down product (rt_dn), in expert order (the row tiles of one token tile are neighbours, so concurrent
// CTAs share its token rows in L2). Each thread keeps eight loads of the pair list in flight per step.
// Shared memory: 4 * n_expert ints.
constexpr int kPlanBatch = 8;
__global__ void route_plan_kernel(const int* __restrict__ selected, int pairs, int n_expert, Shard shard, int group_rows, int* __restrict__ order,
                                  int* __restrict__ inv, GroupDesc* __restrict__ table, int* __restrict__ n_desc,
                                  int* __restrict__ n_rows, int tile_tokens, int rt_gu, int rt_dn, TcTile* __restrict__ t_gu,
                                  int* __restrict__ n_gu, TcTile* __restrict__ t_dn, int* __restrict__ n_dn) {
    extern __shared__ int sh[];
    pdl_wait_then_release();
    int* count = sh;                   // [n_expert] pairs per expert
    int* place = sh + n_expert;        // [n_expert] first sorted position of the expert's run
    int* dstart = sh + 2 * n_expert;   // [n_expert] first table entry of the expert
    int* tstart = sh + 3 * n_expert;   // [n_expert] first token tile of the expert
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p0 = threadIdx.x; p0 < pairs; p0 += blockDim.x * kPlanBatch) {
        int e[kPlanBatch];
#pragma unroll
        for (int i = 0; i < kPlanBatch; ++i) {
            const int p = p0 + i * blockDim.x;
            e[i] = p < pairs ? local_expert(selected[p], n_expert, shard) : -1;
        }
#pragma unroll
        for (int i = 0; i < kPlanBatch; ++i)
            if (e[i] >= 0) atomicAdd(&count[e[i]], 1);
    }
    __syncthreads();
    if (warp == 0) {
        // exclusive scans over the experts: run offsets, table offsets and token-tile offsets, 32 experts per step
        int rows = 0, nd = 0, nt = 0;
        for (int base = 0; base < n_expert; base += 32) {
            const int e = base + lane;
            const int c = e < n_expert ? count[e] : 0;
            const int g = (c + group_rows - 1) / group_rows;
            const int tl = tile_tokens ? (c + tile_tokens - 1) / tile_tokens : 0;
            int ic = c, ig = g, it = tl;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int tc = __shfl_up_sync(0xffffffffu, ic, o), tg = __shfl_up_sync(0xffffffffu, ig, o);
                const int tt = __shfl_up_sync(0xffffffffu, it, o);
                if (lane >= o) ic += tc, ig += tg, it += tt;
            }
            if (e < n_expert) {
                place[e] = rows + ic - c;
                dstart[e] = nd + ig - g;
                tstart[e] = nt + it - tl;
            }
            rows += __shfl_sync(0xffffffffu, ic, 31);
            nd += __shfl_sync(0xffffffffu, ig, 31);
            nt += __shfl_sync(0xffffffffu, it, 31);
        }
        if (lane == 0) {
            *n_desc = nd;
            *n_rows = rows;
            if (tile_tokens) {
                *n_gu = nt * rt_gu;
                *n_dn = nt * rt_dn;
            }
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) {
        const int c = count[e], off = place[e];
        int d = dstart[e];
        for (int j = 0; j < c; j += group_rows) table[d++] = {e, off + j, min(group_rows, c - j), 0};
    }
    if (tile_tokens) {
        // one warp per expert; the entries of a token tile are written by consecutive lanes
        for (int e = warp; e < n_expert; e += warps) {
            const int c = count[e], row0 = place[e], tile0 = tstart[e];
            for (int t0 = 0, tt = 0; t0 < c; t0 += tile_tokens, ++tt) {
                const int nt = min(tile_tokens, c - t0);
                for (int rt = lane; rt < rt_gu; rt += 32) t_gu[(size_t)(tile0 + tt) * rt_gu + rt] = {e, rt, row0 + t0, nt};
                for (int rt = lane; rt < rt_dn; rt += 32) t_dn[(size_t)(tile0 + tt) * rt_dn + rt] = {e, rt, row0 + t0, nt};
            }
        }
    }
    __syncthreads();  // the pass below advances place[]
    for (int p0 = threadIdx.x; p0 < pairs; p0 += blockDim.x * kPlanBatch) {
        int e[kPlanBatch];
#pragma unroll
        for (int i = 0; i < kPlanBatch; ++i) {
            const int p = p0 + i * blockDim.x;
            e[i] = p < pairs ? local_expert(selected[p], n_expert, shard) : -2;
        }
#pragma unroll
        for (int i = 0; i < kPlanBatch; ++i) {
            const int p = p0 + i * blockDim.x;
            if (e[i] == -2) continue;  // past the end of the list
            if (e[i] < 0) {
                inv[p] = -1;  // another shard's expert
                continue;
            }
            const int pos = atomicAdd(&place[e[i]], 1);
            order[pos] = p;
            inv[p] = pos;
        }
    }
}

// out[t] = sum_k w[p] * down[inv[p]], slot order, first slot assigned
// (src/exec/moe_chain.zig:307-330); multiply and add stay separate.
__global__ void combine_kernel(const float* __restrict__ down, const float* __restrict__ weights, const int* __restrict__ inv,
                               int seq, int hidden, int top_k, float* __restrict__ out) {
    pdl_wait_then_release();
    const size_t total = (size_t)seq * hidden;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / hidden), j = (int)(i % hidden);
        float acc = 0.0f;
        bool first = true;
        for (int kk = 0; kk < top_k; ++kk) {
            const int p = t * top_k + kk, pos = inv[p];
            if (pos < 0) continue;  // another shard's expert
            const float v = __fmul_rn(weights[p], down[(size_t)pos * hidden + j]);
            acc = first ? v : __fadd_rn(acc, v);
            first = false;
        }
        out[i] = acc;
    }
}
// The same sum, four columns per thread (hidden % 4 == 0, 16-byte aligned rows): the token's slots are looked
// up once per four outputs instead of once per output.
__global__ void combine4_kernel(const float* __restrict__ down, const float* __restrict__ weights, const int* __restrict__ inv,
                                int seq, int hidden, int top_k, float* __restrict__ out) {
    pdl_wait_then_release();
    const int h4 = hidden >> 2;
    const size_t total = (size_t)seq * h4;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / h4), j = (int)(i % h4) * 4;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        bool first = true;
        // eight slots at a time: their positions, then their rows, are all requested before the first sum (a slot's row
        // address depends on its position: one slot at a time is two dependent round trips per slot); the sums keep slot order
        for (int kk0 = 0; kk0 < top_k; kk0 += 8) {
            int pos[8];
            float wv[8];
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const bool ok = kk0 + u < top_k;
                const int p = t * top_k + kk0 + u;
                pos[u] = ok ? inv[p] : -1;  // -1: another shard's expert, or past the last slot
                wv[u] = ok ? weights[p] : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u)
                v[u] = pos[u] >= 0 ? *reinterpret_cast<const float4*>(down + (size_t)pos[u] * hidden + j) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (pos[u] < 0) continue;
                float4 x = v[u];
                x.x = __fmul_rn(wv[u], x.x), x.y = __fmul_rn(wv[u], x.y), x.z = __fmul_rn(wv[u], x.z), x.w = __fmul_rn(wv[u], x.w);
                if (first) acc = x;
                else acc.x = __fadd_rn(acc.x, x.x), acc.y = __fadd_rn(acc.y, x.y), acc.z = __fadd_rn(acc.z, x.z), acc.w = __fadd_rn(acc.w, x.w);
                first = false;
            }
        }
        *reinterpret_cast<float4*>(out + (size_t)t * hidden + j) = acc;
    }
}
static void launch_combine(const float* down, const float* weights, const int* inv, int seq, int hidden, int top_k, float* out, cudaStream_t st) {
    if (hidden % 4 == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)down & 15) == 0) {
        const size_t total4 = (size_t)seq * (hidden / 4);
        const int blocks4 = (int)((total4 + 127) / 128);
        launch_pdl(combine4_kernel, dim3(blocks4 > 148 * 16 ? 148 * 16 : blocks4), dim3(128), 0, st, down, weights, inv, seq, hidden, top_k, out);
        return;
    }
    const size_t total = (size_t)seq * hidden;
    const int blocks = (int)((total + 255) / 256);
    launch_pdl(combine_kernel, dim3(blocks > 148 * 8 ? 148 * 8 : blocks), dim3(256), 0, st, down, weights, inv, seq, hidden, top_k, out);
}

// Router (src/exec/topk.zig:50-86), one warp per token row: the k largest logits in descending
// order, an equal logit never displaces an earlier one; softmax over all experts with the row
// maximum subtracted; optional renormalisation over the selected k. The lanes share the loads, the
// exponentials and the k arg-max rounds; the sums that fix the result bits (over all experts, over
// the selected k) are added by one lane in index order, as the scalar code does.
constexpr int kMaxTopK = 32;
constexpr int kMaxRouterExperts = 4096;
__global__ void router_topk_kernel(const float* __restrict__ logits, int rows, int experts, int k, int normalize,
                                   int* __restrict__ selected, float* __restrict__ weights) {
    extern __shared__ float rsh[];
    pdl_wait_then_release();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int row = blockIdx.x * warps + warp;
    if (row >= rows) return;  // whole warps leave together
    float* lg = rsh + (size_t)warp * 2 * experts;  // logits; a taken entry becomes NaN and never compares true again
    float* ex = lg + experts;                      // exp(logit - max)
    const float* l = logits + (size_t)row * experts;
    float mx = -INFINITY;
    for (int i = lane; i < experts; i += 32) {
        const float v = l[i];
        lg[i] = v;
        mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    for (int i = lane; i < experts; i += 32) ex[i] = expf(__fsub_rn(lg[i], mx));
    __syncwarp();
    float exp_sum = 0.0f;
    if (lane == 0)
        for (int i = 0; i < experts; ++i) exp_sum = __fadd_rn(exp_sum, ex[i]);
    float w_mine = 0.0f;  // lane s keeps slot s
    int sel_mine = 0;
    for (int s = 0; s < k; ++s) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = lane; i < experts; i += 32) {
            const float v = lg[i];
            if (v > bv) bv = v, bi = i;  // ascending i per lane: an equal later value does not displace
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
        }
        if (bi == 0x7fffffff) bi = 0;  // nothing above -inf is left
        if (lane == s) sel_mine = bi, w_mine = ex[bi];
        __syncwarp();
        if (lane == 0) lg[bi] = __int_as_float(0x7fc00000);
        __syncwarp();
    }
    const float inv_sum = __fdiv_rn(1.0f, __shfl_sync(0xffffffffu, exp_sum, 0));
    w_mine = __fmul_rn(w_mine, inv_sum);
    if (normalize) {
        float total = 0.0f;
        for (int s = 0; s < k; ++s) total = __fadd_rn(total, __shfl_sync(0xffffffffu, w_mine, s));
        if (total > 0.0f) w_mine = __fmul_rn(w_mine, __fdiv_rn(1.0f, total));
    }
    if (lane < k) {
        selected[(size_t)row * k + lane] = sel_mine;
        weights[(size_t)row * k + lane] = w_mine;
    }
}

int max_desc_for(int pairs, int n_expert, int group_rows);

// Test seam of the integer arm: copy the per-pair intermediates out in PAIR order (row p = token p / top_k,
// slot p % top_k): g = swiglu(gate . qx, up . qx) and the unweighted down rows. Pairs another shard serves get zeros.
__global__ void stages_to_pair_order_kernel(const float* __restrict__ sorted_rows, const int* __restrict__ inv, int pairs, int width,
                                            float* __restrict__ out) {
    const size_t total = (size_t)pairs * width;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int p = (int)(i / width), pos = inv[p];
        out[i] = pos < 0 ? 0.0f : sorted_rows[(size_t)pos * width + i % width];
    }
}
struct StageTaps {
    float* g_pairs;     // [pairs][out_pe] or nullptr
    float* down_pairs;  // [pairs][hidden] or nullptr
};

// ---- tensor-core form for prefill-sized batches ------------------------------------------------
// sorted pair position -> bf16 copy of its token row
__global__ void gather_bf16_kernel(const float* __restrict__ x, const int* __restrict__ order, int top_k, const int* __restrict__ n_rows,
                                   int hidden, __nv_bfloat16* __restrict__ out) {
    const size_t total = (size_t)*n_rows * hidden / 4;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t pos = i * 4 / hidden, col = i * 4 % hidden;
        const float4 v = *reinterpret_cast<const float4*>(x + (size_t)(order[pos] / top_k) * hidden + col);
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t*>(&lo);
        o.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(out + pos * hidden + col) = o;
    }
}

// g = source(up) * activation(gate) in f32 (backend/ops.zig:150-190), rounded once to bf16
__global__ void gated_bf16_kernel(const float* __restrict__ gate, const float* __restrict__ up, const int* __restrict__ n_rows, int width,
                                  int gated_op, __nv_bfloat16* __restrict__ out) {
    const size_t n = (size_t)*n_rows * width;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __float2bfloat16_rn(gated_pair(gated_op, gate[i], up[i]));
}
// the same pair in f32 over a fixed number of elements (multi-plane ternary experts: the planes of gate and of up are
// summed first, the activation follows)
__global__ void gated_f32_kernel(const float* __restrict__ gate, const float* __restrict__ up, size_t n, int gated_op, float* __restrict__ out) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = gated_pair(gated_op, gate[i], up[i]);
}

int g_moe_tensor_mode = -1;  // -1 auto (>= 17 rows per expert on average: the measured crossover of the two arms), 0 never, 1 whenever the format allows

int moe_layer_tensor_impl(Ctx* ctx, const DevWeights& gate, const DevWeights& up, const DevWeights& down, const float* x_dev,
                          int seq, int top_k, const int* selected_dev, const float* weights_dev, Shard shard, float* out_dev,
                          cudaStream_t st, int gated_op) {
    const int hidden = gate.k, out_pe = gate.n, n_expert = gate.n_mats;
    const int pairs = seq * top_k;
    const int rt_gu = (out_pe + 127) / 128, rt_dn = (hidden + 127) / 128;
    // expert runs of up to 128 rows on average: 128-token tiles (two alternating accumulators hide the
    // epilogue of these short tiles); longer runs: 256-token tiles
    const int tile_tokens = pairs <= 128 * n_expert ? 128 : 256;
    const int tok_tiles = (pairs < n_expert ? pairs : n_expert) + pairs / tile_tokens;
    const int max_gu = rt_gu * tok_tiles, max_dn = rt_dn * tok_tiles;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off += (bytes + 255) & ~(size_t)255;
        return o;
    };
    const size_t o_order = take(sizeof(int) * pairs), o_inv = take(sizeof(int) * pairs), o_cnt = take(sizeof(int) * 4);
    const size_t o_desc = take(sizeof(GroupDesc) * max_desc_for(pairs, n_expert, kGroupRows));
    const size_t o_tgu = take(sizeof(TcTile) * max_gu), o_tdn = take(sizeof(TcTile) * max_dn);
    const size_t o_xb = take((size_t)pairs * hidden * 2), o_gate = take(sizeof(float) * (size_t)pairs * out_pe);
    const size_t o_up = take(sizeof(float) * (size_t)pairs * out_pe), o_gb = take((size_t)pairs * out_pe * 2);
    const size_t o_down = take(sizeof(float) * (size_t)pairs * hidden);
    uint8_t* s = (uint8_t*)dev_alloc_on(off, st);
    if (!s) return fail(FQ_DECLINED_BUDGET, "MoE scratch allocation of %zu bytes failed", off);
    int* order = (int*)(s + o_order);
    int* inv = (int*)(s + o_inv);
    int* cnt = (int*)(s + o_cnt);  // [0] row-group count (unused here), [1] gate/up tiles, [2] down tiles, [3] rows this shard serves
    cudaError_t e = cudaSuccess;
    int rc = FQ_OK;
    do {
        route_plan_kernel<<<1, 1024, sizeof(int) * 4 * n_expert, st>>>(selected_dev, pairs, n_expert, shard, kGroupRows, order, inv, (GroupDesc*)(s + o_desc), cnt, cnt + 3,
                                                                    tile_tokens, rt_gu, rt_dn, (TcTile*)(s + o_tgu), cnt + 1, (TcTile*)(s + o_tdn), cnt + 2);
        int blocks = (int)(((size_t)pairs * hidden / 4 + 255) / 256);
        gather_bf16_kernel<<<blocks > 148 * 8 ? 148 * 8 : blocks, 256, 0, st>>>(x_dev, order, top_k, cnt + 3, hidden, (__nv_bfloat16*)(s + o_xb));
        if ((e = cudaGetLastError()) != cudaSuccess) break;
        if (tile_tokens == 128) {
            // short runs: gate and up of a tile share one pass, the SwiGLU runs in its epilogue
            if ((rc = gemm_tensor_grouped_gated_dev(ctx, gate, up, s + o_xb, pairs, s + o_gb, out_pe, (const TcTile*)(s + o_tgu), cnt + 1, max_gu, st, nullptr,
                                                    gated_op)) != FQ_OK)
                break;
        } else {
            if ((rc = gemm_tensor_grouped_dev(ctx, gate, s + o_xb, pairs, (float*)(s + o_gate), out_pe, (const TcTile*)(s + o_tgu), cnt + 1, max_gu, tile_tokens, st)) != FQ_OK) break;
            if ((rc = gemm_tensor_grouped_dev(ctx, up, s + o_xb, pairs, (float*)(s + o_up), out_pe, (const TcTile*)(s + o_tgu), cnt + 1, max_gu, tile_tokens, st)) != FQ_OK) break;
            const size_t ng = (size_t)pairs * out_pe;
            blocks = (int)((ng + 255) / 256);
            gated_bf16_kernel<<<blocks > 148 * 8 ? 148 * 8 : blocks, 256, 0, st>>>((const float*)(s + o_gate), (const float*)(s + o_up), cnt + 3, out_pe, gated_op,
                                                                                      (__nv_bfloat16*)(s + o_gb));
            if ((e = cudaGetLastError()) != cudaSuccess) break;
        }
        if ((rc = gemm_tensor_grouped_dev(ctx, down, s + o_gb, pairs, (float*)(s + o_down), hidden, (const TcTile*)(s + o_tdn), cnt + 2, max_dn, tile_tokens, st)) != FQ_OK) break;
        const size_t total = (size_t)seq * hidden;
        blocks = (int)((total + 255) / 256);
        launch_combine((const float*)(s + o_down), weights_dev, inv, seq, hidden, top_k, out_dev, st);
        e = cudaGetLastError();
    } while (false);
    g_trace.launches += 6;
    if (e != cudaSuccess) rc = cuda_fail(e, "MoE tensor-path launch");
    dev_free_on(s, st);  // stream-ordered reuse: no host wait
    return rc;
}

// Upper bound of table entries: every expert run ends in at most one partial group (no more runs than
// experts or pairs) and holds count / group_rows full ones; never more entries than pairs.
int max_desc_for(int pairs, int n_expert, int group_rows) {
    const int bound = (pairs < n_expert ? pairs : n_expert) + pairs / group_rows;
    return bound < pairs ? bound : pairs;
}

int moe_layer_dev_impl(Ctx* ctx, const DevWeights& gate, const DevWeights& up, const DevWeights& down, const float* x_dev,
                       int seq, int top_k, const int* selected_dev, const float* weights_dev, Shard shard, float* out_dev,
                       cudaStream_t st, int gated_op = 0, StageTaps taps = StageTaps{nullptr, nullptr}) {
    // gate and up share a format; down may come in another (Gemma: Q4_K gate/up, Q8_0 down)
    const int hidden = gate.k, out_pe = gate.n, n_expert = gate.n_mats, fmt = gate.fmt, fmt_dn = down.fmt;
    const int pairs = seq * top_k;
    // prefill-sized batches: bf16 tensor-core products (the reference's own GPU arm multiplies rounded
    // operands too); decode-sized batches keep the CPU kernels' int8 arithmetic
    // the grouped tensor-core form is exercised for the formats expert stacks come in (K-quants, Q6_K down tensors of
    // the mixed K-quant files included, and Q8_0)
    auto stack_fmt = [](int f) { return f == FQ_Q4_K || f == FQ_Q5_K || f == FQ_Q6_K || f == FQ_Q8_0; };
    const bool tc_ok = stack_fmt(fmt) && stack_fmt(fmt_dn) && tensor_path_serves(gate) && tensor_path_serves(down);
    const bool tapped = taps.g_pairs || taps.down_pairs;  // the taps read the integer arm's intermediates
    if (!tapped && tc_ok && (g_moe_tensor_mode == 1 || (g_moe_tensor_mode < 0 && pairs >= 17 * n_expert)))
        return moe_layer_tensor_impl(ctx, gate, up, down, x_dev, seq, top_k, selected_dev, weights_dev, shard, out_dev, st, gated_op);
    const ActSizes Sx = act_sizes(fmt, hidden), Sg = act_sizes(fmt_dn, out_pe);
    // Row tile of the grouped kernel. A router sends a token to distinct experts, so an expert's run is
    // normally no longer than the batch; runs are split at this size either way, so repeated experts in
    // one token only cost an extra table entry.
    // K-quant expert stacks stream through the row-per-lane kernel (runs of <= 8 rows, activations quantised
    // inside the kernel); other formats take the lane-per-chunk kernel with pre-quantised rows. The choice is made per
    // product: a layer with K-quant gate/up stacks and a Q8_0 down stack (Gemma) streams its gate/up product.
    const int stream_rows = seq < expert_rows_max_group() ? seq : expert_rows_max_group();
    const bool stream_gu = expert_rows_eligible(gate, &up, stream_rows), stream_dn = expert_rows_eligible(down, nullptr, stream_rows);
    // rows per table entry: what every kernel that will run takes. The lane-per-chunk kernel keeps a group's (padded)
    // rows in shared memory, so a product it serves cuts the group until they fit.
    int rows_cap = (stream_gu || stream_dn) ? expert_rows_max_group() : kGroupRows;
    if (!stream_gu && gemv_rows_that_fit(fmt, (size_t)hidden) < rows_cap) rows_cap = gemv_rows_that_fit(fmt, (size_t)hidden);
    if (!stream_dn && gemv_rows_that_fit(fmt_dn, (size_t)out_pe) < rows_cap) rows_cap = gemv_rows_that_fit(fmt_dn, (size_t)out_pe);
    if (rows_cap == 0) return fail(FQ_DECLINED_ARGS, "expert rows of %d / %d elements are too long for the integer arm", hidden, out_pe);
    const int group_rows = seq < rows_cap ? seq : rows_cap;
    const int max_desc = max_desc_for(pairs, n_expert, group_rows);
    // one scratch block: order, inv, n_desc, table, quantised x rows, g rows, quantised g rows, down rows
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off += (bytes + 255) & ~(size_t)255;
        return o;
    };
    const size_t o_order = take(sizeof(int) * pairs), o_inv = take(sizeof(int) * pairs), o_nd = take(sizeof(int) * 2);
    const size_t o_table = take(sizeof(GroupDesc) * max_desc), o_qx = take(Sx.row * pairs);
    const size_t o_g = take(sizeof(float) * (size_t)pairs * out_pe), o_qg = take(Sg.row * pairs);
    const size_t o_down = take(sizeof(float) * (size_t)pairs * hidden);
    uint8_t* scratch = (uint8_t*)dev_alloc_on(off, st);
    if (!scratch) return fail(FQ_DECLINED_BUDGET, "MoE scratch allocation of %zu bytes failed", off);
    int* order = (int*)(scratch + o_order);
    int* inv = (int*)(scratch + o_inv);
    int* n_desc = (int*)(scratch + o_nd);
    GroupDesc* table = (GroupDesc*)(scratch + o_table);
    uint8_t* qx = scratch + o_qx;
    float* g = (float*)(scratch + o_g);
    uint8_t* qg = scratch + o_qg;
    float* down_rows = (float*)(scratch + o_down);

    cudaError_t e = cudaSuccess;
    int rc = FQ_OK;
    do {
        // positions past a shard's own rows are read by the gather below: point them at pair 0
        if (shard.skip_foreign && (e = cudaMemsetAsync(order, 0, sizeof(int) * pairs, st)) != cudaSuccess) break;
        if ((e = launch_pdl(route_plan_kernel, dim3(1), dim3(1024), sizeof(int) * 4 * n_expert, st, selected_dev, pairs, n_expert, shard, group_rows, order,
                            inv, table, n_desc, n_desc + 1, 0, 0, 0, (TcTile*)nullptr, (int*)nullptr, (TcTile*)nullptr, (int*)nullptr)) != cudaSuccess)
            break;
        if (stream_gu) {
            if ((e = launch_expert_rows(gate, &up, x_dev, order, top_k, g, table, n_desc, max_desc, group_rows, ctx->sm_count, ctx->status_dev,
                                        st, gated_op)) != cudaSuccess)
                break;
        } else {
            // gather each pair's token row and quantise it, in expert order
            if ((e = launch_quantize_acts_layout(x_dev, order, top_k, pairs, hidden, fmt, qx, st)) != cudaSuccess) break;
            GemvArgs ga{gate, up, 0, qx, g, group_rows, out_pe, 0, table, n_desc, max_desc, gated_op};
            if ((e = launch_gemv(ga, ctx->sm_count, st)) != cudaSuccess) break;
        }
        if (stream_dn) {
            if ((e = launch_expert_rows(down, nullptr, g, nullptr, 1, down_rows, table, n_desc, max_desc, group_rows, ctx->sm_count,
                                        ctx->status_dev, st)) != cudaSuccess)
                break;
        } else {
            if ((e = launch_quantize_acts_layout(g, nullptr, 1, pairs, out_pe, fmt_dn, qg, st)) != cudaSuccess) break;
            GemvArgs gd{down, DevWeights{}, 0, qg, down_rows, group_rows, hidden, 0, table, n_desc, max_desc};
            if ((e = launch_gemv(gd, ctx->sm_count, st)) != cudaSuccess) break;
        }
        launch_combine(down_rows, weights_dev, inv, seq, hidden, top_k, out_dev, st);
        e = cudaGetLastError();
    } while (false);
    g_trace.launches += 6;
    if (e == cudaSuccess && rc == FQ_OK && tapped) {
        if (taps.g_pairs) stages_to_pair_order_kernel<<<148 * 4, 256, 0, st>>>(g, inv, pairs, out_pe, taps.g_pairs);
        if (taps.down_pairs) stages_to_pair_order_kernel<<<148 * 4, 256, 0, st>>>(down_rows, inv, pairs, hidden, taps.down_pairs);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) rc = cuda_fail(e, "MoE layer launch");
    dev_free_on(scratch, st);  // stream-ordered reuse: no host wait
    return rc;
}

int check_moe(const fq_weights* gate, const fq_weights* up, const fq_weights* down, size_t seq, size_t top_k, int gated_op,
              bool shard = false) {
    if (!gate || !up || !down) return fail(FQ_DECLINED_ARGS, "null weights");
    if (gated_op < FQ_GATED_SWIGLU || gated_op > FQ_GATED_SITU) return fail(FQ_DECLINED_ARGS, "gated_op %d is not one of FQ_GATED_*", gated_op);
    const DevWeights &g = gate->dw, &u = up->dw, &d = down->dw;
    if (g.fmt != u.fmt) return fail(FQ_DECLINED_ARGS, "gate and up must share one format");
    if (g.n != u.n || g.k != u.k || g.n_mats != u.n_mats || d.n_mats != g.n_mats || d.n != g.k || d.k != g.n)
        return fail(FQ_DECLINED_ARGS, "expert tensor shapes are inconsistent");
    if (seq == 0 || top_k == 0 || (!shard && top_k > (size_t)g.n_mats)) return fail(FQ_DECLINED_ARGS, "bad seq/top_k");
    if (seq * top_k > (size_t)1 << 24) return fail(FQ_DECLINED_ARGS, "too many routed pairs");
    if (g.n_mats > 3072) return fail(FQ_DECLINED_ARGS, "too many experts");  // the route plan keeps four ints per expert in 48 KB of shared memory
    const ActLayout L = act_layout(d.fmt);
    if (g.n % L.act_block != 0 || g.n % format_info(d.fmt).block_elems != 0)
        return fail(FQ_DECLINED_ARGS, "expert width %d is not a whole number of blocks", g.n);
    return FQ_OK;
}

// grow-only staging panels of the grouped entry (backend/cuda.zig:2181-2234)
std::mutex g_qmoe_lock;
struct QMoeStage {
    float *in = nullptr, *out = nullptr;
    size_t in_bytes = 0, out_bytes = 0;
} g_stage;

}  // namespace

int moe_layer_shard_dev(Ctx* ctx, const DevWeights& gate, const DevWeights& up, const DevWeights& down, const float* x_dev, int seq,
                        int top_k, const int* selected_dev, const float* weights_dev, int expert_base, float* partial_dev, cudaStream_t st,
                        int gated_op) {
    return moe_layer_dev_impl(ctx, gate, up, down, x_dev, seq, top_k, selected_dev, weights_dev, Shard{expert_base, 1}, partial_dev, st, gated_op);
}

}  // namespace fq

using namespace fq;

extern "C" {

int fq_router_topk_dev(const float* logits_dev, size_t seq, size_t n_expert, size_t top_k, int normalize, int32_t* selected_dev,
                       float* weights_dev, void* stream) {
    if (!logits_dev || !selected_dev || !weights_dev) return fail(FQ_DECLINED_ARGS, "null pointer");
    if (top_k == 0 || top_k > n_expert || top_k > (size_t)kMaxTopK || seq == 0) return fail(FQ_DECLINED_ARGS, "bad top_k");
    if (n_expert > (size_t)kMaxRouterExperts) return fail(FQ_DECLINED_ARGS, "more than %d experts", kMaxRouterExperts);
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    cudaStream_t st = stream ? (cudaStream_t)stream : ctx->stream;
    // a warp per row with 2 x experts floats of shared memory each
    const int warps = n_expert <= 1024 ? 4 : 1;
    cudaError_t e = launch_pdl(router_topk_kernel, dim3((unsigned)((seq + warps - 1) / warps)), dim3(warps * 32), sizeof(float) * 2 * n_expert * warps, st,
                               logits_dev, (int)seq, (int)n_expert, (int)top_k, normalize, selected_dev, weights_dev);
    g_trace.launches++;
    return e == cudaSuccess ? FQ_OK : cuda_fail(e, "router launch");
}

int fq_moe_layer_dev(const fq_weights* gate, const fq_weights* up, const fq_weights* down, const float* x_dev, size_t seq,
                     size_t top_k, const int32_t* selected_dev, const float* weights_dev, int gated_op, float* out_dev, void* stream) {
    if (int rc = check_moe(gate, up, down, seq, top_k, gated_op)) return rc;
    if (!x_dev || !selected_dev || !weights_dev || !out_dev) return fail(FQ_DECLINED_ARGS, "null pointer");
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    g_trace.calls++;
    return moe_layer_dev_impl(ctx, gate->dw, up->dw, down->dw, x_dev, (int)seq, (int)top_k, selected_dev, weights_dev, Shard{0, 0},
                              out_dev, stream ? (cudaStream_t)stream : ctx->stream, gated_op);
}

int fq_moe_layer_ep_dev(const fq_weights* gate, const fq_weights* up, const fq_weights* down, const float* x_dev, size_t seq,
                        size_t top_k, const int32_t* selected_dev, const float* weights_dev, int expert_base, int gated_op,
                        float* partial_dev, void* stream) {
    if (int rc = check_moe(gate, up, down, seq, top_k, gated_op, true)) return rc;
    if (!x_dev || !selected_dev || !weights_dev || !partial_dev) return fail(FQ_DECLINED_ARGS, "null pointer");
    if (expert_base < 0) return fail(FQ_DECLINED_ARGS, "negative expert_base");
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    g_trace.calls++;
    return moe_layer_dev_impl(ctx, gate->dw, up->dw, down->dw, x_dev, (int)seq, (int)top_k, selected_dev, weights_dev,
                              Shard{expert_base, 1}, partial_dev, stream ? (cudaStream_t)stream : ctx->stream, gated_op);
}

int fq_moe_layer(const fq_weights* gate, const fq_weights* up, const fq_weights* down, const float* x, size_t seq, size_t top_k,
                 const int64_t* selected, const float* weights, int gated_op, float* out) {
    if (int rc = check_moe(gate, up, down, seq, top_k, gated_op)) return rc;
    if (!x || !selected || !weights || !out) return fail(FQ_DECLINED_ARGS, "null pointer");
    const size_t pairs = seq * top_k, hidden = (size_t)gate->dw.k;
    std::vector<int32_t> sel32(pairs);
    for (size_t p = 0; p < pairs; ++p) {
        // the reference returns IndexOutOfBounds before doing any work (exec/moe_chain.zig:243)
        if (selected[p] < 0 || selected[p] >= gate->dw.n_mats) return fail(FQ_DECLINED_ARGS, "selected[%zu]=%lld out of range", p, (long long)selected[p]);
        sel32[p] = (int32_t)selected[p];
    }
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    g_trace.calls++;
    const size_t xb = seq * hidden * sizeof(float), sb = pairs * sizeof(int32_t), wb = pairs * sizeof(float);
    const size_t o_sel = (xb + 255) & ~(size_t)255, o_w = o_sel + ((sb + 255) & ~(size_t)255), o_out = o_w + ((wb + 255) & ~(size_t)255);
    const size_t total = o_out + xb;
    uint8_t* dev = (uint8_t*)dev_alloc(total);
    uint8_t* pin = (uint8_t*)pin_alloc(total);
    int rc = FQ_OK;
    if (!dev || !pin) rc = fail(FQ_DECLINED_BUDGET, "MoE staging allocation failed");
    if (rc == FQ_OK) {
        memcpy(pin, x, xb);
        memcpy(pin + o_sel, sel32.data(), sb);
        memcpy(pin + o_w, weights, wb);
        cudaError_t e = cudaMemcpyAsync(dev, pin, o_out, cudaMemcpyHostToDevice, ctx->stream);
        g_trace.h2d_bytes += xb + sb + wb;
        if (e != cudaSuccess) rc = cuda_fail(e, "MoE upload");
    }
    if (rc == FQ_OK)
        rc = moe_layer_dev_impl(ctx, gate->dw, up->dw, down->dw, (const float*)dev, (int)seq, (int)top_k, (const int*)(dev + o_sel),
                                (const float*)(dev + o_w), Shard{0, 0}, (float*)(dev + o_out), ctx->stream, gated_op);
    if (rc == FQ_OK) {
        cudaError_t e = cudaMemcpyAsync(pin + o_out, dev + o_out, xb, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        g_trace.d2h_bytes += xb;
        if (e != cudaSuccess) rc = cuda_fail(e, "MoE download");
        else if ((rc = device_status(ctx)) == FQ_OK) memcpy(out, pin + o_out, xb);
    }
    cudaStreamSynchronize(ctx->stream);
    dev_free(dev);
    pin_free(pin);
    return rc;
}

// Expert layer over multi-plane ternary (PTQTP) experts (exec/moe.zig:51-78 `MoePtqtpRhs`, :591-631
// `moePtqtpTileDotRange`): each projection is n_planes TQ2_0 expert stacks; the grouped integer kernel runs once
// per plane and adds into the same rows (plane 0 stores, later planes accumulate: dot_p0 + dot_p1 (+ dot_p2)
// per element, left to right), the gated activation follows on the summed gate and up rows, g is requantised
// once and the down planes accumulate the same way.
int fq_moe_layer_ptqtp_dev(const fq_weights* const* gate_planes, const fq_weights* const* up_planes, const fq_weights* const* down_planes,
                           int n_planes, const float* x_dev, size_t seq, size_t top_k, const int32_t* selected_dev, const float* weights_dev,
                           int gated_op, float* out_dev, void* stream) {
    if (!gate_planes || !up_planes || !down_planes || n_planes < 1 || n_planes > 3) return fail(FQ_DECLINED_ARGS, "one to three planes per projection");
    for (int p = 0; p < n_planes; ++p) {
        if (int rc = check_moe(gate_planes[p], up_planes[p], down_planes[p], seq, top_k, gated_op)) return rc;
        const DevWeights &g0 = gate_planes[0]->dw, &g = gate_planes[p]->dw, &d = down_planes[p]->dw;
        if (g.fmt != FQ_TQ2_0 || d.fmt != FQ_TQ2_0) return fail(FQ_DECLINED_ARGS, "PTQTP planes are TQ2_0 tensors");
        if (g.n != g0.n || g.k != g0.k || g.n_mats != g0.n_mats) return fail(FQ_DECLINED_ARGS, "plane shapes differ");
    }
    if (!x_dev || !selected_dev || !weights_dev || !out_dev) return fail(FQ_DECLINED_ARGS, "null pointer");
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> lk(g_dispatch_lock);
    g_trace.calls++;
    cudaStream_t st = stream ? (cudaStream_t)stream : ctx->stream;
    const DevWeights& g0 = gate_planes[0]->dw;
    const int hidden = g0.k, out_pe = g0.n, n_expert = g0.n_mats, fmt = FQ_TQ2_0;
    const int pairs = (int)(seq * top_k);
    int fit_rows = gemv_rows_that_fit(fmt, (size_t)hidden);
    if (gemv_rows_that_fit(fmt, (size_t)out_pe) < fit_rows) fit_rows = gemv_rows_that_fit(fmt, (size_t)out_pe);
    if (fit_rows == 0) return fail(FQ_DECLINED_ARGS, "expert rows of %d / %d elements are too long for the integer arm", hidden, out_pe);
    const int int8_rows = kGroupRows < fit_rows ? kGroupRows : fit_rows;
    const int group_rows = (int)seq < int8_rows ? (int)seq : int8_rows;
    const int max_desc = max_desc_for(pairs, n_expert, group_rows);
    const ActSizes Sx = act_sizes(fmt, hidden), Sg = act_sizes(fmt, out_pe);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off += (bytes + 255) & ~(size_t)255;
        return o;
    };
    const size_t o_order = take(sizeof(int) * pairs), o_inv = take(sizeof(int) * pairs), o_nd = take(sizeof(int) * 2);
    const size_t o_table = take(sizeof(GroupDesc) * max_desc), o_qx = take(Sx.row * pairs);
    const size_t o_gate = take(sizeof(float) * (size_t)pairs * out_pe), o_up = take(sizeof(float) * (size_t)pairs * out_pe);
    const size_t o_qg = take(Sg.row * pairs), o_down = take(sizeof(float) * (size_t)pairs * hidden);
    uint8_t* s = (uint8_t*)dev_alloc_on(off, st);
    if (!s) return fail(FQ_DECLINED_BUDGET, "MoE scratch allocation of %zu bytes failed", off);
    int* order = (int*)(s + o_order);
    int* inv = (int*)(s + o_inv);
    int* n_desc = (int*)(s + o_nd);
    GroupDesc* table = (GroupDesc*)(s + o_table);
    float* gate_rows = (float*)(s + o_gate);
    float* up_rows = (float*)(s + o_up);  // becomes g in place
    float* down_rows = (float*)(s + o_down);
    cudaError_t e = cudaSuccess;
    do {
        route_plan_kernel<<<1, 1024, sizeof(int) * 4 * n_expert, st>>>(selected_dev, pairs, n_expert, Shard{0, 0}, group_rows, order, inv, table, n_desc,
                                                                    n_desc + 1, 0, 0, 0, nullptr, nullptr, nullptr, nullptr);
        if ((e = cudaGetLastError()) != cudaSuccess) break;
        if ((e = launch_quantize_acts_layout(x_dev, order, (int)top_k, pairs, hidden, fmt, s + o_qx, st)) != cudaSuccess) break;
        for (int p = 0; p < n_planes && e == cudaSuccess; ++p) {
            GemvArgs ga{gate_planes[p]->dw, DevWeights{}, 0, s + o_qx, gate_rows, group_rows, out_pe, p > 0, table, n_desc, max_desc};
            if ((e = launch_gemv(ga, ctx->sm_count, st)) != cudaSuccess) break;
            GemvArgs ua{up_planes[p]->dw, DevWeights{}, 0, s + o_qx, up_rows, group_rows, out_pe, p > 0, table, n_desc, max_desc};
            e = launch_gemv(ua, ctx->sm_count, st);
        }
        if (e != cudaSuccess) break;
        const size_t ng = (size_t)pairs * out_pe;
        int blocks = (int)((ng + 255) / 256);
        gated_f32_kernel<<<blocks > 148 * 8 ? 148 * 8 : blocks, 256, 0, st>>>(gate_rows, up_rows, ng, gated_op, up_rows);
        if ((e = cudaGetLastError()) != cudaSuccess) break;
        if ((e = launch_quantize_acts_layout(up_rows, nullptr, 1, pairs, out_pe, fmt, s + o_qg, st)) != cudaSuccess) break;
        for (int p = 0; p < n_planes && e == cudaSuccess; ++p) {
            GemvArgs da{down_planes[p]->dw, DevWeights{}, 0, s + o_qg, down_rows, group_rows, hidden, p > 0, table, n_desc, max_desc};
            e = launch_gemv(da, ctx->sm_count, st);
        }
        if (e != cudaSuccess) break;
        launch_combine(down_rows, weights_dev, inv, (int)seq, hidden, (int)top_k, out_dev, st);
        e = cudaGetLastError();
    } while (false);
    g_trace.launches += 5 + 3 * n_planes;
    dev_free_on(s, st);
    return e == cudaSuccess ? FQ_OK : cuda_fail(e, "PTQTP MoE layer launch");
}

// Test seam: the integer arm of the layer with its two intermediates copied out in pair order, so a test
// can hold each stage to the f32 tolerance separately (g against the CPU kernels' g; the down product
// fed the device's own g against the CPU kernels fed the same g).
int fq_moe_layer_stages_for_test(const fq_weights* gate, const fq_weights* up, const fq_weights* down, const float* x_dev, size_t seq,
                                 size_t top_k, const int32_t* selected_dev, const float* weights_dev, float* g_pairs_dev,
                                 float* down_pairs_dev, float* out_dev) {
    if (int rc = check_moe(gate, up, down, seq, top_k, 0)) return rc;
    if (!x_dev || !selected_dev || !weights_dev || !out_dev) return fail(FQ_DECLINED_ARGS, "null pointer");
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    return moe_layer_dev_impl(ctx, gate->dw, up->dw, down->dw, x_dev, (int)seq, (int)top_k, selected_dev, weights_dev, Shard{0, 0},
                              out_dev, ctx->stream, 0, StageTaps{g_pairs_dev, down_pairs_dev});
}

// Test seam in the spirit of setQuantMmaForTest (backend/cuda.zig:2563): -1 auto, 0 integer path, 1 tensor path.
void fq_set_moe_tensor_for_test(int mode) { g_moe_tensor_mode = mode < 0 ? -1 : (mode ? 1 : 0); }
void fq_set_group_grid_limit_for_test(int limit) { set_gemv_grid_y_limit(limit); }

// ---- grouped GEMM over staged panels (backend/cuda.zig:2181-2333) ------------
void fq_qmoe_lock(void) { g_qmoe_lock.lock(); }
void fq_qmoe_unlock(void) { g_qmoe_lock.unlock(); }

int fq_qmoe_stage(size_t in_bytes, size_t out_bytes, float** in, float** out) {
    if (!in || !out || in_bytes == 0 || out_bytes == 0) return fail(FQ_DECLINED_ARGS, "bad stage request");
    if (!context()) return FQ_DECLINED_NO_GPU;
    if (g_stage.in_bytes < in_bytes) {
        pin_free(g_stage.in);
        g_stage.in = (float*)pin_alloc(in_bytes);
        g_stage.in_bytes = g_stage.in ? in_bytes : 0;
    }
    if (g_stage.out_bytes < out_bytes) {
        pin_free(g_stage.out);
        g_stage.out = (float*)pin_alloc(out_bytes);
        g_stage.out_bytes = g_stage.out ? out_bytes : 0;
    }
    if (!g_stage.in || !g_stage.out) return fail(FQ_DECLINED_BUDGET, "pinned panel allocation failed");
    *in = g_stage.in;
    *out = g_stage.out;
    return FQ_OK;
}

}  // extern "C"

// A run: consecutive activation rows [row0, row0 + m) of the staged panel that one expert multiplies. The caller's
// tiles (32 rows each in the reference's builder, llm/gemma/moe.zig:773-787) of one expert over adjoining rows
// merge into one run, so the expert's weights stream once per run, not once per tile.
struct GroupedRun {
    int expert, row0, m;
};
// Runs at least this long multiply on the tensor cores (bf16 operands, as the reference's own grouped arm rounds its
// operands, backend/cuda/kernels.cu:340-379); shorter ones keep the CPU kernels' int8 arithmetic.
constexpr int kGroupedTensorRows = 17;
constexpr int kQmmTileRows = 32;  // NR1 of the reference's tile kernels (backend/cuda/kernels.cu:168)
static int g_grouped_tensor_mode = -1;  // test seam: -1 by run length, 0 never, 1 every run the format allows

extern "C" void fq_set_grouped_tensor_for_test(int mode) { g_grouped_tensor_mode = mode < 0 ? -1 : (mode ? 1 : 0); }

extern "C" int fq_gemm_q_grouped_nt(int fmt, const void* rhs, size_t rhs_len, int cacheable, size_t nb01, size_t nb02, size_t n_out,
                                    size_t k, const fq_qmm_tile* tiles, size_t n_tiles) {
    // argument rules of backend/cuda.zig:2254-2257
    const FormatInfo f = format_info(fmt);
    if (!f.block_elems) return fail(FQ_DECLINED_ARGS, "format %d is not served", fmt);
    if (k == 0 || k % 32 != 0 || k % f.block_elems != 0) return fail(FQ_DECLINED_ARGS, "k=%zu is not a whole number of blocks", k);
    if (n_out == 0 || n_out % 4 != 0) return fail(FQ_DECLINED_ARGS, "n_out=%zu is not a multiple of 4", n_out);
    if (!tiles || n_tiles == 0 || n_tiles > (1u << 24)) return fail(FQ_DECLINED_ARGS, "bad tile table");
    if (!rhs || nb01 == 0 || nb02 < nb01 * n_out) return fail(FQ_DECLINED_ARGS, "bad rhs strides");
    if (!g_stage.in || !g_stage.out) return fail(FQ_DECLINED_ARGS, "fq_qmoe_stage was not called");
    int max_expert = 0;
    size_t rows = 0;
    // rows per table entry of the integer arm: as many as the kernel's shared memory holds for this K (at most 16)
    const int fit_rows = gemv_rows_that_fit(fmt, k);
    if (fit_rows == 0) return fail(FQ_DECLINED_ARGS, "k=%zu is too long for the grouped kernel", k);
    const int group_rows = kGroupRows < fit_rows ? kGroupRows : fit_rows;
    std::vector<GroupedRun> runs;
    for (size_t t = 0; t < n_tiles; ++t) {
        // The reference's table entry (backend/cuda.zig:1503-1508, filled at llm/gemma/moe.zig:773-787 and in its own
        // test at cuda.zig:3170-3183): `base_row` and `m` are the first panel row and the row count of the expert's
        // whole group, `tile_m` is the index of this 32-row tile inside the group. The tile therefore covers panel
        // rows [base_row + 32 tile_m, base_row + min(m, 32 tile_m + 32)) (backend/cuda/kernels.cu:322-327).
        const fq_qmm_tile& tl = tiles[t];
        if (tl.expert < 0 || tl.base_row < 0 || tl.m <= 0 || tl.tile_m < 0 || (long long)tl.tile_m * kQmmTileRows >= tl.m)
            return fail(FQ_DECLINED_ARGS, "tile %zu is malformed", t);
        const int first = tl.tile_m * kQmmTileRows;
        const int row0 = tl.base_row + first;
        const int cnt = tl.m - first < kQmmTileRows ? tl.m - first : kQmmTileRows;
        if (row0 < 0) return fail(FQ_DECLINED_ARGS, "tile %zu is malformed", t);
        if (tl.expert > max_expert) max_expert = tl.expert;
        if ((size_t)row0 + cnt > rows) rows = (size_t)row0 + cnt;
        if (!runs.empty() && runs.back().expert == tl.expert && runs.back().row0 + runs.back().m == row0) runs.back().m += cnt;
        else runs.push_back({tl.expert, row0, cnt});
    }
    if (rows * k * sizeof(float) > g_stage.in_bytes || rows * n_out * sizeof(float) > g_stage.out_bytes)
        return fail(FQ_DECLINED_ARGS, "tiles reach beyond the staged panels");
    const size_t n_mats = (size_t)max_expert + 1;
    if (rhs_len < nb02 * (n_mats - 1) + nb01 * n_out) return fail(FQ_DECLINED_ARGS, "rhs_len too short for expert %d", max_expert);
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    g_trace.calls++;
    DevWeights view;
    fq_weights* temp = nullptr;
    int rc = resolve_rhs(ctx, fmt, rhs, rhs_len, cacheable, nb01, nb02, n_out, k, n_mats, &view, &temp);
    if (rc != FQ_OK) return rc;
    // split the runs over the two arms
    const bool tc_ok = g_grouped_tensor_mode != 0 && tensor_path_serves(view) && k % 256 == 0;
    std::vector<GroupDesc> descs;
    std::vector<TcTile> tc;
    const int row_tiles = (int)((n_out + 127) / 128);
    for (const GroupedRun& r : runs) {
        if (tc_ok && (g_grouped_tensor_mode == 1 || r.m >= kGroupedTensorRows)) {
            for (int t0 = 0; t0 < r.m; t0 += 128)
                for (int rt = 0; rt < row_tiles; ++rt) tc.push_back({r.expert, rt, r.row0 + t0, r.m - t0 < 128 ? r.m - t0 : 128});
        } else {
            for (int j = 0; j < r.m; j += group_rows) descs.push_back({r.expert, r.row0 + j, r.m - j < group_rows ? r.m - j : group_rows, 0});
        }
    }
    if (descs.size() > (size_t)INT32_MAX / 2 || tc.size() > (size_t)INT32_MAX / 2) {
        if (temp) fq_weights_free(temp);
        return fail(FQ_DECLINED_ARGS, "tile table too large");
    }
    const ActSizes S = act_sizes(fmt, k);
    const size_t in_b = rows * k * sizeof(float), out_b = rows * n_out * sizeof(float);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off += (bytes + 255) & ~(size_t)255;
        return o;
    };
    const size_t o_in = take(in_b), o_out = take(out_b), o_q = take(descs.empty() ? 0 : S.row * rows), o_bf = take(tc.empty() ? 0 : rows * k * 2);
    const size_t tab_b = descs.size() * sizeof(GroupDesc), tc_b = tc.size() * sizeof(TcTile);
    const size_t o_tab = take(tab_b), o_tc = take(tc_b), o_nd = take(2 * sizeof(int));
    uint8_t* dev = (uint8_t*)dev_alloc(off);
    // one page-locked block for both tables and their counts: [descs][tiles][n_desc, n_tiles]
    const size_t p_tc = (tab_b + 15) & ~(size_t)15, p_nd = p_tc + ((tc_b + 15) & ~(size_t)15);
    uint8_t* pin = (uint8_t*)pin_alloc(p_nd + 2 * sizeof(int));
    if (!dev || !pin) rc = fail(FQ_DECLINED_BUDGET, "grouped staging allocation failed");
    cudaError_t e = cudaSuccess;
    if (rc == FQ_OK) {
        if (tab_b) memcpy(pin, descs.data(), tab_b);
        if (tc_b) memcpy(pin + p_tc, tc.data(), tc_b);
        int* pin_nd = (int*)(pin + p_nd);
        pin_nd[0] = (int)descs.size(), pin_nd[1] = (int)tc.size();
        do {
            if ((e = cudaMemcpyAsync(dev + o_in, g_stage.in, in_b, cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess) break;
            if (tab_b && (e = cudaMemcpyAsync(dev + o_tab, pin, tab_b, cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess) break;
            if (tc_b && (e = cudaMemcpyAsync(dev + o_tc, pin + p_tc, tc_b, cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess) break;
            if ((e = cudaMemcpyAsync(dev + o_nd, pin_nd, 2 * sizeof(int), cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess) break;
            // rows no tile names keep whatever the out panel held: copy it up first
            if ((e = cudaMemcpyAsync(dev + o_out, g_stage.out, out_b, cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess) break;
            if (!descs.empty()) {
                if ((e = launch_quantize_acts_layout((const float*)(dev + o_in), nullptr, 1, (int)rows, (int)k, fmt, dev + o_q, ctx->stream)) != cudaSuccess) break;
                GemvArgs ga{view, DevWeights{}, 0, dev + o_q, (float*)(dev + o_out), group_rows, (int)n_out, 0, (const GroupDesc*)(dev + o_tab),
                            (const int*)(dev + o_nd), (int)descs.size()};
                if ((e = launch_gemv(ga, ctx->sm_count, ctx->stream)) != cudaSuccess) break;
                g_trace.launches += 2;
            }
            if (!tc.empty()) {
                if ((e = launch_f32_to_bf16((const float*)(dev + o_in), dev + o_bf, rows * k, ctx->stream)) != cudaSuccess) break;
                g_trace.launches++;
                rc = gemm_tensor_grouped_dev(ctx, view, dev + o_bf, rows, (float*)(dev + o_out), n_out, (const TcTile*)(dev + o_tc), (const int*)(dev + o_nd) + 1,
                                             (int)tc.size(), 128, ctx->stream);
                if (rc != FQ_OK) break;
            }
            if ((e = cudaMemcpyAsync(g_stage.out, dev + o_out, out_b, cudaMemcpyDeviceToHost, ctx->stream)) != cudaSuccess) break;
            e = cudaStreamSynchronize(ctx->stream);
        } while (false);
        g_trace.h2d_bytes += in_b + out_b;
        g_trace.d2h_bytes += out_b;
        if (e != cudaSuccess) rc = cuda_fail(e, "grouped GEMM");
    }
    cudaStreamSynchronize(ctx->stream);
    if (rc == FQ_OK) rc = device_status(ctx);
    dev_free_idle(dev);
    pin_free(pin);
    if (temp) fq_weights_free(temp);
    return rc;
}
