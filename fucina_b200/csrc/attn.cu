// Streaming attention forward: online-softmax grouped attention over an f16 or f32 KV cache.
//
// The reference provider has one kernel for it (src/backend/cuda/kernels.cu:574-681 `fucina_attn_fwd_{f16,f32}`, host
// side src/backend/cuda.zig:2601-2736): one warp per query row walks the whole key range. Same contract here --
// q [q_seq][heads][d] f32, k/v [kv_seq][kv_heads][d], per-head kv map, query row i at absolute position
// source_offset + i, causal with an optional sliding window or bidirectional, optional {row max, sum exp} stats --
// but the key range of a (row, head) is cut into splits that run on different SMs (a decode step has one query row and
// thousands of keys), each split walked by four warps, and a second kernel merges the splits' (max, sum, accumulator)
// triples. Everything is f32 arithmetic in a fixed order: results do not depend on the grid.
//
// Bound: HBM (K and V bytes are read once per head that maps to them; heads sharing a kv head hit L2).
#include <cuda_fp16.h>

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

// four consecutive values of a V row (8 or 16 bytes)
__device__ __forceinline__ float4 load4(const __half* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }

// dot of the staged (pre-scaled) query row with one key row, 16 bytes of K per load
__device__ __forceinline__ float key_dot(const float* sq, const __half* krow, int d) {
    float dot = 0.0f;
#pragma unroll 4
    for (int t = 0; t < d; t += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(krow + t);
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
        const float4 q0 = *reinterpret_cast<const float4*>(sq + t), q1 = *reinterpret_cast<const float4*>(sq + t + 4);  // broadcast reads
        const float2 k0 = __half22float2(h[0]), k1 = __half22float2(h[1]), k2 = __half22float2(h[2]), k3 = __half22float2(h[3]);
        dot = fmaf(q0.x, k0.x, dot);
        dot = fmaf(q0.y, k0.y, dot);
        dot = fmaf(q0.z, k1.x, dot);
        dot = fmaf(q0.w, k1.y, dot);
        dot = fmaf(q1.x, k2.x, dot);
        dot = fmaf(q1.y, k2.y, dot);
        dot = fmaf(q1.z, k3.x, dot);
        dot = fmaf(q1.w, k3.y, dot);
    }
    return dot;
}
__device__ __forceinline__ float key_dot(const float* sq, const float* krow, int d) {
    float dot = 0.0f;
#pragma unroll 8
    for (int t = 0; t < d; t += 4) {
        const float4 kk = *reinterpret_cast<const float4*>(krow + t);
        const float4 qq = *reinterpret_cast<const float4*>(sq + t);
        dot = fmaf(qq.x, kk.x, dot);
        dot = fmaf(qq.y, kk.y, dot);
        dot = fmaf(qq.z, kk.z, dot);
        dot = fmaf(qq.w, kk.w, dot);
    }
    return dot;
}

// grid (splits, heads, q_seq), 4 warps: warp w takes the 32-key steps w, w + 4, ... of the split
template <typename KVT>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_split_kernel(const AttnArgs A) {
    __shared__ __align__(16) float sh_q[kAttnMaxD];
    __shared__ float sh_p[kAttnWarps][32];
    __shared__ float sh_m[kAttnWarps], sh_l[kAttnWarps];
    __shared__ float sh_acc[kAttnWarps][kAttnMaxD];
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s = blockIdx.x, h = blockIdx.y, qi = blockIdx.z;
    const int d = A.d, kvh = A.kvmap[h];
    const KVT* K = reinterpret_cast<const KVT*>(A.k);
    const KVT* V = reinterpret_cast<const KVT*>(A.v);

    const float* qrow = A.q + ((size_t)qi * A.heads + h) * d;
    for (int t = threadIdx.x; t < d; t += kAttnWarps * 32) sh_q[t] = qrow[t] * A.scale;
    __syncthreads();

    // this row's key range (kernels.cu:600-602), cut to the split
    const int p_abs = A.source_offset + qi;
    int end = A.causal ? min(p_abs + 1, A.kv_seq) : A.kv_seq;
    int start = (A.causal && A.window > 0 && p_abs + 1 > A.window) ? (p_abs + 1 - A.window) : 0;
    start = max(start, s * A.split_len);
    end = min(end, (s + 1) * A.split_len);

    constexpr int ND = kAttnMaxD / 128;  // lane holds the four dims from (lane + 32 * t) * 4
    float acc[ND][4];
#pragma unroll
    for (int t = 0; t < ND; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f;
    float m_run = kNegBig, l_run = 0.0f;

    for (int j0 = start + w * 32; j0 < end; j0 += kAttnWarps * 32) {
        const int j = j0 + lane;
        float sc = kNegBig;
        if (j < end) sc = key_dot(sh_q, K + ((size_t)j * A.kv_heads + kvh) * d, d);
        float m_tile = sc;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, off));
        const float m_new = fmaxf(m_run, m_tile);
        const float p = (j < end) ? expf(sc - m_new) : 0.0f;
        const float rescale = (m_run > -3.0e38f) ? expf(m_run - m_new) : 0.0f;
        float p_sum = p;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) p_sum += __shfl_xor_sync(0xffffffffu, p_sum, off);
        l_run = l_run * rescale + p_sum;
        m_run = m_new;
        sh_p[w][lane] = p;
        __syncwarp();
        const int jn = min(32, end - j0);
        const size_t vstride = (size_t)A.kv_heads * d;
#pragma unroll
        for (int t = 0; t < ND; ++t) {
            const int dim = (lane + 32 * t) * 4;
            float a0 = acc[t][0] * rescale, a1 = acc[t][1] * rescale, a2 = acc[t][2] * rescale, a3 = acc[t][3] * rescale;
            if (dim < d) {
                const KVT* vbase = V + ((size_t)j0 * A.kv_heads + kvh) * d + dim;
                // eight rows of V in flight before their multiply-adds: the loads of a group do not wait for one another
                for (int jj0 = 0; jj0 < jn; jj0 += 8) {
                    float4 vv[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        vv[u] = (jj0 + u < jn) ? load4(vbase + (size_t)(jj0 + u) * vstride) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const float pj = sh_p[w][jj0 + u];  // zero past the row's last key
                        a0 = fmaf(pj, vv[u].x, a0);
                        a1 = fmaf(pj, vv[u].y, a1);
                        a2 = fmaf(pj, vv[u].z, a2);
                        a3 = fmaf(pj, vv[u].w, a3);
                    }
                }
            }
            acc[t][0] = a0, acc[t][1] = a1, acc[t][2] = a2, acc[t][3] = a3;
        }
        __syncwarp();
    }

    // merge the four warps in warp order
    if (lane == 0) sh_m[w] = m_run, sh_l[w] = l_run;
#pragma unroll
    for (int t = 0; t < ND; ++t) {
        const int dim = (lane + 32 * t) * 4;
        if (dim < d) sh_acc[w][dim] = acc[t][0], sh_acc[w][dim + 1] = acc[t][1], sh_acc[w][dim + 2] = acc[t][2], sh_acc[w][dim + 3] = acc[t][3];
    }
    __syncthreads();
    float m = kNegBig;
    for (int i = 0; i < kAttnWarps; ++i) m = fmaxf(m, sh_m[i]);
    float l = 0.0f, f[kAttnWarps];
    for (int i = 0; i < kAttnWarps; ++i) {
        f[i] = sh_m[i] > -3.0e38f ? expf(sh_m[i] - m) : 0.0f;
        l += sh_l[i] * f[i];
    }
    float* part = A.splits > 1 ? A.part + (((size_t)qi * A.heads + h) * A.splits + s) * (d + 2) : nullptr;
    const float inv_l = l > 0.0f ? 1.0f / l : 0.0f;
    for (int dim = threadIdx.x; dim < d; dim += kAttnWarps * 32) {
        float a = 0.0f;
        for (int i = 0; i < kAttnWarps; ++i) a += sh_acc[i][dim] * f[i];
        if (part) part[2 + dim] = a;
        else A.out[((size_t)qi * A.heads + h) * d + dim] = a * inv_l;
    }
    if (threadIdx.x == 0) {
        if (part) part[0] = m, part[1] = l;
        else if (A.stats) {
            const size_t sb = ((size_t)h * A.q_seq + qi) * 2;
            A.stats[sb] = m, A.stats[sb + 1] = l;
        }
    }
}

// one CTA per (head, row): the splits' triples merged in split order
__global__ void __launch_bounds__(128) attn_merge_kernel(const AttnArgs A) {
    const int h = blockIdx.x, qi = blockIdx.y, d = A.d;
    const float* part = A.part + ((size_t)qi * A.heads + h) * A.splits * (d + 2);
    float m = kNegBig;
    for (int s = 0; s < A.splits; ++s) m = fmaxf(m, part[(size_t)s * (d + 2)]);
    float l = 0.0f;
    for (int s = 0; s < A.splits; ++s) {
        const float ms = part[(size_t)s * (d + 2)];
        l += part[(size_t)s * (d + 2) + 1] * (ms > -3.0e38f ? expf(ms - m) : 0.0f);
    }
    const float inv_l = l > 0.0f ? 1.0f / l : 0.0f;
    for (int dim = threadIdx.x; dim < d; dim += blockDim.x) {
        float a = 0.0f;
        for (int s = 0; s < A.splits; ++s) {
            const float ms = part[(size_t)s * (d + 2)];
            a += part[(size_t)s * (d + 2) + 2 + dim] * (ms > -3.0e38f ? expf(ms - m) : 0.0f);
        }
        A.out[((size_t)qi * A.heads + h) * d + dim] = a * inv_l;
    }
    if (A.stats && threadIdx.x == 0) {
        const size_t sb = ((size_t)h * A.q_seq + qi) * 2;
        A.stats[sb] = m, A.stats[sb + 1] = l;
    }
}

int check_attn(size_t q_seq, size_t kv_seq, size_t heads, size_t kv_heads, size_t d, int kv_is_f16) {
    if (q_seq == 0 || kv_seq == 0 || heads == 0 || kv_heads == 0 || d == 0) return fail(FQ_DECLINED_ARGS, "empty attention problem");
    if (d > (size_t)kAttnMaxD || heads > 512) return fail(FQ_DECLINED_ARGS, "d <= 256 and heads <= 512 (backend/cuda.zig:617-625)");
    if (d % (kv_is_f16 ? 8 : 4) != 0) return fail(FQ_DECLINED_ARGS, "d=%zu: rows of K and V are read 16 bytes at a time", d);
    if (q_seq > 65535 || heads > 65535 || kv_seq > (size_t)INT32_MAX) return fail(FQ_DECLINED_ARGS, "attention problem too large for one launch");
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
    if (!gpu_enabled()) return fail(FQ_DECLINED_GATE, "disabled by FUCINA_GPU=0");
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    g_trace.calls++;
    cudaStream_t st = stream ? (cudaStream_t)stream : ctx->stream;
    // splits: enough CTAs for about four per SM, at least 128 keys (one step of every warp) each
    const size_t rows = q_seq * heads;
    size_t splits = ((size_t)4 * ctx->sm_count + rows - 1) / rows;
    const size_t max_splits = (kv_seq + 127) / 128;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    size_t split_len = ((kv_seq + splits - 1) / splits + 127) / 128 * 128;
    splits = (kv_seq + split_len - 1) / split_len;
    if (window > kv_seq) window = kv_seq;  // any window >= kv_seq is plain causal (backend/cuda.zig:2621-2625)
    float* part = nullptr;
    if (splits > 1) {
        part = (float*)dev_alloc_on(rows * splits * (d + 2) * sizeof(float), st);
        if (!part) return fail(FQ_DECLINED_BUDGET, "attention scratch allocation failed");
    }
    AttnArgs a{q_dev, k_dev, v_dev, out_dev, stats_dev, kv_head_for_head_dev, part, (int)q_seq, (int)kv_seq, (int)heads, (int)kv_heads, (int)d,
               (int)source_offset, (int)window, causal ? 1 : 0, scale, (int)splits, (int)split_len};
    const dim3 grid((unsigned)splits, (unsigned)heads, (unsigned)q_seq);
    if (kv_is_f16) attn_split_kernel<__half><<<grid, kAttnWarps * 32, 0, st>>>(a);
    else attn_split_kernel<float><<<grid, kAttnWarps * 32, 0, st>>>(a);
    cudaError_t e = cudaGetLastError();
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
