// Expert-parallel MoE layer over the GPUs of one node: tokens sharded by rank, experts split E / G per rank
// (rank r owns global experts [r * E/G, (r+1) * E/G)). No counterpart in the reference, which is
// single-device (src/backend/cuda.zig:439); the per-pair arithmetic is that of the single-GPU tensor arm
// (moe.cu), and because every routed pair is multiplied by the same kernels on the same bf16 operands,
// whichever GPU serves it, and the weighted sum runs in slot order on the token's home rank
// (src/exec/moe_chain.zig:307-330), the result equals the one-GPU tensor arm bit for bit.
//
// Fused exchange (the default when every peer's arena is mapped), per layer, epoch-numbered flags:
//   plan      histogram of this rank's pairs by global expert; the row goes into EVERY peer's count table
//             (plain peer stores), followed by a flag per peer; then the bounded wait for every rank's row.
//             The full [rank][expert] table fixes every pair's row in
//             the owning rank's token panel -- expert-major, source-rank-minor, the order one global counting
//             sort would give -- so sources write final positions and the owner multiplies whole expert runs.
//             Also builds this rank's tile lists and checks every panel's capacity (all ranks see the same table
//             and reach the same verdict).
//   dispatch  the gather IS the dispatch: each pair's token row is rounded to bf16 and stored straight into the
//             owner's panel together with its return address (source rank, pair index); then a flag per peer.
//   gate/up   grouped tcgen05 GEMM with the SwiGLU in its epilogue; its token-tile producer starts loading
//             once every source's dispatch flag is in.
//   down      grouped tcgen05 GEMM whose epilogue stores each output row straight into the return panel of
//             the rank that owns the token (f32, peer stores), then a flag per peer.
//   combine   waits for every owner's return flag, then the slot-ordered weighted sum.
// Every wait is bounded (about a second); a wait that gives up records FQ_ERR_TIMEOUT in the status word and
// the layer's output is invalid, but nothing hangs and the context stays usable.
//
// Baseline form (flag FQ_EP_NCCL, or peers not mapped): NCCL all-gather of token rows and routing, each rank
// computes the partial sums of its experts for all tokens, NCCL reduce-scatter (sum) back. Fixed sizes, no host
// synchronisation; equal to the fused form within f32 summation order.
#include <cuda_bf16.h>

#include <cstdio>
#include <cstdlib>
#include <vector>

#include "multi.h"

namespace fq {

namespace {

constexpr int kEpMaxExperts = 1024;
constexpr int kHdrInts = 8;                       // per-rank header in front of its count row
constexpr size_t kFlagBytes = 256;                // int flags[3][kMaxPeers]: counts, dispatch, return
constexpr size_t kTableBytes = sizeof(int) * kMaxPeers * (kHdrInts + kEpMaxExperts);
constexpr size_t kFixedBytes = 64 * 1024;         // flags + table, rounded up
static_assert(kFlagBytes + kTableBytes <= kFixedBytes, "fixed arena region too small");
constexpr unsigned kSpinLimit = 1u << 22;         // x ~0.2 us of sleep per poll: about a second

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait for *p >= want. False when it gave up.
__device__ __forceinline__ bool wait_flag(const int* p, int want) {
    for (unsigned i = 0; i < kSpinLimit; ++i) {
        if (ld_acquire_sys(p) >= want) return true;
        __nanosleep(200);
    }
    return false;
}

// One rank's view of the exchange (a real rank of fq_moe_layer_ep, or an emulated one of the test seam).
struct EpView {
    int rank, world;
    uint8_t* peer[kMaxPeers];
    size_t arena_bytes;
};
__host__ __device__ inline int* flags_of(uint8_t* arena, int kind) { return reinterpret_cast<int*>(arena) + kind * kMaxPeers; }
__host__ __device__ inline int* table_row(uint8_t* arena, int rank) {
    return reinterpret_cast<int*>(arena + kFlagBytes) + (size_t)rank * (kHdrInts + kEpMaxExperts);
}

// Layout of one rank's arena behind the fixed region: [ret: pairs x hidden f32][meta: rows_cap x int2][x: rows_cap x hidden bf16].
struct EpLayout {
    size_t off_ret, off_meta, off_x;
    int rows_cap;
};
EpLayout ep_layout(size_t arena_bytes, int pairs, int hidden) {
    EpLayout L;
    L.off_ret = kFixedBytes;
    const size_t ret_bytes = ((size_t)pairs * hidden * 4 + 255) & ~(size_t)255;
    const size_t rest = arena_bytes > L.off_ret + ret_bytes + 512 ? arena_bytes - L.off_ret - ret_bytes - 512 : 0;
    long long cap = (long long)(rest / ((size_t)hidden * 2 + 8));
    cap &= ~127LL;  // keeps the x panel 256-byte aligned behind the meta array
    if (cap > (1 << 24)) cap = 1 << 24;
    L.rows_cap = (int)(cap < 0 ? 0 : cap);
    L.off_meta = L.off_ret + ret_bytes;
    L.off_x = L.off_meta + (size_t)L.rows_cap * 8;
    return L;
}

// What the plan leaves for the later kernels of the layer (device memory, one per rank and layer).
struct EpPlan {
    int ok;            // 0: a wait gave up or a panel would overflow -- the later kernels do nothing
    int n_rows;        // rows arriving in this rank's panel
    int n_gu, n_dn;    // tiles of the gate/up and the down product
    int done[2];       // CTAs of the dispatch kernel / the down product that have finished (zeroed by the plan)
    unsigned long long dst_x[kMaxPeers];     // byte offset of rank d's x panel / meta array inside ITS arena
    unsigned long long dst_meta[kMaxPeers];
};

struct EpArgs {
    EpView v;
    int epoch;
    int pairs, top_k, hidden, n_expert, per;  // this rank's routed pairs; experts in total and per rank
    EpLayout mine;
    int tile_gu, tile_dn, rt_gu, rt_dn;  // token-tile widths of the two products, weight-row tiles per token tile
    const int* selected;
    int* status;
    EpPlan* plan;
    int2* pair_dst;   // [pairs] (owner rank, row in its panel)
    TcTile* t_gu;
    TcTile* t_dn;
};

// ---- plan: count, publish, wait, place ------------------------------------------------------------------
// One CTA. Histogram of this rank's pairs by global expert; the row goes into every peer's table followed by a
// flag per peer; then the bounded wait for every rank's row, and from the full table: every pair's final row in
// its owner's panel, this rank's tile lists, the capacity verdict.
// Shared memory: tbl[world][E] | tot[E] | cursor[E] | base[E] | tiles_gu[per] | tiles_dn[per]
// `stages`: bit 0 = count and publish, bit 1 = wait and place. A real rank runs both in one launch; the one-GPU
// emulation publishes for every rank first and places afterwards (no kernel may wait for one that runs later).
__global__ void ep_plan_kernel(const EpArgs A, int stages) {
    extern __shared__ int sh[];
    const int E = A.n_expert, W = A.v.world, per = A.per;
    int* tbl = sh;
    int* tot = tbl + W * E;
    int* cursor = tot + E;
    int* base = cursor + E;
    int* tiles_gu = base + E;
    int* tiles_dn = tiles_gu + per;
    __shared__ int s_ok;
    __shared__ int s_rows;
    if (threadIdx.x == 0) s_ok = 1;
    if (stages & 1) {
        // -- count and publish
        for (int e = threadIdx.x; e < E; e += blockDim.x) tot[e] = 0;
        __syncthreads();
        for (int p = threadIdx.x; p < A.pairs; p += blockDim.x) {
            const int e = A.selected[p];
            if (e >= 0 && e < E) atomicAdd(&tot[e], 1);
        }
        __syncthreads();
        for (int d = 0; d < W; ++d) {
            int* row = table_row(A.v.peer[d], A.v.rank);
            if (threadIdx.x == 0) {
                row[0] = (int)(A.mine.off_meta & 0xffffffffu), row[1] = (int)(A.mine.off_meta >> 32);
                row[2] = (int)(A.mine.off_x & 0xffffffffu), row[3] = (int)(A.mine.off_x >> 32);
                row[4] = A.mine.rows_cap;
                row[5] = A.pairs;
            }
            for (int e = threadIdx.x; e < E; e += blockDim.x) row[kHdrInts + e] = tot[e];
        }
        if (threadIdx.x < 2) A.plan->done[threadIdx.x] = 0;  // the dispatch and down kernels of this layer count their CTAs here
        __threadfence_system();
        __syncthreads();
        if ((int)threadIdx.x < W) st_release_sys(flags_of(A.v.peer[threadIdx.x], 0) + A.v.rank, A.epoch);
    }
    if (!(stages & 2)) return;
    __syncthreads();
    // -- wait for every rank's row
    if ((int)threadIdx.x < W && !wait_flag(flags_of(A.v.peer[A.v.rank], 0) + threadIdx.x, A.epoch)) s_ok = 0;
    __syncthreads();
    if (!s_ok) {
        if (threadIdx.x == 0) {
            *(volatile int*)A.status = FQ_ERR_TIMEOUT;
            A.plan->ok = 0, A.plan->n_rows = 0, A.plan->n_gu = 0, A.plan->n_dn = 0;
        }
        return;
    }
    for (int i = threadIdx.x; i < W * E; i += blockDim.x) tbl[i] = table_row(A.v.peer[A.v.rank], i / E)[kHdrInts + i % E];
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int t = 0, before = 0;
        for (int s = 0; s < W; ++s) {
            if (s == A.v.rank) before = t;
            t += tbl[s * E + e];
        }
        tot[e] = t;
        cursor[e] = before;  // rows of this expert that lower ranks send: my rows follow them
    }
    __syncthreads();
    // per owner rank: exclusive scan of its experts' totals (thread d walks rank d's experts) and the capacity check
    if ((int)threadIdx.x < W) {
        const int d = threadIdx.x;
        int run = 0;
        for (int e = d * per; e < (d + 1) * per; ++e) {
            base[e] = run;
            run += tot[e];
        }
        const int* hdr = table_row(A.v.peer[A.v.rank], d);
        if (run > hdr[4]) atomicExch(&s_ok, 0);  // rank d's panel would overflow: every rank sees this
        A.plan->dst_meta[d] = (unsigned long long)(unsigned)hdr[0] | ((unsigned long long)(unsigned)hdr[1] << 32);
        A.plan->dst_x[d] = (unsigned long long)(unsigned)hdr[2] | ((unsigned long long)(unsigned)hdr[3] << 32);
        if (d == A.v.rank) s_rows = run;
    }
    __syncthreads();
    if (!s_ok) {
        if (threadIdx.x == 0) {
            *(volatile int*)A.status = FQ_ERR_CAPACITY;  // the host reports it at the next synchronisation
            A.plan->ok = 0, A.plan->n_rows = 0, A.plan->n_gu = 0, A.plan->n_dn = 0;
        }
        return;
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) cursor[e] += base[e];
    // tile lists of this rank's experts: token tiles per expert (the two products may cut them differently),
    // exclusive scans by one thread (at most a few hundred experts)
    if (threadIdx.x == 0) {
        int ngu = 0, ndn = 0;
        for (int le = 0; le < per; ++le) {
            const int c = tot[A.v.rank * per + le];
            tiles_gu[le] = ngu, tiles_dn[le] = ndn;
            ngu += (c + A.tile_gu - 1) / A.tile_gu;
            ndn += (c + A.tile_dn - 1) / A.tile_dn;
        }
        A.plan->ok = 1;
        A.plan->n_rows = s_rows;
        A.plan->n_gu = ngu * A.rt_gu;
        A.plan->n_dn = ndn * A.rt_dn;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int le = warp; le < per; le += warps) {
        const int e = A.v.rank * per + le, c = tot[e], row0 = base[e];
        for (int t0 = 0, tt = 0; t0 < c; t0 += A.tile_gu, ++tt)
            for (int rt = lane; rt < A.rt_gu; rt += 32) A.t_gu[(size_t)(tiles_gu[le] + tt) * A.rt_gu + rt] = {le, rt, row0 + t0, min(A.tile_gu, c - t0)};
        for (int t0 = 0, tt = 0; t0 < c; t0 += A.tile_dn, ++tt)
            for (int rt = lane; rt < A.rt_dn; rt += 32) A.t_dn[(size_t)(tiles_dn[le] + tt) * A.rt_dn + rt] = {le, rt, row0 + t0, min(A.tile_dn, c - t0)};
    }
    // every pair's final row in its owner's panel (positions inside a (source, expert) run do not affect any value)
    for (int p = threadIdx.x; p < A.pairs; p += blockDim.x) {
        const int e = A.selected[p];
        if (e < 0 || e >= E) {
            A.pair_dst[p] = make_int2(-1, 0);
            continue;
        }
        A.pair_dst[p] = make_int2(e / per, atomicAdd(&cursor[e], 1));
    }
}

// The last CTA of a grid to get here tells every peer "rank `rank` finished phase `kind` of layer `epoch`".
// Every thread's peer stores are fenced system-wide first; the CTA count lives in the layer's plan block.
__device__ __forceinline__ void signal_when_grid_done(const EpView& v, int* counter, int kind, int epoch) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(counter, 1) == (int)gridDim.x - 1) {
        __threadfence_system();
        for (int d = 0; d < v.world; ++d) st_release_sys(flags_of(v.peer[d], kind) + v.rank, epoch);
    }
}

// ---- dispatch: bf16 token rows and return addresses into the owners' panels ---------------------------
__global__ void ep_dispatch_kernel(const EpArgs A, const float* __restrict__ x) {
    if (!A.plan->ok) {
        signal_when_grid_done(A.v, &A.plan->done[0], 1, A.epoch);  // the peers' waits still end
        return;
    }
    const int h8 = A.hidden >> 3;
    const size_t total = (size_t)A.pairs * h8;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int p = (int)(i / h8), col = (int)(i % h8) * 8;
        const int2 dst = A.pair_dst[p];
        if (dst.x < 0) continue;
        uint8_t* arena = A.v.peer[dst.x];
        const float4* src = reinterpret_cast<const float4*>(x + (size_t)(p / A.top_k) * A.hidden + col);
        const float4 v0 = __ldg(src), v1 = __ldg(src + 1);
        const __nv_bfloat162 b0 = __floats2bfloat162_rn(v0.x, v0.y), b1 = __floats2bfloat162_rn(v0.z, v0.w);
        const __nv_bfloat162 b2 = __floats2bfloat162_rn(v1.x, v1.y), b3 = __floats2bfloat162_rn(v1.z, v1.w);
        uint4 o;
        o.x = *reinterpret_cast<const uint32_t*>(&b0), o.y = *reinterpret_cast<const uint32_t*>(&b1);
        o.z = *reinterpret_cast<const uint32_t*>(&b2), o.w = *reinterpret_cast<const uint32_t*>(&b3);
        __nv_bfloat16* panel = reinterpret_cast<__nv_bfloat16*>(arena + A.plan->dst_x[dst.x]);
        *reinterpret_cast<uint4*>(panel + (size_t)dst.y * A.hidden + col) = o;
        if (col == 0) reinterpret_cast<int2*>(arena + A.plan->dst_meta[dst.x])[dst.y] = make_int2(A.v.rank, p);
    }
    signal_when_grid_done(A.v, &A.plan->done[0], 1, A.epoch);
}

// Diagnosis only (FUCINA_B200_EP_TRACE): the wait for the sources' dispatch flags as a kernel of its own, so the
// trace separates waiting from multiplying. The product after it finds the flags posted.
__global__ void ep_wait_kernel(const EpArgs A, int kind) {
    if ((int)threadIdx.x < A.v.world) wait_flag(flags_of(A.v.peer[A.v.rank], kind) + threadIdx.x, A.epoch);
}

// ---- combine: out[t] = sum over the token's slots, in slot order, of w[p] * ret[p] ---------------------
__global__ void ep_combine_kernel(const EpArgs A, const float* __restrict__ weights, float* __restrict__ out, int seq) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = A.plan->ok;
    __syncthreads();
    if ((int)threadIdx.x < A.v.world && s_ok && !wait_flag(flags_of(A.v.peer[A.v.rank], 2) + threadIdx.x, A.epoch)) {
        s_ok = 0;
        *(volatile int*)A.status = FQ_ERR_TIMEOUT;
    }
    __syncthreads();
    if (!s_ok) return;
    const float* ret = reinterpret_cast<const float*>(A.v.peer[A.v.rank] + A.mine.off_ret);
    const int h4 = A.hidden >> 2;
    const size_t total = (size_t)seq * h4;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / h4), j = (int)(i % h4) * 4;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        bool first = true;
        for (int kk = 0; kk < A.top_k; ++kk) {
            const int p = t * A.top_k + kk;
            if (A.pair_dst[p].x < 0) continue;
            const float wv = weights[p];
            // the rows were written by other GPUs during this kernel's lifetime: read them past the L1
            float4 v = __ldcg(reinterpret_cast<const float4*>(ret + (size_t)p * A.hidden + j));
            v.x = __fmul_rn(wv, v.x), v.y = __fmul_rn(wv, v.y), v.z = __fmul_rn(wv, v.z), v.w = __fmul_rn(wv, v.w);
            if (first) acc = v;
            else acc.x = __fadd_rn(acc.x, v.x), acc.y = __fadd_rn(acc.y, v.y), acc.z = __fadd_rn(acc.z, v.z), acc.w = __fadd_rn(acc.w, v.w);
            first = false;
        }
        *reinterpret_cast<float4*>(out + (size_t)t * A.hidden + j) = acc;
    }
}

// ---- host side: one rank's layer as six phases -----------------------------------------------------------
struct EpCall {
    EpArgs a;
    const DevWeights *gate, *up, *down;
    const float* x;
    const float* weights;
    float* out;
    int seq;
    uint8_t* scratch;
    __nv_bfloat16* g_panel;
    int max_gu, max_dn;
    int plan_stages = 3;  // see ep_plan_kernel
    int gated_op = 0;
};

int ep_prepare(Ctx* ctx, const EpView& v, int epoch, const DevWeights& gate, const DevWeights& up, const DevWeights& down, const float* x,
               int seq, int top_k, const int* selected, const float* weights, float* out, cudaStream_t st, EpCall* c) {
    const int hidden = gate.k, out_pe = gate.n, per = gate.n_mats, E = per * v.world;
    if (E > kEpMaxExperts) return fail(FQ_DECLINED_ARGS, "expert parallelism serves up to %d experts", kEpMaxExperts);
    if (hidden % 8 != 0) return fail(FQ_DECLINED_ARGS, "hidden must be a multiple of 8");
    const int pairs = seq * top_k;
    EpArgs& a = c->a;
    a.v = v;
    a.epoch = epoch;
    a.pairs = pairs, a.top_k = top_k, a.hidden = hidden, a.n_expert = E, a.per = per;
    a.mine = ep_layout(v.arena_bytes, pairs, hidden);
    if (a.mine.rows_cap < 128) return fail(FQ_DECLINED_BUDGET, "exchange arena of %zu bytes is too small for %d pairs of %d elements", v.arena_bytes, pairs, hidden);
    // the fused gate/up pass (SwiGLU in the epilogue) runs on 128-token tiles; the down product takes 256-token
    // tiles once expert runs are long (a weight is expanded to bf16 once per token tile)
    static const int down_tile_env = getenv("FUCINA_B200_EP_DOWN_TILE") ? atoi(getenv("FUCINA_B200_EP_DOWN_TILE")) : 0;
    a.tile_gu = 128;
    // (over several GPUs the result rows leave through the epilogue's peer stores, which 128-token tiles overlap with the
    // next tile's MMAs -- two alternating accumulators -- while a 256-token tile's epilogue is exposed: measured 142 us
    // against 156 us for the down product at eight GPUs)
    a.tile_dn = down_tile_env == 128 || down_tile_env == 256 ? down_tile_env : (v.world == 1 && pairs > 128 * per ? 256 : 128);
    a.rt_gu = (out_pe + 127) / 128, a.rt_dn = (hidden + 127) / 128;
    a.selected = selected;
    a.status = ctx->status_dev;
    c->gate = &gate, c->up = &up, c->down = &down;
    c->x = x, c->weights = weights, c->out = out, c->seq = seq;
    c->max_gu = (per + a.mine.rows_cap / a.tile_gu) * a.rt_gu, c->max_dn = (per + a.mine.rows_cap / a.tile_dn) * a.rt_dn;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off += (bytes + 255) & ~(size_t)255;
        return o;
    };
    const size_t o_plan = take(sizeof(EpPlan)), o_dst = take(sizeof(int2) * pairs);
    const size_t o_tgu = take(sizeof(TcTile) * c->max_gu), o_tdn = take(sizeof(TcTile) * c->max_dn);
    const size_t o_g = take((size_t)a.mine.rows_cap * out_pe * 2);
    c->scratch = (uint8_t*)dev_alloc_on(off, st);
    if (!c->scratch) return fail(FQ_DECLINED_BUDGET, "expert-parallel scratch of %zu bytes could not be allocated", off);
    a.plan = (EpPlan*)(c->scratch + o_plan);
    a.pair_dst = (int2*)(c->scratch + o_dst);
    a.t_gu = (TcTile*)(c->scratch + o_tgu);
    a.t_dn = (TcTile*)(c->scratch + o_tdn);
    c->g_panel = (__nv_bfloat16*)(c->scratch + o_g);
    return FQ_OK;
}

int ep_phase(Ctx* ctx, EpCall& c, int phase, cudaStream_t st) {
    EpArgs& a = c.a;
    uint8_t* me = a.v.peer[a.v.rank];
    cudaError_t e = cudaSuccess;
    int rc = FQ_OK;
    switch (phase) {
        case 0: {
            const size_t smem = sizeof(int) * ((size_t)a.v.world * a.n_expert + 3 * (size_t)a.n_expert + 2 * (size_t)a.per);
            // at most 8 * 1024 + 3 * 1024 + 2 * 128 ints: fits 48 KB
            ep_plan_kernel<<<1, 1024, smem, st>>>(a, c.plan_stages);
            break;
        }
        case 1: {
            int blocks = (int)(((size_t)a.pairs * (a.hidden / 8) + 255) / 256);
            ep_dispatch_kernel<<<blocks > 148 * 8 ? 148 * 8 : (blocks < 1 ? 1 : blocks), 256, 0, st>>>(a, c.x);
            break;
        }
        case 2: {
            TcPeer peer;
            peer.wait_flags = flags_of(me, 1);
            peer.n_wait = a.v.world;
            peer.wait_value = a.epoch;
            const uint8_t* x_panel = me + a.mine.off_x;
            rc = gemm_tensor_grouped_gated_dev(ctx, *c.gate, *c.up, x_panel, (size_t)a.mine.rows_cap, c.g_panel, (size_t)c.gate->n,
                                               a.t_gu, &a.plan->n_gu, c.max_gu, st, &peer, c.gated_op);
            break;
        }
        case 3: {
            TcPeer peer;
            peer.row_meta = reinterpret_cast<const int2*>(me + a.mine.off_meta);
            for (int s = 0; s < a.v.world; ++s) {
                peer.dst_base[s] = reinterpret_cast<float*>(a.v.peer[s] + kFixedBytes);
                peer.signal_flag[s] = flags_of(a.v.peer[s], 2) + a.v.rank;
            }
            peer.n_signal = a.v.world;
            peer.signal_value = a.epoch;
            peer.done_counter = &a.plan->done[1];
            rc = gemm_tensor_grouped_dev(ctx, *c.down, c.g_panel, (size_t)a.mine.rows_cap, nullptr, (size_t)a.hidden, a.t_dn, &a.plan->n_dn, c.max_dn,
                                         a.tile_dn, st, &peer);
            break;
        }
        default: {
            int blocks = (int)(((size_t)c.seq * (a.hidden / 4) + 127) / 128);
            ep_combine_kernel<<<blocks > 148 * 16 ? 148 * 16 : (blocks < 1 ? 1 : blocks), 128, 0, st>>>(a, c.weights, c.out, c.seq);
            break;
        }
    }
    g_trace.launches += 2;
    if (rc != FQ_OK) return rc;
    e = cudaGetLastError();
    return e == cudaSuccess ? FQ_OK : cuda_fail(e, "expert-parallel launch");
}
constexpr int kEpPhases = 5;
std::vector<std::vector<cudaEvent_t>> g_ep_events;  // FUCINA_B200_EP_TRACE: one set of phase events per layer

int check_ep_weights(const fq_weights* gate, const fq_weights* up, const fq_weights* down, size_t seq, size_t top_k, int gated_op) {
    if (!gate || !up || !down) return fail(FQ_DECLINED_ARGS, "null weights");
    if (gated_op < FQ_GATED_SWIGLU || gated_op > FQ_GATED_SITU) return fail(FQ_DECLINED_ARGS, "gated_op %d is not one of FQ_GATED_*", gated_op);
    const DevWeights &g = gate->dw, &u = up->dw, &d = down->dw;
    if (g.fmt != u.fmt) return fail(FQ_DECLINED_ARGS, "gate and up must share one format");
    if (g.n != u.n || g.k != u.k || g.n_mats != u.n_mats || d.n_mats != g.n_mats || d.n != g.k || d.k != g.n)
        return fail(FQ_DECLINED_ARGS, "expert tensor shapes are inconsistent");
    if (seq == 0 || top_k == 0 || seq * top_k > (size_t)1 << 22) return fail(FQ_DECLINED_ARGS, "bad seq/top_k");
    return FQ_OK;
}

bool fused_form_serves(const DevWeights& g, const DevWeights& d) {
    auto stack_fmt = [](int f) { return f == FQ_Q4_K || f == FQ_Q5_K || f == FQ_Q6_K || f == FQ_Q8_0; };  // as the one-GPU tensor arm
    return stack_fmt(g.fmt) && stack_fmt(d.fmt) && tensor_path_serves(g) && tensor_path_serves(d) && g.k % 8 == 0;
}

}  // namespace

void ep_trace_dump(int rank) {
    if (g_ep_events.empty()) return;
    static const char* names[kEpPhases] = {"plan", "dispatch+wait", "gate/up", "down+wait", "combine"};
    double sum[kEpPhases] = {0, 0, 0, 0, 0};
    long long layers = 0;
    // the second half of the recorded layers: steady state, the host running ahead of the device
    for (size_t i = 0; i < g_ep_events.size(); ++i) {
        auto& ev = g_ep_events[i];
        if (i >= g_ep_events.size() / 2 && cudaEventSynchronize(ev[kEpPhases]) == cudaSuccess) {
            for (int ph = 0; ph < kEpPhases; ++ph) {
                float ms = 0.0f;
                if (cudaEventElapsedTime(&ms, ev[ph], ev[ph + 1]) == cudaSuccess) sum[ph] += ms;
            }
            ++layers;
        }
        for (auto& e : ev) cudaEventDestroy(e);
    }
    g_ep_events.clear();
    cudaGetLastError();
    char line[512];
    int n = snprintf(line, sizeof line, "[fucina_b200] rank %d expert-parallel layers=%lld, mean device ms per phase:", rank, layers);
    for (int ph = 0; ph < kEpPhases && layers; ++ph) n += snprintf(line + n, sizeof line - n, " %s=%.4f", names[ph], sum[ph] / (double)layers);
    fprintf(stderr, "%s\n", line);
}

}  // namespace fq

using namespace fq;

extern "C" {

int fq_moe_layer_ep(const fq_weights* gate, const fq_weights* up, const fq_weights* down, const float* x_dev, size_t seq, size_t top_k,
                    const int32_t* selected_dev, const float* weights_dev, int gated_op, float* out_dev, int flags, void* stream) {
    if (int rc = check_ep_weights(gate, up, down, seq, top_k, gated_op)) return rc;
    if (!x_dev || !selected_dev || !weights_dev || !out_dev) return fail(FQ_DECLINED_ARGS, "null pointer");
    TpCtx* t = tp_context();
    if (!t) return fail(FQ_DECLINED_ARGS, "fq_tp_init was not called");
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    g_trace.calls++;
    cudaStream_t st = stream ? (cudaStream_t)stream : ctx->stream;
    const DevWeights &gw = gate->dw, &uw = up->dw, &dw = down->dw;
    const int hidden = gw.k;
    const bool fused = !(flags & 1) && t->peer_ok && fused_form_serves(gw, dw);
    if ((flags & 2) && !fused) return fail(FQ_DECLINED_ARGS, "the fused form was asked for but the peers' arenas are not mapped or the format has no tensor-core kernel");
    if (fused) {
        EpView v;
        v.rank = t->rank, v.world = t->world, v.arena_bytes = t->arena_bytes;
        for (int r = 0; r < kMaxPeers; ++r) v.peer[r] = t->peer[r];
        EpCall c;
        const int epoch = ++t->epoch;
        if (int rc = ep_prepare(ctx, v, epoch, gw, uw, dw, x_dev, (int)seq, (int)top_k, selected_dev, weights_dev, out_dev, st, &c)) {
            --t->epoch;
            return rc;
        }
        c.gated_op = gated_op;
        int rc = FQ_OK;
        // FUCINA_B200_EP_TRACE=1: device time of each phase (CUDA events on the layer's stream), summed per phase and
        // printed by fq_tp_shutdown -- the per-kind timing of backend/cuda.zig:231-257 for this layer
        static const bool trace = getenv("FUCINA_B200_EP_TRACE") != nullptr;
        std::vector<cudaEvent_t> ev;
        if (trace && g_ep_events.size() < 4096) {
            ev.resize(kEpPhases + 1);
            for (auto& e : ev) cudaEventCreate(&e);
            cudaEventRecord(ev[0], st);
        }
        for (int ph = 0; ph < kEpPhases && rc == FQ_OK; ++ph) {
            if (!ev.empty() && ph == 2) {  // the wait for the dispatch flags counts towards the dispatch phase of the trace
                ep_wait_kernel<<<1, 32, 0, st>>>(c.a, 1);
                cudaEventRecord(ev[ph], st);
            }
            if (!ev.empty() && ph == 4) {  // and the wait for the return flags towards the down phase
                ep_wait_kernel<<<1, 32, 0, st>>>(c.a, 2);
                cudaEventRecord(ev[ph], st);
            }
            rc = ep_phase(ctx, c, ph, st);
            if (!ev.empty()) cudaEventRecord(ev[ph + 1], st);
        }
        if (!ev.empty()) g_ep_events.push_back(ev);  // read when the trace is dumped: no host wait per layer
        dev_free_on(c.scratch, st);
        return rc;
    }
    // baseline: gather everything, multiply this rank's experts for all tokens, reduce-scatter the partial sums
    const int W = t->world;
    const size_t rows = seq * W, pk = seq * top_k;
    const size_t xb = rows * hidden * sizeof(float), rb = ((pk * 8 + 255) & ~(size_t)255);
    uint8_t* s = (uint8_t*)dev_alloc_on(2 * xb + rb * (W + 1) + 512, st);
    if (!s) return fail(FQ_DECLINED_BUDGET, "expert-parallel scratch could not be allocated");
    float* x_all = (float*)s;
    float* partial = (float*)(s + xb);
    uint8_t* route_mine = s + 2 * xb;       // [seq*top_k] ids, then [seq*top_k] weights
    uint8_t* route_all = route_mine + rb;   // W such records
    int rc = FQ_OK;
    cudaError_t e = cudaMemcpyAsync(route_mine, selected_dev, pk * 4, cudaMemcpyDeviceToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(route_mine + pk * 4, weights_dev, pk * 4, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) rc = cuda_fail(e, "routing staging");
    if (rc == FQ_OK) rc = tp_all_gather(route_mine, route_all, rb, st);
    if (rc == FQ_OK) rc = tp_all_gather(x_dev, x_all, seq * hidden * sizeof(float), st);
    // the gathered routing is [rank][ids | weights]: repack to [all tokens][top_k] ids and weights
    int* sel_all = nullptr;
    float* w_all = nullptr;
    if (rc == FQ_OK) {
        sel_all = (int*)dev_alloc_on(rows * top_k * 8, st);
        if (!sel_all) rc = fail(FQ_DECLINED_BUDGET, "routing scratch could not be allocated");
    }
    if (rc == FQ_OK) {
        w_all = (float*)(sel_all + rows * top_k);
        for (int r = 0; r < W && e == cudaSuccess; ++r) {
            e = cudaMemcpyAsync(sel_all + (size_t)r * pk, route_all + (size_t)r * rb, pk * 4, cudaMemcpyDeviceToDevice, st);
            if (e == cudaSuccess) e = cudaMemcpyAsync(w_all + (size_t)r * pk, route_all + (size_t)r * rb + pk * 4, pk * 4, cudaMemcpyDeviceToDevice, st);
        }
        if (e != cudaSuccess) rc = cuda_fail(e, "routing repack");
    }
    if (rc == FQ_OK)
        rc = moe_layer_shard_dev(ctx, gw, uw, dw, x_all, (int)rows, (int)top_k, sel_all, w_all, t->rank * gw.n_mats, partial, st, gated_op);
    if (rc == FQ_OK) rc = tp_reduce_scatter_f32(partial, out_dev, seq * hidden, st);
    dev_free_on(sel_all, st);
    dev_free_on(s, st);
    return rc;
}

// Test seam: `world` ranks of the fused form emulated on ONE GPU. Every emulated rank has its own arena,
// weights shard, tokens and routing; the phases run in lockstep on the library stream (phase p of every rank
// before phase p + 1 of any), so each wait finds its flags already posted by completed kernels -- nothing
// waits on a kernel that runs beside it. Exercises the count / plan / dispatch / peer-store / combine logic
// exactly as the multi-process form runs it, pointer mapping aside.
int fq_ep_emulate_for_test(int world, const fq_weights* const* gate, const fq_weights* const* up, const fq_weights* const* down,
                           const float* const* x_dev, size_t seq, size_t top_k, const int32_t* const* selected_dev,
                           const float* const* weights_dev, float* const* out_dev, size_t arena_bytes, int layers) {
    // layers < 0: one layer in which the LAST rank's count publication is dropped (a message that never arrives):
    // every rank's bounded wait gives up, the status word reports FQ_ERR_TIMEOUT, nothing hangs
    const bool drop_last = layers < 0;
    if (drop_last) layers = 1;
    if (world < 1 || world > kMaxPeers || !gate || !up || !down || !x_dev || !selected_dev || !weights_dev || !out_dev || layers < 1)
        return fail(FQ_DECLINED_ARGS, "bad emulation request");
    for (int r = 0; r < world; ++r) {
        if (int rc = check_ep_weights(gate[r], up[r], down[r], seq, top_k, 0)) return rc;
        if (!fused_form_serves(gate[r]->dw, down[r]->dw)) return fail(FQ_DECLINED_ARGS, "format has no tensor-core kernel");
    }
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    cudaStream_t st = ctx->stream;
    if (arena_bytes < kFixedBytes + 4096) return fail(FQ_DECLINED_ARGS, "arena too small");
    std::vector<uint8_t*> arenas(world, nullptr);
    int rc = FQ_OK;
    for (int r = 0; r < world && rc == FQ_OK; ++r) {
        arenas[r] = (uint8_t*)dev_alloc_on(arena_bytes, st);
        if (!arenas[r]) rc = fail(FQ_DECLINED_BUDGET, "arena allocation failed");
        else cudaMemsetAsync(arenas[r], 0, kFixedBytes, st);
    }
    for (int layer = 1; layer <= layers && rc == FQ_OK; ++layer) {
        std::vector<EpCall> calls(world);
        int prepared = 0;
        for (int r = 0; r < world && rc == FQ_OK; ++r) {
            EpView v;
            v.rank = r, v.world = world, v.arena_bytes = arena_bytes;
            for (int q = 0; q < kMaxPeers; ++q) v.peer[q] = q < world ? arenas[q] : nullptr;
            rc = ep_prepare(ctx, v, layer, gate[r]->dw, up[r]->dw, down[r]->dw, x_dev[r], (int)seq, (int)top_k, selected_dev[r], weights_dev[r],
                            out_dev[r], st, &calls[r]);
            if (rc == FQ_OK) ++prepared;
        }
        // publication of every rank's counts first, then the phases in lockstep
        for (int r = 0; r < world && rc == FQ_OK; ++r) {
            calls[r].plan_stages = 1;
            if (!(drop_last && world > 1 && r == world - 1)) rc = ep_phase(ctx, calls[r], 0, st);
            calls[r].plan_stages = 2;
        }
        for (int ph = 0; ph < kEpPhases && rc == FQ_OK; ++ph)
            for (int r = 0; r < world && rc == FQ_OK; ++r) rc = ep_phase(ctx, calls[r], ph, st);
        for (int r = 0; r < prepared; ++r) dev_free_on(calls[r].scratch, st);
    }
    cudaError_t e = cudaStreamSynchronize(st);
    for (int r = 0; r < world; ++r) dev_free_on(arenas[r], st);
    if (rc == FQ_OK && e != cudaSuccess) rc = cuda_fail(e, "emulated expert-parallel layer");
    if (rc == FQ_OK) rc = device_status(ctx);
    return rc;
}

}  // extern "C"
