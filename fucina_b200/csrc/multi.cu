// Multi-GPU plumbing behind the C ABI: one process per GPU of one NVLink-connected node.
//
// The reference provider is single-device (src/backend/cuda.zig:439 takes device 0), so nothing here has a
// counterpart there. Two things are set up by fq_tp_init:
//   * an NCCL communicator (the library is loaded at run time, so libfucina_b200.so has no link dependency on
//     it) for the fixed-size exchanges: all-gather of column shards, all-gather / reduce-scatter of the
//     baseline expert-parallel form;
//   * a per-rank exchange arena (plain cudaMalloc memory) whose CUDA IPC handle is all-gathered over that
//     communicator and opened by every peer, so kernels can store straight into another GPU's memory over
//     NVLink (plain peer stores and loads; no multicast of any kind).
// The rendezvous id is produced by rank 0 (fq_tp_unique_id) and carried to the other processes by the host.
#include <dlfcn.h>

#include <cstring>
#include <mutex>

#include "multi.h"

namespace fq {

namespace {

// ---- the NCCL entry points this file uses, resolved at run time -------------------------------------------
struct NcclId {
    char bytes[128];
};
typedef int (*GetUniqueIdFn)(NcclId*);
typedef int (*CommInitRankFn)(void**, int, NcclId, int);
typedef int (*CommDestroyFn)(void*);
typedef int (*AllGatherFn)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*ReduceScatterFn)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef const char* (*GetErrorStringFn)(int);
constexpr int kNcclInt8 = 0, kNcclFloat32 = 7, kNcclSum = 0;

struct Nccl {
    void* handle = nullptr;
    GetUniqueIdFn get_unique_id = nullptr;
    CommInitRankFn comm_init_rank = nullptr;
    CommDestroyFn comm_destroy = nullptr;
    AllGatherFn all_gather = nullptr;
    ReduceScatterFn reduce_scatter = nullptr;
    GetErrorStringFn error_string = nullptr;
};
Nccl g_nccl;
std::mutex g_tp_lock;
TpCtx g_tp;
bool g_tp_ready = false;

int load_nccl() {
    if (g_nccl.handle) return FQ_OK;
    // a host that already uses NCCL (torch.distributed, for instance) has it loaded: share that copy
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return fail(FQ_DECLINED_NO_GPU, "libnccl.so.2 could not be loaded: %s", dlerror());
    Nccl n;
    n.handle = h;
    n.get_unique_id = (GetUniqueIdFn)dlsym(h, "ncclGetUniqueId");
    n.comm_init_rank = (CommInitRankFn)dlsym(h, "ncclCommInitRank");
    n.comm_destroy = (CommDestroyFn)dlsym(h, "ncclCommDestroy");
    n.all_gather = (AllGatherFn)dlsym(h, "ncclAllGather");
    n.reduce_scatter = (ReduceScatterFn)dlsym(h, "ncclReduceScatter");
    n.error_string = (GetErrorStringFn)dlsym(h, "ncclGetErrorString");
    if (!n.get_unique_id || !n.comm_init_rank || !n.comm_destroy || !n.all_gather || !n.reduce_scatter || !n.error_string)
        return fail(FQ_DECLINED_NO_GPU, "libnccl.so.2 lacks an entry point this library needs");
    g_nccl = n;
    return FQ_OK;
}

int nccl_fail(int rc, const char* what) {
    return fail(FQ_ERR_CUDA, "%s: %s", what, g_nccl.error_string ? g_nccl.error_string(rc) : "NCCL error");
}

void unmap_peers(TpCtx& t) {
    for (int r = 0; r < t.world; ++r)
        if (r != t.rank && t.peer[r]) cudaIpcCloseMemHandle(t.peer[r]);
    for (int r = 0; r < kMaxPeers; ++r) t.peer[r] = nullptr;
    t.peer_ok = false;
}

}  // namespace

TpCtx* tp_context() { return g_tp_ready ? &g_tp : nullptr; }

int tp_all_gather(const void* send, void* recv, size_t bytes_per_rank, cudaStream_t st) {
    TpCtx* t = tp_context();
    if (!t) return fail(FQ_DECLINED_ARGS, "fq_tp_init was not called");
    const int rc = g_nccl.all_gather(send, recv, bytes_per_rank, kNcclInt8, t->comm, st);
    return rc == 0 ? FQ_OK : nccl_fail(rc, "all-gather");
}
int tp_reduce_scatter_f32(const float* send, float* recv, size_t count_per_rank, cudaStream_t st) {
    TpCtx* t = tp_context();
    if (!t) return fail(FQ_DECLINED_ARGS, "fq_tp_init was not called");
    const int rc = g_nccl.reduce_scatter(send, recv, count_per_rank, kNcclFloat32, kNcclSum, t->comm, st);
    return rc == 0 ? FQ_OK : nccl_fail(rc, "reduce-scatter");
}

}  // namespace fq

using namespace fq;

extern "C" {

int fq_tp_unique_id(void* id128) {
    if (!id128) return fail(FQ_DECLINED_ARGS, "null pointer");
    if (int rc = load_nccl()) return rc;
    NcclId id;
    const int rc = g_nccl.get_unique_id(&id);
    if (rc != 0) return nccl_fail(rc, "ncclGetUniqueId");
    memcpy(id128, id.bytes, sizeof id.bytes);
    return FQ_OK;
}

int fq_tp_init(int n_ranks, int rank, const void* id128, size_t arena_bytes) {
    if (!id128 || n_ranks < 1 || n_ranks > kMaxPeers || rank < 0 || rank >= n_ranks)
        return fail(FQ_DECLINED_ARGS, "fq_tp_init needs 1..%d ranks, a rank below that and the rendezvous id", kMaxPeers);
    if (!gpu_enabled()) return fail(FQ_DECLINED_GATE, "disabled by FUCINA_GPU=0");
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::mutex> g(g_tp_lock);
    if (g_tp_ready) return fail(FQ_DECLINED_ARGS, "fq_tp_init was already called (rank %d of %d)", g_tp.rank, g_tp.world);
    if (int rc = load_nccl()) return rc;
    TpCtx t;
    t.world = n_ranks;
    t.rank = rank;
    NcclId id;
    memcpy(id.bytes, id128, sizeof id.bytes);
    int rc = g_nccl.comm_init_rank(&t.comm, n_ranks, id, rank);
    if (rc != 0) return nccl_fail(rc, "ncclCommInitRank");
    // the exchange arena: plain cudaMalloc memory (IPC handles cannot be taken of pooled or virtual allocations)
    t.arena_bytes = arena_bytes ? (arena_bytes + 255) & ~(size_t)255 : (size_t)1 << 30;
    cudaError_t e = cudaMalloc((void**)&t.arena, t.arena_bytes);
    if (e != cudaSuccess) {
        g_nccl.comm_destroy(t.comm);
        cudaGetLastError();
        return fail(FQ_DECLINED_BUDGET, "exchange arena of %zu bytes could not be allocated", t.arena_bytes);
    }
    cudaMemsetAsync(t.arena, 0, t.arena_bytes < (64u << 10) ? t.arena_bytes : (64u << 10), ctx->stream);  // flags and tables start at zero
    t.peer[rank] = t.arena;
    t.peer_ok = true;
    if (n_ranks > 1) {
        // every rank's IPC handle to every rank, through the communicator itself
        cudaIpcMemHandle_t mine;
        cudaIpcMemHandle_t* dev_handles = nullptr;
        cudaIpcMemHandle_t all[kMaxPeers];
        e = cudaIpcGetMemHandle(&mine, t.arena);
        if (e == cudaSuccess) e = cudaMalloc((void**)&dev_handles, sizeof(cudaIpcMemHandle_t) * (n_ranks + 1));
        if (e == cudaSuccess) e = cudaMemcpyAsync(dev_handles + n_ranks, &mine, sizeof mine, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) {
            rc = g_nccl.all_gather(dev_handles + n_ranks, dev_handles, sizeof mine, kNcclInt8, t.comm, ctx->stream);
            if (rc != 0) e = cudaErrorUnknown;
        }
        if (e == cudaSuccess) e = cudaMemcpyAsync(all, dev_handles, sizeof(cudaIpcMemHandle_t) * n_ranks, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (dev_handles) cudaFree(dev_handles);
        if (e != cudaSuccess) {
            cudaGetLastError();
            t.peer_ok = false;  // the NCCL forms still work
        } else {
            for (int r = 0; r < n_ranks; ++r) {
                if (r == rank) continue;
                void* p = nullptr;
                if (cudaIpcOpenMemHandle(&p, all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                    cudaGetLastError();
                    t.peer_ok = false;
                    break;
                }
                t.peer[r] = (uint8_t*)p;
            }
            if (!t.peer_ok) {
                for (int r = 0; r < n_ranks; ++r)
                    if (r != rank && t.peer[r]) cudaIpcCloseMemHandle(t.peer[r]), t.peer[r] = nullptr;
            }
        }
    }
    cudaStreamSynchronize(ctx->stream);
    g_tp = t;
    g_tp_ready = true;
    return FQ_OK;
}

int fq_tp_shutdown(void) {
    std::lock_guard<std::mutex> g(g_tp_lock);
    if (!g_tp_ready) return FQ_OK;
    Ctx* ctx = context();
    if (ctx) cudaStreamSynchronize(ctx->stream);
    ep_trace_dump(g_tp.rank);
    unmap_peers(g_tp);
    if (g_tp.arena) cudaFree(g_tp.arena);
    if (g_tp.comm) g_nccl.comm_destroy(g_tp.comm);
    g_tp = TpCtx{};
    g_tp_ready = false;
    return FQ_OK;
}

int fq_tp_ranks(void) { return g_tp_ready ? g_tp.world : 0; }
int fq_tp_rank(void) { return g_tp_ready ? g_tp.rank : -1; }
int fq_tp_peer_access(void) { return g_tp_ready && g_tp.peer_ok ? 1 : 0; }

// Column-sharded product: this rank multiplies its shard of the output columns, one all-gather assembles
// c_dev as [rank][m][n_shard] (every rank's shard must have the same number of rows).
int fq_gemm_quant_nt_tp(const fq_weights* w_shard, const float* a_dev, float* c_dev, size_t m, int mode, void* stream) {
    if (!w_shard || !a_dev || !c_dev) return fail(FQ_DECLINED_ARGS, "null pointer");
    TpCtx* t = tp_context();
    if (!t) return fail(FQ_DECLINED_ARGS, "fq_tp_init was not called");
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    g_trace.calls++;
    cudaStream_t st = stream ? (cudaStream_t)stream : ctx->stream;
    const size_t n = (size_t)w_shard->dw.n;
    float* mine = c_dev + (size_t)t->rank * m * n;  // the shard lands in its slot of the gathered result: an in-place all-gather
    int rc = gemm_dev(ctx, w_shard->dw, 0, a_dev, mine, m, n, mode, 0, st);
    if (rc != FQ_OK) return rc;
    if (t->world == 1) return FQ_OK;
    return tp_all_gather(mine, c_dev, m * n * sizeof(float), st);
}

}  // extern "C"
