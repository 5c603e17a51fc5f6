// Runtime services shared by the translation units (context, allocators,
// error text, trace counters).
#pragma once
#include <atomic>
#include <mutex>

#include "common.cuh"

struct fq_weights {
    fq::DevWeights dw;
    void* alloc;   // owning allocation (nullptr for views)
    size_t bytes;  // device bytes of the allocation
};

namespace fq {

struct Ctx {
    int device = -1;
    int sm_count = 0;
    cudaStream_t stream = nullptr;    // compute stream: every library kernel and copy is ordered here
    cudaStream_t transfer = nullptr;  // result copies of asynchronous submits, behind an event of their product
    cudaStream_t upload = nullptr;    // activation uploads of asynchronous submits (backend/cuda.zig's upload_stream)
    cudaEvent_t upload_ev = nullptr;  // marks the end of the latest upload; the compute stream waits on it
    size_t vram_budget = 0;
    int* status_host = nullptr;  // mapped status word, host view
    int* status_dev = nullptr;   // and the pointer kernels receive
    char name[256] = {0};
};

struct Trace {
    std::atomic<uint64_t> calls{0}, launches{0}, h2d_bytes{0}, d2h_bytes{0};
    std::atomic<uint64_t> resident_hits{0}, resident_adopts{0}, gate_pass{0}, gate_fail{0};
};
extern Trace g_trace;
extern std::recursive_mutex g_dispatch_lock;

int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
bool gpu_enabled();  // false when FUCINA_GPU=0 switched the provider off
Ctx* context();
Ctx* context_if_ready();  // the context only if it already exists; never creates it
int device_status(Ctx* ctx);  // FQ_OK, or the code a kernel's bounded wait left behind (then cleared)
// Device blocks from the caching allocator. Reuse is stream-ordered: the plain forms belong to the
// library's compute stream, the *_on forms name the stream that touches the block first (alloc) or
// last (free); neither waits on the host.
void* dev_alloc(size_t n);
void dev_free(void* p);
void* dev_alloc_on(size_t n, cudaStream_t st);
void dev_free_on(void* p, cudaStream_t st);
void dev_free_idle(void* p);  // for a block whose last use the host has already waited for
void* pin_alloc(size_t n);
void pin_free(void* p);

// Empty device weights in the layout an upload of this shape gets (tile-major for dense K-quants the decode kernel
// serves); gguf.cu repacks into them chunk by chunk.
int weights_alloc_layout(Ctx* ctx, int fmt, size_t n, size_t k, size_t n_mats, bool allow_tile, fq_weights** out);

// Host rhs bytes -> device view (resident registry hit, adoption, or a
// transient upload the caller frees through *temp after its launches).
int resolve_rhs(Ctx* ctx, int fmt, const void* rhs, size_t rhs_len, int cacheable, size_t nb01, size_t nb02, size_t n, size_t k,
                size_t n_mats, DevWeights* view, fq_weights** temp);

// c[m, ldc] (+)= a[m, k] . dequant(W[mat])^T on device buffers.
// split_n != 0: `w` stacks several matrices of split_n rows that share the activations (decode shapes only) and
// c_dev is laid out [matrix][m][split_n].
// pre: an activation prologue (rms_norm_mul / split_swiglu) applied to a_dev before the product: inside the decode
// kernel's quantiser where that kernel serves the shape, as a pass of its own otherwise.
int gemm_dev(Ctx* ctx, const DevWeights& w, int mat, const float* a_dev, float* c_dev, size_t m, size_t ldc, int mode,
             int accumulate, cudaStream_t st, int split_n = 0, const PreArgs* pre = nullptr);
// gemm_tc.cu: bf16 tensor-core path; returns FQ_DECLINED_ARGS for shapes it does not take.
int gemm_tensor_dev(Ctx* ctx, const DevWeights& w, int mat, const float* a_dev, float* c_dev, size_t m, size_t ldc,
                    cudaStream_t st);

// grouped form over bf16 activation rows and a device-built tile list (moe.cu)
struct TcTile;
struct TcPeer;
bool tensor_path_serves(const DevWeights& w);
int gemm_tensor_grouped_dev(Ctx* ctx, const DevWeights& w, const void* a_bf16, size_t rows, float* c_dev, size_t ldc,
                            const TcTile* table, const int* n_tiles_dev, int max_tiles, int tile_tokens, cudaStream_t st,
                            const TcPeer* peer = nullptr);
int gemm_tensor_grouped_gated_dev(Ctx* ctx, const DevWeights& gate, const DevWeights& up, const void* a_bf16, size_t rows, void* g_bf16,
                                  size_t ldc, const TcTile* table, const int* n_tiles_dev, int max_tiles, cudaStream_t st,
                                  const TcPeer* peer = nullptr, int gated_op = 0);

}  // namespace fq
