// An allocation-free variant of the small-batch quantized matmul.
//
// Some hosts of this library must not allocate device memory while they are
// running: an inference server that handed its whole VRAM budget to the KV
// cache and weights at start-up, a caller inside a latency-critical decode
// loop where a cudaMalloc (a device-wide synchronising call) would stall every
// stream, or an embedder whose memory is owned by an external pool it cannot
// grow. The regular entry points take their activation scratch from the
// library's caching allocator, which may call cudaMalloc the first time a size
// class is seen. This entry point never does: the int8 activation records the
// decode kernel consumes live in one fixed array inside the library image.
//
// Limits and rules (also stated in include/fucina_b200.h):
//   * m <= 16 activation rows; act_sizes(fmt, k).row * m <= kScratchBytes
//     (512 KiB); and, because the kernel keeps the rows padded to 1/2/4/8/16
//     in shared memory, act_sizes(fmt, k).row * pad(m) <= 227 KiB. A row is
//     about 1.1 * k bytes (1.3 * k for Q8_0). Larger requests are declined
//     with a clear message before anything is launched or written.
//   * every GPU that loads the library holds the 512 KiB until process exit.
//   * all calls share the array and it keeps the last call's contents; each
//     call rewrites every byte it later reads, so nothing needs clearing, but
//     two calls that overlap on the GPU (different streams, no ordering) race.
//   * the first call on a device resolves the array's device address; make
//     that first call before any stream capture.
//   * the library must already be initialised (fq_init): this entry never
//     creates the context, streams or any other resource itself.
#include "acts.cuh"
#include "internal.h"
#include "runtime.h"

namespace {

constexpr size_t kScratchBytes = 512 * 1024;
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for the symbol, not a device
// address: kernels get the pointer cudaGetSymbolAddress returns below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

// device address of the array, per device ordinal, resolved on first use
static unsigned char* g_scratch_ptr[kMaxDevices] = {nullptr};

}  // namespace

using namespace fq;

extern "C" int fq_gemm_quant_nt_dev_noalloc(const fq_weights* w, size_t mat, const float* a_dev, float* c_dev, size_t m,
                                            void* stream) {
    if (!w || !a_dev || !c_dev) return fail(FQ_DECLINED_ARGS, "null pointer");
    if (!gpu_enabled()) return fail(FQ_DECLINED_GATE, "disabled by FUCINA_GPU=0");
    Ctx* ctx = context_if_ready();
    if (!ctx) return fail(FQ_DECLINED_NO_GPU, "call fq_init before the allocation-free entry point");
    const DevWeights& dw = w->dw;
    if (mat >= (size_t)dw.n_mats) return fail(FQ_DECLINED_ARGS, "matrix index out of range");
    if (m == 0 || m > gemv_max_rows())
        return fail(FQ_DECLINED_ARGS, "the allocation-free entry takes 1..%zu activation rows, got %zu", gemv_max_rows(), m);
    const ActSizes S = act_sizes(dw.fmt, (size_t)dw.k);
    if (S.row == 0 || S.row * m > kScratchBytes)
        return fail(FQ_DECLINED_ARGS, "activation records need %zu bytes, the fixed scratch holds %zu", S.row * m, kScratchBytes);
    // the kernel keeps the rows, padded to 1/2/4/8/16, in shared memory: that is the tighter bound for long rows
    if (gemv_padded_rows(m) > gemv_rows_that_fit(dw.fmt, (size_t)dw.k))
        return fail(FQ_DECLINED_ARGS, "%d padded activation rows of %zu bytes do not fit the kernel's 227 KiB of shared memory",
                    gemv_padded_rows(m), S.row);

    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) return fail(FQ_DECLINED_ARGS, "device ordinal %d is outside the %d this entry keeps an address for", dev, kMaxDevices);
    if (!g_scratch_ptr[dev]) {
        // set-up, once per device, with that device current
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) return cuda_fail(e, "cudaGetSymbolAddress(scratch)");
        g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
    }
    unsigned char* scratch = g_scratch_ptr[dev];
    cudaStream_t st = stream ? (cudaStream_t)stream : ctx->stream;

    // same two kernels as the regular small-batch path, scratch aside
    e = launch_quantize_acts_layout(a_dev, nullptr, 1, (int)m, dw.k, dw.fmt, scratch, st);
    if (e != cudaSuccess) return cuda_fail(e, "activation quantise launch");
    GemvArgs ga{dw, DevWeights{}, (int)mat, scratch, c_dev, (int)m, dw.n, 0, nullptr, nullptr, 0};
    e = launch_gemv(ga, ctx->sm_count, st);
    g_trace.launches += 2;
    g_trace.calls++;
    return e == cudaSuccess ? FQ_OK : cuda_fail(e, "gemv launch");
}
