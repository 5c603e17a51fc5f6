// Provider runtime behind the C ABI: lazy context, caching device / pinned
// allocators, the resident-weight registry, completion tokens, gates and
// trace counters. Mirrors the host side of the reference's CUDA provider
// (src/backend/cuda.zig) on the CUDA runtime API; kernels live in formats.cu,
// gemv.cu, gemm_tc.cu and moe.cu.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "acts.cuh"
#include "internal.h"
#include "runtime.h"

namespace fq {

// ---------------------------------------------------------------------------
// error text
// ---------------------------------------------------------------------------
static std::mutex g_err_lock;
static std::string g_last_error;

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    std::lock_guard<std::mutex> g(g_err_lock);
    g_last_error = buf;
    return code;
}
int cuda_fail(cudaError_t e, const char* what) {
    cudaGetLastError();  // a launch or API error is reported once: the next healthy call must not find it
    return fail(FQ_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

// ---------------------------------------------------------------------------
// trace counters (backend/cuda.zig:191-317)
// ---------------------------------------------------------------------------
Trace g_trace;
static bool g_trace_on = false;
// FUCINA_B200_DECODE_ROWS=0 keeps every decode shape on the lane-per-chunk kernel (diagnosis switch)
static bool g_decode_rows_on = true;

// Device-side duration of the decode kernel, the CUDA-event twin of the
// reference's per-kind nanosecond counters (backend/cuda.zig:231-257). While
// enabled, every decode-kernel launch is bracketed by an event pair on its
// stream; the pairs are read back when the totals are queried.
static bool g_ktime_on = false;
static std::vector<std::pair<cudaEvent_t, cudaEvent_t>> g_ktime_events;
static std::vector<cudaEvent_t> g_ktime_pool;
static cudaEvent_t ktime_event() {
    if (!g_ktime_pool.empty()) {
        cudaEvent_t e = g_ktime_pool.back();
        g_ktime_pool.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}

// ---------------------------------------------------------------------------
// configuration read once from the environment (backend/cuda.zig:321-408)
// ---------------------------------------------------------------------------
struct Config {
    bool gpu_enabled = true;
    bool decode_enabled = true;  // the decode kernels match the CPU kernels' int8 arithmetic, so on by default
    // Work floors (m * n * k) below which the host should keep a product on the CPU. The reference's defaults
    // (backend/cuda.zig:118-159) are the crossovers of an RTX 5000 Ada laptop GPU against its CPU arms; these are the
    // crossovers measured on B200: the blocking host-buffer call (about 25 us at decode sizes, resident weights)
    // against the all-core CPU arm on the reference's packed row layouts (x8 K-quants, x4 Q8_0), its fastest. One
    // activation row: the CPU wins up to n * k = 2^21 (17 against 25 us), ties at 2^22, loses from 2^23; four rows:
    // the GPU wins from m * n * k = 2^22 (31 against 34 us); 64 rows: everywhere measured.
    uint64_t min_work_qmoe = 1ull << 24;        // grouped MoE GEMM over staged panels (reference 2^30)
    uint64_t min_work_dense = 1ull << 22;       // prefill-sized dense products against the plain CPU arm (reference 2^30 via the QMoE floor)
    uint64_t min_work_packed_q4 = 1ull << 22;   // ... against the packed (x8) CPU arms (reference 2^27)
    uint64_t min_work_packed_q5 = 1ull << 22;   // (reference 2^24)
    uint64_t min_work_packed_q8 = 1ull << 22;   // (reference 2^24)
    uint64_t min_work_decode = 1ull << 22;      // decode products, every format (the reference has no floor except for Q5_K)
    uint64_t min_work_decode_q5 = 1ull << 22;   // (reference 3 * 2^23)
    uint64_t qmoe_min_fill_pct = 50;
    size_t vram_budget_env = 0;
};
static Config g_cfg;
static std::once_flag g_cfg_once;

static bool env_u64(const char* name, uint64_t* out) {
    const char* v = getenv(name);
    if (!v || !*v) return false;
    char* end = nullptr;
    const unsigned long long x = strtoull(v, &end, 10);
    if (end == v) return false;
    *out = x;
    return true;
}
static void ensure_config() {
    std::call_once(g_cfg_once, [] {
        uint64_t v;
        if (env_u64("FUCINA_GPU", &v)) g_cfg.gpu_enabled = v != 0;
        if (env_u64("FUCINA_GPU_DECODE", &v)) g_cfg.decode_enabled = v != 0;
        if (env_u64("FUCINA_GPU_TRACE", &v)) g_trace_on = v != 0;
        if (env_u64("FUCINA_B200_DECODE_ROWS", &v)) g_decode_rows_on = v != 0;
        env_u64("FUCINA_GPU_MIN_WORK_QMOE", &g_cfg.min_work_qmoe);
        env_u64("FUCINA_GPU_MIN_WORK_DENSE_Q4", &g_cfg.min_work_packed_q4);
        env_u64("FUCINA_GPU_MIN_WORK_DENSE_Q5", &g_cfg.min_work_packed_q5);
        env_u64("FUCINA_GPU_MIN_WORK_DENSE_Q8", &g_cfg.min_work_packed_q8);
        env_u64("FUCINA_GPU_MIN_WORK_DECODE_Q5", &g_cfg.min_work_decode_q5);
        env_u64("FUCINA_GPU_MIN_WORK_GEMV", &g_cfg.min_work_decode);
        env_u64("FUCINA_GPU_MIN_WORK", &g_cfg.min_work_dense);
        env_u64("FUCINA_GPU_QMOE_MIN_FILL", &g_cfg.qmoe_min_fill_pct);
        if (env_u64("FUCINA_GPU_VRAM_BUDGET", &v)) g_cfg.vram_budget_env = (size_t)v;
    });
}

// ---------------------------------------------------------------------------
// context (backend/cuda.zig:412-508)
// ---------------------------------------------------------------------------
static Ctx g_ctx;
static std::mutex g_init_lock;
static std::atomic<int> g_init_state{0};  // 0 = not tried, 1 = ok, 2 = failed
std::recursive_mutex g_dispatch_lock;

static int init_locked(int device) {
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) return fail(FQ_DECLINED_NO_GPU, "no CUDA device: %s", cudaGetErrorString(e));
    if (device < 0) {
        if (cudaGetDevice(&device) != cudaSuccess) device = 0;
    }
    if (device >= count) return fail(FQ_DECLINED_NO_GPU, "device %d out of range (%d present)", device, count);
    if ((e = cudaSetDevice(device)) != cudaSuccess) return fail(FQ_DECLINED_NO_GPU, "cudaSetDevice: %s", cudaGetErrorString(e));
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess)
        return fail(FQ_DECLINED_NO_GPU, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    if (prop.major != 10)
        return fail(FQ_DECLINED_NO_GPU, "device %d is sm_%d%d; this library holds sm_100a code only", device, prop.major, prop.minor);
    g_ctx.device = device;
    g_ctx.sm_count = prop.multiProcessorCount;
    snprintf(g_ctx.name, sizeof g_ctx.name, "%s", prop.name);
    if ((e = cudaStreamCreateWithFlags(&g_ctx.stream, cudaStreamNonBlocking)) != cudaSuccess)
        return fail(FQ_DECLINED_NO_GPU, "cudaStreamCreate: %s", cudaGetErrorString(e));
    if ((e = cudaStreamCreateWithFlags(&g_ctx.transfer, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaStreamCreateWithFlags(&g_ctx.upload, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&g_ctx.upload_ev, cudaEventDisableTiming)) != cudaSuccess)
        return fail(FQ_DECLINED_NO_GPU, "cudaStreamCreate: %s", cudaGetErrorString(e));
    size_t free_b = 0, total_b = 0;
    cudaMemGetInfo(&free_b, &total_b);
    g_ctx.vram_budget = g_cfg.vram_budget_env ? g_cfg.vram_budget_env : (size_t)((double)free_b * 0.8);
    // status word kernels write when a bounded wait gives up: mapped host memory, read without a copy
    if ((e = cudaHostAlloc((void**)&g_ctx.status_host, sizeof(int), cudaHostAllocMapped)) != cudaSuccess ||
        (e = cudaHostGetDevicePointer((void**)&g_ctx.status_dev, g_ctx.status_host, 0)) != cudaSuccess)
        return fail(FQ_DECLINED_NO_GPU, "status word allocation: %s", cudaGetErrorString(e));
    *g_ctx.status_host = 0;
    return FQ_OK;
}

bool gpu_enabled() {
    ensure_config();
    return g_cfg.gpu_enabled;
}

Ctx* context() {
    ensure_config();
    int st = g_init_state.load(std::memory_order_acquire);
    if (st == 0) {
        std::lock_guard<std::mutex> g(g_init_lock);
        st = g_init_state.load(std::memory_order_relaxed);
        if (st == 0) {
            st = (init_locked(-1) == FQ_OK) ? 1 : 2;
            g_init_state.store(st, std::memory_order_release);
        }
    }
    if (st != 1) return nullptr;
    // entries can arrive on arbitrary threads (backend/cuda.zig:1776-1779)
    cudaSetDevice(g_ctx.device);
    return &g_ctx;
}

// The context if fq_init (or an earlier entry) already created it; never initialises.
Ctx* context_if_ready() {
    if (g_init_state.load(std::memory_order_acquire) != 1) return nullptr;
    cudaSetDevice(g_ctx.device);
    return &g_ctx;
}

// A kernel whose bounded wait gave up leaves its code in the status word; the
// host reports it at the next synchronisation point and clears it.
int device_status(Ctx* ctx) {
    const int s = *(volatile int*)ctx->status_host;
    if (s == 0) return FQ_OK;
    *(volatile int*)ctx->status_host = 0;
    if (s == FQ_ERR_CAPACITY) return fail(s, "the routing sent a GPU more rows than its exchange arena holds");
    return fail(s, "a device-side wait gave up (status %d)", s);
}

// ---------------------------------------------------------------------------
// caching allocators (the device-side twin of src/caching_allocator.zig's
// size-class freelist; replaces the grow-only DeviceBuf / PinnedBuf of
// backend/cuda.zig:873-890, :1026-1041). Blocks are recycled by class and
// only returned to the driver by trim().
//
// Reuse is stream-ordered: a block goes back to the cache together with the
// stream of its last use and an event recorded there, and nothing waits on
// the host. The next taker on the same stream is ordered by the stream
// itself; a taker on another stream first makes its stream wait for that
// event, so kernels still reading the block finish before the new owner's
// first write. Blocks released while their stream is being captured into a
// graph carry no event (an event recorded during capture cannot be waited on
// outside it); a taker on another stream then waits for that stream on the
// host.
// ---------------------------------------------------------------------------
static size_t size_class(size_t n) {
    if (n <= 512) return 512;
    if (n <= (1u << 20)) {
        size_t c = 512;
        while (c < n) c <<= 1;
        return c;
    }
    const size_t mb2 = 2u << 20;
    return (n + mb2 - 1) / mb2 * mb2;
}

class BlockCache {
   public:
    explicit BlockCache(bool pinned) : pinned_(pinned) {}
    // `st`: the stream that touches the block first (ignored for pinned host blocks)
    void* alloc(size_t n, cudaStream_t st) {
        const size_t c = size_class(n);
        std::lock_guard<std::mutex> g(lock_);
        auto it = free_.find(c);
        if (it != free_.end() && !it->second.empty()) {
            std::vector<Cached>& v = it->second;
            // a block whose last use is already ordered before `st` costs nothing
            size_t pick = v.size() - 1;
            for (size_t i = v.size(); i-- > 0;)
                if (v[i].idle || v[i].stream == st) {
                    pick = i;
                    break;
                }
            Cached b = v[pick];
            v.erase(v.begin() + pick);
            if (!b.idle && b.stream != st) {
                // a capturing stream cannot take an outside event as a dependency: wait on the host then
                cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
                if (st && cudaStreamIsCapturing(st, &cs) != cudaSuccess) cudaGetLastError();
                if (b.ev && cs == cudaStreamCaptureStatusNone) cudaStreamWaitEvent(st, b.ev, 0);
                else if (b.ev) cudaEventSynchronize(b.ev);
                else cudaStreamSynchronize(b.stream);
            }
            if (b.ev) events_.push_back(b.ev);
            live_[b.p] = c;
            cached_ -= c;
            return b.p;
        }
        void* p = nullptr;
        cudaError_t e = pinned_ ? cudaHostAlloc(&p, c, cudaHostAllocDefault) : cudaMalloc(&p, c);
        if (e != cudaSuccess) {
            // give cached blocks back to the driver and retry once
            cudaGetLastError();
            trim_locked();
            e = pinned_ ? cudaHostAlloc(&p, c, cudaHostAllocDefault) : cudaMalloc(&p, c);
            if (e != cudaSuccess) {
                cudaGetLastError();
                return nullptr;
            }
        }
        live_[p] = c;
        total_ += c;
        return p;
    }
    // `st`: the stream of the block's last use; `idle` = the host already waited for it
    void release(void* p, cudaStream_t st, bool idle) {
        if (!p) return;
        std::lock_guard<std::mutex> g(lock_);
        auto it = live_.find(p);
        if (it == live_.end()) return;
        Cached b{p, st, nullptr, idle || pinned_};
        if (!b.idle) {
            cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
            if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) cudaGetLastError();
            if (cs == cudaStreamCaptureStatusNone) {
                cudaEvent_t ev = nullptr;
                if (!events_.empty()) {
                    ev = events_.back();
                    events_.pop_back();
                } else if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) {
                    cudaGetLastError();
                    ev = nullptr;
                }
                if (ev && cudaEventRecord(ev, st) != cudaSuccess) {
                    cudaGetLastError();
                    events_.push_back(ev);
                    ev = nullptr;
                }
                b.ev = ev;
            }
        }
        free_[it->second].push_back(b);
        cached_ += it->second;
        live_.erase(it);
    }
    void trim() {
        std::lock_guard<std::mutex> g(lock_);
        trim_locked();
    }
    size_t total() const { return total_; }

   private:
    struct Cached {
        void* p;
        cudaStream_t stream;
        cudaEvent_t ev;
        bool idle;
    };
    void trim_locked() {
        for (auto& kv : free_)
            for (Cached& b : kv.second) {
                if (!b.idle) {
                    if (b.ev) cudaEventSynchronize(b.ev);
                    else cudaStreamSynchronize(b.stream);
                }
                if (b.ev) events_.push_back(b.ev);
                if (pinned_) cudaFreeHost(b.p); else cudaFree(b.p);
                total_ -= kv.first;
            }
        free_.clear();
        cached_ = 0;
    }
    bool pinned_;
    std::mutex lock_;
    std::map<size_t, std::vector<Cached>> free_;
    std::unordered_map<void*, size_t> live_;
    std::vector<cudaEvent_t> events_;
    size_t total_ = 0, cached_ = 0;
};
static BlockCache g_dev_cache(false), g_pin_cache(true);

// Without a stream argument a block belongs to the library's compute stream.
void* dev_alloc(size_t n) { return g_dev_cache.alloc(n, g_ctx.stream); }
void dev_free(void* p) { g_dev_cache.release(p, g_ctx.stream, false); }
void* dev_alloc_on(size_t n, cudaStream_t st) { return g_dev_cache.alloc(n, st); }
void dev_free_on(void* p, cudaStream_t st) { g_dev_cache.release(p, st, false); }
void dev_free_idle(void* p) { g_dev_cache.release(p, nullptr, true); }  // the host already waited for the block's last use
void* pin_alloc(size_t n) { return g_pin_cache.alloc(n, nullptr); }
void pin_free(void* p) { g_pin_cache.release(p, nullptr, true); }

// ---------------------------------------------------------------------------
// weights
// ---------------------------------------------------------------------------
}  // namespace fq

namespace fq {

static int check_format(int fmt) {
    return format_info(fmt).block_elems ? FQ_OK : fail(FQ_DECLINED_ARGS, "format %d is not served by this provider", fmt);
}

static int check_dims(int fmt, size_t n, size_t k, size_t n_mats, size_t nb01, size_t nb02) {
    if (int rc = check_format(fmt)) return rc;
    const FormatInfo f = format_info(fmt);
    if (n == 0 || k == 0 || n_mats == 0) return fail(FQ_DECLINED_ARGS, "empty weight matrix");
    if (n > INT32_MAX || k > INT32_MAX || n_mats > INT32_MAX) return fail(FQ_DECLINED_ARGS, "dimension exceeds int32");
    if (k % 32 != 0 || k % f.block_elems != 0) return fail(FQ_DECLINED_ARGS, "k=%zu is not a whole number of %d-element blocks", k, f.block_elems);
    const size_t row = k / f.block_elems * f.block_bytes;
    if (nb01 < row || nb01 % 2 != 0) return fail(FQ_DECLINED_ARGS, "nb01=%zu too small or odd for k=%zu", nb01, k);
    if (f.sc_bytes == 0 && nb01 % 16 != 0) return fail(FQ_DECLINED_ARGS, "K-quant row stride must be a multiple of 16 bytes");
    if (n_mats > 1 && (nb02 < nb01 * n || nb02 % 2 != 0 || (f.sc_bytes == 0 && nb02 % 16 != 0)))
        return fail(FQ_DECLINED_ARGS, "nb02=%zu inconsistent with n=%zu nb01=%zu", nb02, n, nb01);
    return FQ_OK;
}

// Build the device layout from raw GGUF bytes already on the device.
// Dense K-quant matrices the streaming decode kernel serves are stored tile-major (common.cuh).
static bool want_tile_major(int fmt, size_t n, size_t k, size_t n_mats, bool allow) {
    static const bool off = getenv("FUCINA_B200_NO_TILE") != nullptr;
    return allow && !off && n_mats == 1 && (fmt == FQ_Q4_K || fmt == FQ_Q5_K) && k % 256 == 0 && k >= 2048 && n >= 64;
}

static int weights_from_dev_bytes(Ctx* ctx, int fmt, const uint8_t* raw_dev, size_t nb01, size_t nb02, size_t n, size_t k,
                                  size_t n_mats, bool allow_tile, fq_weights** out) {
    const bool tile = want_tile_major(fmt, n, k, n_mats, allow_tile);
    const size_t stride = dev_row_stride(fmt, k);
    const size_t mat_stride = stride * (tile ? (n + 31) / 32 * 32 : n);
    const size_t bytes = mat_stride * n_mats;
    void* p = dev_alloc(bytes);
    if (!p) return fail(FQ_DECLINED_BUDGET, "device allocation of %zu bytes failed", bytes);
    if (tile && n % 32 != 0) cudaMemsetAsync(p, 0, bytes, ctx->stream);  // rows padding the last tile read as zero blocks
    fq_weights* w = new fq_weights();
    w->dw = {(const uint8_t*)p, stride, mat_stride, fmt, (int)n, (int)k, (int)n_mats, tile ? 32 : 0};
    w->alloc = p;
    w->bytes = bytes;
    if ((stride * n) % 16 != 0 || ((uintptr_t)raw_dev % 2) != 0) {
        dev_free(p);
        delete w;
        return fail(FQ_DECLINED_ARGS, "unaligned weight bytes");
    }
    // K-quant rows are copied in 16-byte units: the source must be 16-byte aligned
    if (format_info(fmt).sc_bytes == 0 && ((uintptr_t)raw_dev % 16) != 0) {
        dev_free(p);
        delete w;
        return fail(FQ_DECLINED_ARGS, "K-quant device bytes must be 16-byte aligned");
    }
    cudaError_t e = launch_repack(w->dw, raw_dev, nb01, n_mats > 1 ? nb02 : nb01 * n, true, ctx->stream);
    g_trace.launches++;
    if (e != cudaSuccess) {
        dev_free(p);
        delete w;
        return cuda_fail(e, "repack launch");
    }
    *out = w;
    return FQ_OK;
}

// Empty device weights in the layout weights_from_dev_bytes would choose; the caller repacks into them piece by piece.
int weights_alloc_layout(Ctx* ctx, int fmt, size_t n, size_t k, size_t n_mats, bool allow_tile, fq_weights** out) {
    if (int rc = check_dims(fmt, n, k, n_mats, fq_row_bytes(fmt, k), fq_row_bytes(fmt, k) * n)) return rc;
    const bool tile = want_tile_major(fmt, n, k, n_mats, allow_tile);
    const size_t stride = dev_row_stride(fmt, k);
    const size_t mat_stride = stride * (tile ? (n + 31) / 32 * 32 : n);
    const size_t bytes = mat_stride * n_mats;
    void* p = dev_alloc(bytes);
    if (!p) return fail(FQ_DECLINED_BUDGET, "device allocation of %zu bytes failed", bytes);
    if (tile && n % 32 != 0) cudaMemsetAsync(p, 0, bytes, ctx->stream);  // rows padding the last tile read as zero blocks
    fq_weights* w = new fq_weights();
    w->dw = {(const uint8_t*)p, stride, mat_stride, fmt, (int)n, (int)k, (int)n_mats, tile ? 32 : 0};
    w->alloc = p;
    w->bytes = bytes;
    *out = w;
    return FQ_OK;
}

static int weights_upload_impl(Ctx* ctx, int fmt, const void* host, size_t nb01, size_t nb02, size_t n, size_t k, size_t n_mats,
                               bool allow_tile, fq_weights** out) {
    if (int rc = check_dims(fmt, n, k, n_mats, nb01, nb02)) return rc;
    const size_t span = (n_mats > 1 ? nb02 * (n_mats - 1) : 0) + nb01 * n;
    void* raw = dev_alloc(span);
    if (!raw) return fail(FQ_DECLINED_BUDGET, "device allocation of %zu bytes failed", span);
    cudaError_t e = cudaMemcpyAsync(raw, host, span, cudaMemcpyHostToDevice, ctx->stream);
    g_trace.h2d_bytes += span;
    if (e != cudaSuccess) {
        dev_free(raw);
        return cuda_fail(e, "weight upload");
    }
    int rc = weights_from_dev_bytes(ctx, fmt, (const uint8_t*)raw, nb01, nb02, n, k, n_mats, allow_tile, out);
    // the raw copy is only read by the repack kernel queued above on the same stream
    e = cudaStreamSynchronize(ctx->stream);
    dev_free(raw);
    if (rc == FQ_OK && e != cudaSuccess) {
        fq_weights_free(*out);
        *out = nullptr;
        return cuda_fail(e, "weight repack");
    }
    return rc;
}

// ---------------------------------------------------------------------------
// resident registry (backend/cuda.zig:1518-1611, :1733-1806): host source
// range -> device twin, budgeted, 512 entries.
// ---------------------------------------------------------------------------
struct ResidentEntry {
    uintptr_t src_base;
    size_t len;
    bool owned;          // fq_alloc_resident bytes (page-locked host memory we own)
    fq_weights* twin;    // device copy, made on first use
    size_t nb01;
};
static const size_t kResidentSlots = 512;
static std::mutex g_res_lock;
static std::vector<ResidentEntry> g_res;
static size_t g_res_outstanding = 0;

static int resident_find(uintptr_t p, size_t len) {
    for (size_t i = 0; i < g_res.size(); ++i)
        if (p >= g_res[i].src_base && p + len <= g_res[i].src_base + g_res[i].len) return (int)i;
    return -1;
}

// Resolve host rhs bytes to a device view of `n` rows x `n_mats` matrices.
// temp != nullptr on return means the caller must free it after the launch.
int resolve_rhs(Ctx* ctx, int fmt, const void* rhs, size_t rhs_len, int cacheable, size_t nb01, size_t nb02, size_t n,
                       size_t k, size_t n_mats, DevWeights* view, fq_weights** temp) {
    *temp = nullptr;
    if (int rc = check_dims(fmt, n, k, n_mats, nb01, nb02)) return rc;
    const size_t span = (n_mats > 1 ? nb02 * (n_mats - 1) : 0) + nb01 * n;
    if (rhs_len < span) return fail(FQ_DECLINED_ARGS, "rhs_len=%zu shorter than the %zu bytes the shape needs", rhs_len, span);
    const uintptr_t p = (uintptr_t)rhs;
    {
        std::unique_lock<std::mutex> g(g_res_lock);
        int i = resident_find(p, span);
        if (i < 0 && cacheable) {
            // adopt by source address
            if (g_res.size() >= kResidentSlots) return fail(FQ_DECLINED_BUDGET, "resident registry full");
            const size_t need = dev_row_stride(fmt, k) * (rhs_len / nb01);
            if (ctx->vram_budget > 0 && g_res_outstanding + need > ctx->vram_budget)
                return fail(FQ_DECLINED_BUDGET, "resident budget exceeded (%zu + %zu > %zu)", g_res_outstanding, need, ctx->vram_budget);
            g_res.push_back({p, rhs_len, false, nullptr, 0});
            i = (int)g_res.size() - 1;
            g_trace.resident_adopts++;
        }
        if (i >= 0) {
            ResidentEntry& e = g_res[i];
            if (!e.twin) {
                // the whole range becomes rows of nb01 bytes (an expert stack is rows too when nb02 == n*nb01)
                if (n_mats > 1 && nb02 != nb01 * n) return fail(FQ_DECLINED_ARGS, "resident expert stacks must be dense (nb02 == n*nb01)");
                const size_t rows_total = e.len / nb01;
                const size_t need = dev_row_stride(fmt, k) * rows_total;
                if (ctx->vram_budget > 0 && g_res_outstanding + need > ctx->vram_budget)
                    return fail(FQ_DECLINED_BUDGET, "resident budget exceeded (%zu + %zu > %zu)", g_res_outstanding, need, ctx->vram_budget);
                fq_weights* w = nullptr;
                const void* src_base = (const void*)e.src_base;  // `e` may move once the lock drops
                g.unlock();
                int rc = weights_upload_impl(ctx, fmt, src_base, nb01, 0, rows_total, k, 1, n_mats == 1 && rows_total == n, &w);
                g.lock();
                if (rc != FQ_OK) return rc;
                ResidentEntry& e2 = g_res[resident_find(p, span)];
                if (e2.twin) {
                    fq_weights_free(w);  // raced with another adopter; keep theirs
                } else {
                    e2.twin = w;
                    e2.nb01 = nb01;
                    g_res_outstanding += w->bytes;
                }
            } else {
                g_trace.resident_hits++;
            }
            ResidentEntry& e3 = g_res[resident_find(p, span)];
            const fq_weights* tw = e3.twin;
            if (tw->dw.fmt != fmt || tw->dw.k != (int)k || e3.nb01 != nb01)
                return fail(FQ_DECLINED_ARGS, "resident bytes were registered with a different format or row shape");
            const size_t off = p - e3.src_base;
            if (off % nb01 != 0 || (n_mats > 1 && nb02 != nb01 * n))
                return fail(FQ_DECLINED_ARGS, "rhs does not start on a weight row of its resident range");
            if (tw->dw.tile_rows && ((off / nb01) % 32 != 0 || (n_mats > 1 && n % 32 != 0)))
                return fail(FQ_DECLINED_ARGS, "a sub-range of tile-major resident weights must start on a 32-row boundary");
            *view = tw->dw;
            view->base += (off / nb01) * tw->dw.row_stride;
            view->n = (int)n;
            view->n_mats = (int)n_mats;
            view->mat_stride = tw->dw.row_stride * n;
            return FQ_OK;
        }
    }
    // transient: stream the bytes for this call only
    fq_weights* w = nullptr;
    int rc = weights_upload_impl(ctx, fmt, rhs, nb01, nb02, n, k, n_mats, true, &w);
    if (rc != FQ_OK) return rc;
    *view = w->dw;
    *temp = w;
    return FQ_OK;
}

// ---------------------------------------------------------------------------
// dense matmul on device buffers
// ---------------------------------------------------------------------------
int gemm_dev(Ctx* ctx, const DevWeights& w, int mat, const float* a_dev, float* c_dev, size_t m, size_t ldc, int mode,
             int accumulate, cudaStream_t st, int split_n, const PreArgs* pre) {
    if (m == 0) return fail(FQ_DECLINED_ARGS, "m == 0");
    if (mat < 0 || mat >= w.n_mats) return fail(FQ_DECLINED_ARGS, "matrix index out of range");
    if (pre && pre->op != FQ_PRE_NONE) {
        const bool fuse = !accumulate && g_decode_rows_on && mode != FQ_MODE_TENSOR && decode_rows_fuses_prologue(w, m);
        if (!fuse) {
            // shapes whose kernel has no fused prologue: the same arithmetic as a pass of its own into a scratch
            // [m][k] block, then the plain product
            float* act = (float*)dev_alloc_on(m * (size_t)w.k * sizeof(float), st);
            if (!act) return fail(FQ_DECLINED_BUDGET, "activation scratch allocation failed");
            cudaError_t e = launch_act_prologue(*pre, a_dev, act, (int)m, w.k, st);
            g_trace.launches++;
            int rc = e == cudaSuccess ? gemm_dev(ctx, w, mat, act, c_dev, m, ldc, mode, accumulate, st, split_n, nullptr)
                                      : cuda_fail(e, "activation prologue launch");
            dev_free_on(act, st);
            return rc;
        }
    }
    if (split_n && !(g_decode_rows_on && !accumulate && decode_rows_eligible(w, m) && w.n % split_n == 0))
        return fail(FQ_DECLINED_ARGS, "stacked matrices are served by the decode kernel only");
    if (split_n) mode = FQ_MODE_INT8;
    if (mode == FQ_MODE_TENSOR || (mode == FQ_MODE_AUTO && m > gemv_max_rows() && !accumulate)) {
        int rc = gemm_tensor_dev(ctx, w, mat, a_dev, c_dev, m, ldc, st);
        if (rc != FQ_DECLINED_ARGS || mode == FQ_MODE_TENSOR) return rc;
        // shapes the tensor-core kernel does not take fall through to the integer kernel
    }
    // dense decode shapes: the row-per-lane kernel with TMA-staged weights
    if ((!accumulate || w.fmt == FQ_TQ2_0) && g_decode_rows_on && decode_rows_eligible(w, m)) {
        const size_t sb = decode_rows_scratch_bytes(w, m);
        uint8_t* nat = sb ? (uint8_t*)dev_alloc_on(sb, st) : nullptr;
        if (sb && !nat) return fail(FQ_DECLINED_BUDGET, "activation scratch allocation failed");
        cudaEvent_t t0 = nullptr, t1 = nullptr;
        if (g_ktime_on) {
            t0 = ktime_event();
            t1 = ktime_event();
            cudaEventRecord(t0, st);
        }
        cudaError_t e = launch_decode_rows(w, mat, a_dev, nat, c_dev, (int)m, (int)ldc, ctx->sm_count, ctx->status_dev, st, split_n, pre, accumulate);
        if (g_ktime_on) {
            cudaEventRecord(t1, st);
            g_ktime_events.emplace_back(t0, t1);
        }
        g_trace.launches += sb ? 2 : 1;
        dev_free_on(nat, st);  // stream-ordered reuse: no host wait
        return e == cudaSuccess ? FQ_OK : cuda_fail(e, "decode launch");
    }
    const ActSizes S = act_sizes(w.fmt, w.k);
    // rows per launch: what the kernel is instantiated for, cut down until the padded rows fit its shared memory
    const size_t chunk_max = (size_t)gemv_rows_that_fit(w.fmt, (size_t)w.k);
    if (chunk_max == 0) return fail(FQ_DECLINED_ARGS, "k=%d is too long for the small-batch kernel (one activation row needs %zu bytes of shared memory)", w.k, S.row);
    const size_t rows_scratch = m < chunk_max ? m : chunk_max;
    uint8_t* scratch = (uint8_t*)dev_alloc_on(S.row * rows_scratch, st);
    if (!scratch) return fail(FQ_DECLINED_BUDGET, "activation scratch allocation failed");
    int rc = FQ_OK;
    for (size_t r0 = 0; r0 < m && rc == FQ_OK; r0 += chunk_max) {
        const int rows = (int)((m - r0) < chunk_max ? (m - r0) : chunk_max);
        cudaError_t e = launch_quantize_acts_layout(a_dev + r0 * w.k, nullptr, 1, rows, w.k, w.fmt, scratch, st);
        g_trace.launches++;
        if (e != cudaSuccess) { rc = cuda_fail(e, "activation quantise launch"); break; }
        GemvArgs ga{w, DevWeights{}, mat, scratch, c_dev + r0 * ldc, rows, (int)ldc, accumulate, nullptr, nullptr, 0};
        cudaEvent_t t0 = nullptr, t1 = nullptr;
        if (g_ktime_on) {
            t0 = ktime_event();
            t1 = ktime_event();
            cudaEventRecord(t0, st);
        }
        e = launch_gemv(ga, ctx->sm_count, st);
        if (g_ktime_on) {
            cudaEventRecord(t1, st);
            g_ktime_events.emplace_back(t0, t1);
        }
        g_trace.launches++;
        if (e != cudaSuccess) rc = cuda_fail(e, "gemv launch");
    }
    // the scratch block returns to the cache with its stream and an event: a later taker is
    // ordered after these kernels without a host wait
    dev_free_on(scratch, st);
    return rc;
}

// ---------------------------------------------------------------------------
// host-buffer helpers
// ---------------------------------------------------------------------------
static bool host_is_pinned(const void* p) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return attr.type == cudaMemoryTypeHost;
}

// ---------------------------------------------------------------------------
// host registration (backend/cuda.zig:1047-1082 `ensureHostRegistered`): the caller page-locks a storage range
// once; activations are then copied by DMA straight from it and decode-sized results are written by the kernel
// straight into it -- no bounce through a staging buffer.
// ---------------------------------------------------------------------------
struct HostRange {
    uintptr_t base;
    size_t len;
    uint8_t* dev;  // the range as the device addresses it
};
static std::mutex g_host_lock;
static std::vector<HostRange> g_host_ranges;

// device view of [p, p + len) when it lies inside a registered range, else nullptr
static void* registered_dev_ptr(const void* p, size_t len) {
    const uintptr_t a = (uintptr_t)p;
    std::lock_guard<std::mutex> g(g_host_lock);
    for (const HostRange& r : g_host_ranges)
        if (a >= r.base && a + len <= r.base + r.len) return r.dev + (a - r.base);
    return nullptr;
}

struct Staged {
    void* dev = nullptr;
    void* pin = nullptr;
};

// `st`: the stream the copy is queued on (and the first to touch the staging block)
static int upload_f32(Ctx* ctx, const float* host, size_t bytes, Staged* s, cudaStream_t st = nullptr) {
    if (!st) st = ctx->stream;
    s->dev = dev_alloc_on(bytes, st);
    if (!s->dev) return fail(FQ_DECLINED_BUDGET, "device allocation of %zu bytes failed", bytes);
    const void* src = host;
    // registered storage is DMA-able as it is; other small rows are always staged (copying a few KB costs less
    // than asking the driver what kind of memory it is)
    if (registered_dev_ptr(host, bytes)) {
    } else if (bytes <= 64 * 1024 || !host_is_pinned(host)) {
        s->pin = pin_alloc(bytes);
        if (!s->pin) return fail(FQ_DECLINED_BUDGET, "pinned allocation of %zu bytes failed", bytes);
        memcpy(s->pin, host, bytes);
        src = s->pin;
    }
    cudaError_t e = cudaMemcpyAsync(s->dev, src, bytes, cudaMemcpyHostToDevice, st);
    g_trace.h2d_bytes += bytes;
    return e == cudaSuccess ? FQ_OK : cuda_fail(e, "activation upload");
}

static int download_f32(Ctx* ctx, const void* dev, float* host, size_t bytes) {
    cudaError_t e;
    if (host_is_pinned(host)) {
        e = cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    } else {
        void* pin = pin_alloc(bytes);
        if (!pin) return fail(FQ_DECLINED_BUDGET, "pinned allocation of %zu bytes failed", bytes);
        e = cudaMemcpyAsync(pin, dev, bytes, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e == cudaSuccess) memcpy(host, pin, bytes);
        pin_free(pin);
    }
    g_trace.d2h_bytes += bytes;
    return e == cudaSuccess ? FQ_OK : cuda_fail(e, "result download");
}

static int gate_and_ctx(Ctx** out) {
    ensure_config();
    if (!g_cfg.gpu_enabled) return fail(FQ_DECLINED_GATE, "disabled by FUCINA_GPU=0");
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    *out = ctx;
    return FQ_OK;
}

static int check_gemm_args(int fmt, size_t batch, size_t m, size_t n, size_t k) {
    if (int rc = check_format(fmt)) return rc;
    if (batch == 0 || m == 0 || n == 0 || k == 0) return fail(FQ_DECLINED_ARGS, "empty problem");
    if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX || batch > INT32_MAX) return fail(FQ_DECLINED_ARGS, "dimension exceeds int32");
    // backend/cuda.zig:2017: n % 4 == 0, k a whole number of blocks and of 32
    if (n % 4 != 0) return fail(FQ_DECLINED_ARGS, "n=%zu is not a multiple of 4", n);
    if (k % 32 != 0 || k % format_info(fmt).block_elems != 0) return fail(FQ_DECLINED_ARGS, "k=%zu is not a whole number of blocks", k);
    return FQ_OK;
}

// shared body of the blocking host entries: batch weight matrices, one shared input
static int gemm_host(int fmt, const void* rhs, size_t rhs_len, int cacheable, size_t nb01, size_t nb02, const float* a, float* c,
                     size_t batch, size_t m, size_t n, size_t k) {
    if (!rhs || !a || !c) return fail(FQ_DECLINED_ARGS, "null pointer");
    if (int rc = check_gemm_args(fmt, batch, m, n, k)) return rc;
    Ctx* ctx = nullptr;
    if (int rc = gate_and_ctx(&ctx)) return rc;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    g_trace.calls++;
    DevWeights view;
    fq_weights* temp = nullptr;
    // A dense stack of matrices that share a decode-sized input (Q/K/V, gate/up) is one matrix of batch * n
    // rows to the streaming kernel: one launch, activations quantised once per CTA, every SM busy
    // (backend/cuda.zig:2441-2492 launches per matrix).
    bool stacked = false;
    if (batch > 1 && nb02 == nb01 * n && g_decode_rows_on && batch * n <= (size_t)INT32_MAX) {
        DevWeights probe{};
        probe.fmt = fmt, probe.n = (int)(batch * n), probe.k = (int)k, probe.n_mats = 1;
        stacked = decode_rows_eligible(probe, m);
    }
    int rc = stacked ? resolve_rhs(ctx, fmt, rhs, rhs_len, cacheable, nb01, 0, batch * n, k, 1, &view, &temp)
                     : resolve_rhs(ctx, fmt, rhs, rhs_len, cacheable, nb01, nb02, n, k, batch, &view, &temp);
    if (rc != FQ_OK) return rc;
    Staged in;
    const size_t out_bytes = batch * m * n * sizeof(float);
    void* c_dev = nullptr;
    void* c_pin = nullptr;
    rc = upload_f32(ctx, a, m * k * sizeof(float), &in);
    // Decode-sized results are written by the kernel straight into page-locked host memory (device-visible
    // under unified addressing): one copy operation and its latency less per call.
    const bool direct_out = m <= 8 && out_bytes <= (size_t)1 << 20;
    void* c_reg = direct_out ? registered_dev_ptr(c, out_bytes) : nullptr;  // registered result storage: the kernel writes it in place
    if (rc == FQ_OK) {
        if (c_reg) {
            c_dev = c_reg;
        } else if (direct_out) {
            c_pin = pin_alloc(out_bytes);
            c_dev = c_pin;
        } else {
            c_dev = dev_alloc(out_bytes);
        }
        if (!c_dev) rc = fail(FQ_DECLINED_BUDGET, "result allocation of %zu bytes failed", out_bytes);
    }
    bool submitted = false;
    if (stacked && rc == FQ_OK) {
        rc = gemm_dev(ctx, view, 0, (const float*)in.dev, (float*)c_dev, m, n, FQ_MODE_INT8, 0, ctx->stream, (int)n);
        submitted = true;
    }
    for (size_t b = 0; b < batch && rc == FQ_OK && !stacked; ++b) {
        rc = gemm_dev(ctx, view, (int)b, (const float*)in.dev, (float*)c_dev + b * m * n, m, n, FQ_MODE_AUTO, 0, ctx->stream);
        submitted = true;
    }
    if (rc == FQ_OK && direct_out) {
        cudaError_t e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) rc = cuda_fail(e, "result wait");
        else if (!c_reg) memcpy(c, c_pin, out_bytes);
        g_trace.d2h_bytes += out_bytes;
    } else if (rc == FQ_OK) {
        rc = download_f32(ctx, c_dev, c, out_bytes);
    } else if (submitted) {
        cudaStreamSynchronize(ctx->stream);
    }
    if (rc == FQ_OK) rc = device_status(ctx);  // a bounded device-side wait that gave up invalidates the result
    // every path above ended in a host wait on the stream: the blocks go back idle (no event to record)
    if (c_reg) {
    } else if (direct_out) pin_free(c_pin);
    else dev_free_idle(c_dev);
    dev_free_idle(in.dev);
    pin_free(in.pin);
    if (temp) fq_weights_free(temp);
    // a decline after kernels were queued wrote nothing to `c`; device failures stay negative
    return rc;
}

// ---------------------------------------------------------------------------
// async completion tokens (accelerator.zig:22-133; backend/cuda.zig:1087-1218)
// ---------------------------------------------------------------------------
static const int kAsyncSlots = 8;
static std::atomic<int> g_slots_in_use{0};
// completion events are recycled: creating and destroying one per submit costs microseconds of driver time
static std::vector<cudaEvent_t> g_token_events;
static cudaEvent_t token_event_get() {
    if (!g_token_events.empty()) {
        cudaEvent_t e = g_token_events.back();
        g_token_events.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return e;
}
static void token_event_put(cudaEvent_t e) {
    if (e) g_token_events.push_back(e);
}

}  // namespace fq

struct fq_work {
    void* c_dev;
    size_t bytes;
    float* c_host;
    cudaEvent_t done;
    int state;  // 0 submitted, 1 host_ready, 2 discarded, -1 failed
    void* in_dev;  // staged activations: released once the product has run (finish / destroy)
    void* in_pin;
    void* c_pin;   // decode-sized results are copied out at submit time: page-locked staging (or nullptr)
    int early_copy;  // 1: the device-to-host copy was queued behind the product (into c_pin, or into registered c_host)
};

using namespace fq;

extern "C" {

int fq_init(int device) {
    ensure_config();
    std::lock_guard<std::mutex> g(g_init_lock);
    if (g_init_state.load() == 1) return (device < 0 || device == g_ctx.device) ? FQ_OK : fail(FQ_DECLINED_ARGS, "already initialised on device %d", g_ctx.device);
    const int rc = init_locked(device);
    g_init_state.store(rc == FQ_OK ? 1 : 2);
    return rc;
}
int fq_device_count(void) {
    int c = 0;
    if (cudaGetDeviceCount(&c) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return c;
}
const char* fq_device_name(void) { return context() ? g_ctx.name : ""; }
int fq_sm_count(void) { return context() ? g_ctx.sm_count : 0; }
int fq_last_error(char* buf, size_t len) {
    std::lock_guard<std::mutex> g(g_err_lock);
    if (buf && len) snprintf(buf, len, "%s", g_last_error.c_str());
    return (int)g_last_error.size();
}
void* fq_stream(void) { return context() ? (void*)g_ctx.stream : nullptr; }
// Test seam: exercise the device-side time-out path. A warp waits `limit` polls (at most 2^20) on a barrier
// that is never completed, gives up and records FQ_ERR_TIMEOUT; the next fq_synchronize (or blocking entry)
// returns it, and the context stays usable. No counterpart in the reference.
int fq_selftest_bounded_wait(unsigned limit) {
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    if (limit == 0 || limit > (1u << 20)) return fail(FQ_DECLINED_ARGS, "limit must be in 1..2^20");
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    cudaError_t e = launch_bounded_wait_probe(ctx->status_dev, limit, ctx->stream);
    return e == cudaSuccess ? FQ_OK : cuda_fail(e, "bounded-wait probe launch");
}
int fq_synchronize(void) {
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->transfer);  // result copies of asynchronous submits
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->upload);
    if (e != cudaSuccess) return cuda_fail(e, "synchronize");
    return device_status(ctx);
}

size_t fq_block_elems(int fmt) { return format_info(fmt).block_elems; }
size_t fq_block_bytes(int fmt) { return format_info(fmt).block_bytes; }
size_t fq_row_bytes(int fmt, size_t k) {
    const FormatInfo f = format_info(fmt);
    return f.block_elems ? k / f.block_elems * f.block_bytes : 0;
}

// ---- residency ------------------------------------------------------------
void* fq_alloc_resident(size_t len) {
    Ctx* ctx = nullptr;
    if (len == 0 || gate_and_ctx(&ctx) != FQ_OK) return nullptr;
    {
        std::lock_guard<std::mutex> g(g_res_lock);
        if (g_res.size() >= kResidentSlots || (ctx->vram_budget > 0 && g_res_outstanding + len > ctx->vram_budget)) {
            fail(FQ_DECLINED_BUDGET, "resident budget exceeded");
            return nullptr;
        }
    }
    void* p = nullptr;
    if (cudaHostAlloc(&p, len, cudaHostAllocDefault) != cudaSuccess) {
        cudaGetLastError();
        fail(FQ_DECLINED_BUDGET, "page-locked allocation of %zu bytes failed", len);
        return nullptr;
    }
    std::lock_guard<std::mutex> g(g_res_lock);
    g_res.push_back({(uintptr_t)p, len, true, nullptr, 0});
    return p;
}
static void drop_entry_locked(size_t i) {
    ResidentEntry e = g_res[i];
    g_res.erase(g_res.begin() + i);
    if (e.twin) {
        g_res_outstanding -= e.twin->bytes;
        fq_weights_free(e.twin);
    }
    if (e.owned) cudaFreeHost((void*)e.src_base);
}
void fq_free_resident(const void* p) {
    if (!p || !context()) return;
    std::lock_guard<std::recursive_mutex> d(g_dispatch_lock);
    cudaStreamSynchronize(g_ctx.stream);
    std::lock_guard<std::mutex> g(g_res_lock);
    for (size_t i = 0; i < g_res.size(); ++i)
        if (g_res[i].src_base == (uintptr_t)p) {
            drop_entry_locked(i);
            return;
        }
}
int fq_evict_resident(const void* host_ptr) {
    if (!context()) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> d(g_dispatch_lock);
    cudaStreamSynchronize(g_ctx.stream);
    std::lock_guard<std::mutex> g(g_res_lock);
    const int i = resident_find((uintptr_t)host_ptr, 1);
    if (i < 0) return fail(FQ_DECLINED_ARGS, "address is not resident");
    if (g_res[i].owned) return fail(FQ_DECLINED_ARGS, "owned resident bytes are released with fq_free_resident");
    drop_entry_locked(i);
    return FQ_OK;
}
size_t fq_resident_bytes(void) {
    std::lock_guard<std::mutex> g(g_res_lock);
    return g_res_outstanding;
}
int fq_host_register(void* host_ptr, size_t len) {
    if (!host_ptr || len == 0) return fail(FQ_DECLINED_ARGS, "null range");
    Ctx* ctx = nullptr;
    if (int rc = gate_and_ctx(&ctx)) return rc;
    {
        std::lock_guard<std::mutex> g(g_host_lock);
        for (const HostRange& r : g_host_ranges)
            if ((uintptr_t)host_ptr >= r.base && (uintptr_t)host_ptr + len <= r.base + r.len) return FQ_OK;  // already covered
        if (g_host_ranges.size() >= 4096) return fail(FQ_DECLINED_BUDGET, "too many registered host ranges");
    }
    cudaError_t e = cudaHostRegister(host_ptr, len, cudaHostRegisterMapped | cudaHostRegisterPortable);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(FQ_DECLINED_ARGS, "cudaHostRegister of %zu bytes: %s", len, cudaGetErrorString(e));
    }
    void* dev = nullptr;
    if (cudaHostGetDevicePointer(&dev, host_ptr, 0) != cudaSuccess || !dev) {
        cudaGetLastError();
        cudaHostUnregister(host_ptr);
        return fail(FQ_DECLINED_ARGS, "registered memory has no device address");
    }
    std::lock_guard<std::mutex> g(g_host_lock);
    g_host_ranges.push_back({(uintptr_t)host_ptr, len, (uint8_t*)dev});
    return FQ_OK;
}
int fq_host_unregister(void* host_ptr) {
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> d(g_dispatch_lock);
    cudaStreamSynchronize(ctx->stream);  // no copy or kernel may still address the range
    cudaStreamSynchronize(ctx->transfer);
    cudaStreamSynchronize(ctx->upload);
    std::lock_guard<std::mutex> g(g_host_lock);
    for (size_t i = 0; i < g_host_ranges.size(); ++i)
        if (g_host_ranges[i].base == (uintptr_t)host_ptr) {
            g_host_ranges.erase(g_host_ranges.begin() + i);
            cudaHostUnregister(host_ptr);
            cudaGetLastError();
            return FQ_OK;
        }
    return fail(FQ_DECLINED_ARGS, "address is not the start of a registered range");
}
int fq_set_vram_budget(size_t bytes) {
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    ctx->vram_budget = bytes;
    return FQ_OK;
}

// ---- explicit device weights ----------------------------------------------
int fq_weights_upload(int fmt, const void* host_blocks, size_t nb01, size_t nb02, size_t n, size_t k, size_t n_mats,
                      fq_weights** out) {
    if (!host_blocks || !out) return fail(FQ_DECLINED_ARGS, "null pointer");
    Ctx* ctx = nullptr;
    if (int rc = gate_and_ctx(&ctx)) return rc;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    return weights_upload_impl(ctx, fmt, host_blocks, nb01, nb02, n, k, n_mats, true, out);
}
int fq_weights_from_device(int fmt, const void* dev_blocks, size_t nb01, size_t nb02, size_t n, size_t k, size_t n_mats,
                           fq_weights** out) {
    if (!dev_blocks || !out) return fail(FQ_DECLINED_ARGS, "null pointer");
    Ctx* ctx = nullptr;
    if (int rc = gate_and_ctx(&ctx)) return rc;
    if (int rc = check_dims(fmt, n, k, n_mats, nb01, nb02)) return rc;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    int rc = weights_from_dev_bytes(ctx, fmt, (const uint8_t*)dev_blocks, nb01, nb02, n, k, n_mats, true, out);
    if (rc == FQ_OK) {
        cudaError_t e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) return cuda_fail(e, "weight repack");
    }
    return rc;
}
// Rows [row0, row0 + rows) of every matrix of `w` as weights of their own (no copy; `w` must outlive the view and is
// freed separately). A fused gate_up tensor [E][2 * out_pe][hidden] splits into its gate and up halves this way
// (llm/gemma/moe.zig:696-901), and a resident matrix into column shards.
int fq_weights_view(const fq_weights* w, size_t row0, size_t rows, fq_weights** out) {
    if (!w || !out) return fail(FQ_DECLINED_ARGS, "null pointer");
    const DevWeights& d = w->dw;
    if (rows == 0 || row0 + rows > (size_t)d.n) return fail(FQ_DECLINED_ARGS, "row range [%zu, %zu) outside the %d rows of the matrix", row0, row0 + rows, d.n);
    if (d.tile_rows && (row0 % 32 != 0 || (d.n_mats > 1 && rows % 32 != 0)))
        return fail(FQ_DECLINED_ARGS, "a view of tile-major weights must start on a 32-row boundary");
    fq_weights* v = new fq_weights();
    v->dw = d;
    v->dw.base = d.base + (d.tile_rows ? (row0 / 32) * ((size_t)32 * d.row_stride) : row0 * d.row_stride);
    v->dw.n = (int)rows;
    v->alloc = nullptr;  // a view owns nothing
    v->bytes = 0;
    *out = v;
    return FQ_OK;
}
void fq_weights_free(fq_weights* w) {
    if (!w) return;
    if (w->alloc) dev_free(w->alloc);
    delete w;
}
size_t fq_weights_device_bytes(const fq_weights* w) { return w ? w->bytes : 0; }

int fq_weights_download_gguf(const fq_weights* w, void* host_blocks, size_t len) {
    if (!w || !host_blocks) return fail(FQ_DECLINED_ARGS, "null pointer");
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    const size_t nb01 = fq_row_bytes(w->dw.fmt, w->dw.k);
    const size_t span = nb01 * w->dw.n * w->dw.n_mats;
    if (len < span) return fail(FQ_DECLINED_ARGS, "buffer too small (%zu < %zu)", len, span);
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    void* raw = dev_alloc(span);
    if (!raw) return fail(FQ_DECLINED_BUDGET, "device allocation failed");
    cudaError_t e = launch_repack(w->dw, (const uint8_t*)raw, nb01, nb01 * w->dw.n, false, ctx->stream);
    g_trace.launches++;
    if (e == cudaSuccess) e = cudaMemcpyAsync(host_blocks, raw, span, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    dev_free(raw);
    g_trace.d2h_bytes += span;
    return e == cudaSuccess ? FQ_OK : cuda_fail(e, "weight download");
}

int fq_dequantize_rows_dev(const fq_weights* w, size_t mat, size_t row0, size_t rows, float* dev_out) {
    if (!w || !dev_out) return fail(FQ_DECLINED_ARGS, "null pointer");
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    if (mat >= (size_t)w->dw.n_mats || row0 + rows > (size_t)w->dw.n || rows == 0) return fail(FQ_DECLINED_ARGS, "row range out of bounds");
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    cudaError_t e = launch_dequant_rows(w->dw, (int)mat, (int)row0, (int)rows, dev_out, ctx->stream);
    g_trace.launches++;
    return e == cudaSuccess ? FQ_OK : cuda_fail(e, "dequant launch");
}
int fq_dequantize_rows(const fq_weights* w, size_t mat, size_t row0, size_t rows, float* host_out) {
    if (!w || !host_out) return fail(FQ_DECLINED_ARGS, "null pointer");
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    const size_t bytes = rows * (size_t)w->dw.k * sizeof(float);
    void* d = dev_alloc(bytes);
    if (!d) return fail(FQ_DECLINED_BUDGET, "device allocation failed");
    int rc = fq_dequantize_rows_dev(w, mat, row0, rows, (float*)d);
    if (rc == FQ_OK) rc = download_f32(ctx, d, host_out, bytes);
    cudaStreamSynchronize(ctx->stream);
    dev_free(d);
    return rc;
}

int fq_quantize_rows_dev(int fmt, const float* dev_src, size_t n, size_t k, void* dev_blocks) {
    if (!dev_src || !dev_blocks) return fail(FQ_DECLINED_ARGS, "null pointer");
    if (fmt == FQ_TQ2_0_FOLDED) return fail(FQ_DECLINED_ARGS, "folded blocks are built from two planes, not from f32 rows");
    const FormatInfo f = format_info(fmt);
    if (!f.block_elems || k == 0 || n == 0 || k % f.block_elems != 0) return fail(FQ_DECLINED_ARGS, "k=%zu is not a whole number of blocks", k);
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    cudaError_t e = launch_quantize_weights(fmt, dev_src, n, k, (uint8_t*)dev_blocks, ctx->stream);
    g_trace.launches++;
    return e == cudaSuccess ? FQ_OK : cuda_fail(e, "weight encoder launch");
}

// ---- dense, host buffers ----------------------------------------------------
int fq_gemm_quant_nt(int fmt, const void* rhs, size_t rhs_len, int cacheable, size_t nb01, const float* a, float* c, size_t m,
                     size_t n, size_t k) {
    return gemm_host(fmt, rhs, rhs_len, cacheable, nb01, 0, a, c, 1, m, n, k);
}
int fq_gemm_quant_nt_shared_a_batch(int fmt, const void* rhs, size_t rhs_len, int cacheable, size_t nb01, size_t nb02,
                                    const float* a, float* c, size_t batch, size_t m, size_t n, size_t k) {
    return gemm_host(fmt, rhs, rhs_len, cacheable, nb01, nb02, a, c, batch, m, n, k);
}

// ---- async -------------------------------------------------------------------
int fq_gemm_quant_nt_async(int fmt, const void* rhs, size_t rhs_len, int cacheable, size_t nb01, size_t nb02, const float* a,
                           fq_work* a_dep, float* c_host, size_t batch, size_t m, size_t n, size_t k, fq_work** out_work) {
    if (!rhs || (!a && !a_dep) || !out_work) return fail(FQ_DECLINED_ARGS, "null pointer");
    // the async arm only takes stable model weights (backend/cuda.zig:2014)
    if (!cacheable) return fail(FQ_DECLINED_ARGS, "async submit needs a cacheable rhs");
    if (int rc = check_gemm_args(fmt, batch, m, n, k)) return rc;
    if (a_dep && (a_dep->state != 0 || a_dep->bytes < m * k * sizeof(float))) return fail(FQ_DECLINED_ARGS, "dependency is not a pending producer of m*k floats");
    Ctx* ctx = nullptr;
    if (int rc = gate_and_ctx(&ctx)) return rc;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    if (g_slots_in_use.load() >= kAsyncSlots) return fail(FQ_DECLINED_BUSY, "all %d async slots are in flight", kAsyncSlots);
    g_trace.calls++;
    DevWeights view;
    fq_weights* temp = nullptr;
    bool stacked = false;  // a dense stack sharing a decode-sized input runs as one launch (see gemm_host)
    if (batch > 1 && nb02 == nb01 * n && g_decode_rows_on && batch * n <= (size_t)INT32_MAX) {
        DevWeights probe{};
        probe.fmt = fmt, probe.n = (int)(batch * n), probe.k = (int)k, probe.n_mats = 1;
        stacked = decode_rows_eligible(probe, m);
    }
    int rc = stacked ? resolve_rhs(ctx, fmt, rhs, rhs_len, 1, nb01, 0, batch * n, k, 1, &view, &temp)
                     : resolve_rhs(ctx, fmt, rhs, rhs_len, 1, nb01, nb02, n, k, batch, &view, &temp);
    if (rc != FQ_OK) return rc;
    Staged in;
    const float* a_dev = a_dep ? (const float*)a_dep->c_dev : nullptr;
    if (!a_dev) {
        // The upload runs on its own stream and the compute stream waits for its event (backend/cuda.zig:2056-2057):
        // a copy queued between two products on the compute stream would hold the second one back until the first
        // has drained, while here the next product's activations arrive under the current product. The event can
        // be recorded again by the next submit: a stream wait refers to the record that preceded it.
        rc = upload_f32(ctx, a, m * k * sizeof(float), &in, ctx->upload);
        a_dev = (const float*)in.dev;
        if (rc == FQ_OK) {
            cudaError_t e = cudaEventRecord(ctx->upload_ev, ctx->upload);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->stream, ctx->upload_ev, 0);
            if (e != cudaSuccess) rc = cuda_fail(e, "upload ordering");
        }
    }
    fq_work* w = nullptr;
    if (rc == FQ_OK) {
        w = new fq_work();
        w->bytes = batch * m * n * sizeof(float);
        // The result always has a device copy (a consumer chained on this token reads it there). Letting the kernel
        // store decode-sized results straight into registered host storage, as the blocking entry does, was
        // measured slower here: the next product of the queue may only pass its dependency wait once the
        // predecessor's stores across PCIe have drained (66 against 63.5 us for the four-product decode step).
        w->c_dev = dev_alloc(w->bytes);
        w->c_host = c_host;
        w->state = 0;
        w->done = nullptr;
        w->in_dev = nullptr;
        w->in_pin = nullptr;
        w->c_pin = nullptr;
        w->early_copy = 0;
        if (!w->c_dev) rc = fail(FQ_DECLINED_BUDGET, "device allocation failed");
        else if (!(w->done = token_event_get())) rc = fail(FQ_ERR_CUDA, "event create failed");
    }
    if (stacked && rc == FQ_OK) rc = gemm_dev(ctx, view, 0, a_dev, (float*)w->c_dev, m, n, FQ_MODE_INT8, 0, ctx->stream, (int)n);
    for (size_t b = 0; b < batch && rc == FQ_OK && !stacked; ++b)
        rc = gemm_dev(ctx, view, (int)b, a_dev, (float*)w->c_dev + b * m * n, m, n, FQ_MODE_AUTO, 0, ctx->stream);
    // Decode-sized results start their way to the host right behind the product, so a later finish only waits:
    // into the caller's registered storage directly, else into page-locked staging copied out by finish.
    // The copy runs on the transfer stream behind an event of the product, so the next product queued on the
    // compute stream does not wait for it; `done` then marks the end of the copy.
    if (rc == FQ_OK) {
        cudaError_t e = cudaEventRecord(w->done, ctx->stream);
        if (e != cudaSuccess) rc = cuda_fail(e, "event record");
    }
    if (rc == FQ_OK && c_host && w->bytes <= (size_t)1 << 20) {
        void* dst = registered_dev_ptr(c_host, w->bytes) ? (void*)c_host : (w->c_pin = pin_alloc(w->bytes));
        if (dst && cudaStreamWaitEvent(ctx->transfer, w->done, 0) == cudaSuccess &&
            cudaMemcpyAsync(dst, w->c_dev, w->bytes, cudaMemcpyDeviceToHost, ctx->transfer) == cudaSuccess &&
            cudaEventRecord(w->done, ctx->transfer) == cudaSuccess) {
            w->early_copy = 1;
            g_trace.d2h_bytes += w->bytes;
        } else {
            // `done` may have been left unrecorded on the transfer stream: mark the product's end again
            cudaGetLastError();
            cudaStreamSynchronize(ctx->transfer);
            cudaEventRecord(w->done, ctx->stream);
            pin_free(w->c_pin);
            w->c_pin = nullptr;
        }
    }
    // the staged activations stay with the token until it is finished: no host wait inside a submit
    if (rc == FQ_OK) {
        w->in_dev = in.dev;
        w->in_pin = in.pin;
    }
    if (rc != FQ_OK) {
        cudaStreamSynchronize(ctx->upload);
        cudaStreamSynchronize(ctx->stream);
        dev_free_idle(in.dev);
        pin_free(in.pin);
        if (w) {
            token_event_put(w->done);
            dev_free_idle(w->c_dev);
            pin_free(w->c_pin);
            delete w;
        }
        return rc;
    }
    g_slots_in_use++;
    *out_work = w;
    return FQ_OK;
}

int fq_work_finish(fq_work* w, int copy_to_host) {
    if (!w) return fail(FQ_DECLINED_ARGS, "null work");
    // host_ready, or waited without a copy and still none asked for: nothing left to do. A token that was
    // waited on first (copy_to_host = 0) and is now asked for the host copy falls through and downloads.
    if (w->state == 1 || (w->state == 2 && !(copy_to_host && w->c_host))) return FQ_OK;
    if (w->state < 0) return FQ_ERR_CUDA;
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    cudaError_t e = cudaEventSynchronize(w->done);
    if (e != cudaSuccess) {
        w->state = -1;
        return cuda_fail(e, "work wait");
    }
    dev_free_idle(w->in_dev);  // the product that read them has finished (the event above)
    pin_free(w->in_pin);
    w->in_dev = w->in_pin = nullptr;
    if (copy_to_host && w->c_host && w->early_copy) {
        // the copy was queued with the product and has landed: in place (registered storage) or in the staging block
        if (w->c_pin) memcpy(w->c_host, w->c_pin, w->bytes);
        w->state = 1;
    } else if (copy_to_host && w->c_host) {
        // order the copy after the producer on the compute stream
        int rc = download_f32(ctx, w->c_dev, w->c_host, w->bytes);
        if (rc != FQ_OK) {
            w->state = -1;
            return rc;
        }
        w->state = 1;
    } else {
        w->state = 2;
    }
    if (int st = device_status(ctx)) {  // a bounded device-side wait gave up somewhere before this point
        w->state = -1;
        return st;
    }
    return FQ_OK;
}
uintptr_t fq_work_device_ptr(fq_work* w) { return w ? (uintptr_t)w->c_dev : 0; }
void fq_work_destroy(fq_work* w) {
    if (!w) return;
    if (context()) {
        std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
        if (w->state == 0) cudaEventSynchronize(w->done);
        token_event_put(w->done);
        // a consumer chained on this output may still be queued on the library stream: the block returns
        // stream-ordered (an event, no host wait), so a later taker runs after that consumer
        dev_free(w->c_dev);
        dev_free_idle(w->in_dev);  // its reader finished before `done`
        pin_free(w->in_pin);
        pin_free(w->c_pin);
    }
    g_slots_in_use--;
    delete w;
}

// ---- dense, device buffers ---------------------------------------------------
int fq_gemm_quant_nt_dev(const fq_weights* w, size_t mat, const float* a_dev, float* c_dev, size_t m, int mode, void* stream) {
    if (!w || !a_dev || !c_dev) return fail(FQ_DECLINED_ARGS, "null pointer");
    Ctx* ctx = nullptr;
    if (int rc = gate_and_ctx(&ctx)) return rc;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    g_trace.calls++;
    return gemm_dev(ctx, w->dw, (int)mat, a_dev, c_dev, m, (size_t)w->dw.n, mode, 0, stream ? (cudaStream_t)stream : ctx->stream);
}
// ---- fused neighbours of the CPU path (exec/quant_matmul.zig:480-757) -------------------------------------------
static int check_pre(int pre_op, const DevWeights* dw, size_t k, const float* pre_w_dev) {
    if (pre_op != FQ_PRE_RMS_NORM_MUL && pre_op != FQ_PRE_SPLIT_SWIGLU) return fail(FQ_DECLINED_ARGS, "prologue %d is not one of FQ_PRE_*", pre_op);
    if (pre_op == FQ_PRE_RMS_NORM_MUL && !pre_w_dev) return fail(FQ_DECLINED_ARGS, "rms_norm_mul needs the norm weights");
    if (k == 0 || k % 256 != 0) return fail(FQ_DECLINED_ARGS, "activation prologues need k to be a multiple of 256");
    if (dw && (size_t)dw->k != k) return fail(FQ_DECLINED_ARGS, "k mismatch");
    return FQ_OK;
}
int fq_gemm_quant_nt_pre_dev(const fq_weights* w, size_t mat, int pre_op, const float* a_dev, const float* pre_w_dev, float eps,
                             float* c_dev, size_t m, int mode, void* stream) {
    if (!w || !a_dev || !c_dev) return fail(FQ_DECLINED_ARGS, "null pointer");
    if (pre_op == FQ_PRE_NONE) return fq_gemm_quant_nt_dev(w, mat, a_dev, c_dev, m, mode, stream);
    if (int rc = check_pre(pre_op, &w->dw, (size_t)w->dw.k, pre_w_dev)) return rc;
    Ctx* ctx = nullptr;
    if (int rc = gate_and_ctx(&ctx)) return rc;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    g_trace.calls++;
    const PreArgs pre{pre_op, pre_w_dev, eps};
    return gemm_dev(ctx, w->dw, (int)mat, a_dev, c_dev, m, (size_t)w->dw.n, mode, 0, stream ? (cudaStream_t)stream : ctx->stream, 0, &pre);
}
int fq_act_prologue_dev(int pre_op, const float* a_dev, const float* pre_w_dev, float eps, float* out_dev, size_t m, size_t k, void* stream) {
    if (!a_dev || !out_dev || m == 0 || m > 65535u * 32u) return fail(FQ_DECLINED_ARGS, "null pointer or row count");
    if (int rc = check_pre(pre_op, nullptr, k, pre_w_dev)) return rc;
    if (k > (size_t)1 << 22) return fail(FQ_DECLINED_ARGS, "k too large");
    Ctx* ctx = nullptr;
    if (int rc = gate_and_ctx(&ctx)) return rc;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    g_trace.calls++;
    const PreArgs pre{pre_op, pre_w_dev, eps};
    cudaError_t e = launch_act_prologue(pre, a_dev, out_dev, (int)m, (int)k, stream ? (cudaStream_t)stream : ctx->stream);
    g_trace.launches++;
    return e == cudaSuccess ? FQ_OK : cuda_fail(e, "activation prologue launch");
}
int fq_small_batch_max_rows(int fmt, size_t k) {
    const FormatInfo f = format_info(fmt);
    if (!f.block_elems || k == 0 || k % f.block_elems != 0 || k % 32 != 0) return 0;
    return gemv_rows_that_fit(fmt, k);
}
int fq_gemm_ptqtp_dev(const fq_weights* const* planes, int n_planes, const float* a_dev, float* c_dev, size_t m, void* stream) {
    if (!planes || n_planes < 1 || n_planes > 3 || !a_dev || !c_dev) return fail(FQ_DECLINED_ARGS, "bad plane list");
    for (int p = 0; p < n_planes; ++p) {
        if (!planes[p] || planes[p]->dw.fmt != FQ_TQ2_0) return fail(FQ_DECLINED_ARGS, "PTQTP planes are TQ2_0 tensors");
        if (planes[p]->dw.n != planes[0]->dw.n || planes[p]->dw.k != planes[0]->dw.k) return fail(FQ_DECLINED_ARGS, "plane shapes differ");
    }
    Ctx* ctx = nullptr;
    if (int rc = gate_and_ctx(&ctx)) return rc;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    g_trace.calls++;
    cudaStream_t st = stream ? (cudaStream_t)stream : ctx->stream;
    const size_t n = (size_t)planes[0]->dw.n;
    if (m > gemv_max_rows() && tensor_path_serves(planes[0]->dw) && (m * n) % 4 == 0) {
        // prefill-sized: each plane is a tensor-core product, summed per element in plane order (weights.zig:286-300)
        float* tmp = n_planes > 1 ? (float*)dev_alloc_on(m * n * sizeof(float), st) : nullptr;
        if (n_planes > 1 && !tmp) return fail(FQ_DECLINED_BUDGET, "plane scratch allocation failed");
        int rc = FQ_OK;
        for (int p = 0; p < n_planes && rc == FQ_OK; ++p) {
            rc = gemm_tensor_dev(ctx, planes[p]->dw, 0, a_dev, p ? tmp : c_dev, m, n, st);
            if (rc == FQ_OK && p) {
                cudaError_t e = launch_add_f32(c_dev, tmp, m * n, st);
                g_trace.launches++;
                if (e != cudaSuccess) rc = cuda_fail(e, "plane sum launch");
            }
        }
        dev_free_on(tmp, st);
        return rc;
    }
    for (int p = 0; p < n_planes; ++p) {
        int rc = gemm_dev(ctx, planes[p]->dw, 0, a_dev, c_dev, m, n, FQ_MODE_INT8, p > 0, st);
        if (rc != FQ_OK) return rc;
    }
    return FQ_OK;
}
static int quantize_acts_struct(const float* a_dev, size_t m, size_t k, void* dev_blocks, bool q8k) {
    if (!a_dev || !dev_blocks || m == 0 || k == 0) return fail(FQ_DECLINED_ARGS, "bad arguments");
    if (k % (q8k ? 256 : 32) != 0) return fail(FQ_DECLINED_ARGS, "k=%zu is not a whole number of activation blocks", k);
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    cudaError_t e = launch_quantize_acts_struct(a_dev, (int)m, (int)k, q8k, (uint8_t*)dev_blocks, ctx->stream);
    g_trace.launches++;
    return e == cudaSuccess ? FQ_OK : cuda_fail(e, "activation quantise launch");
}
int fq_quantize_acts_q8_k_dev(const float* a_dev, size_t m, size_t k, void* dev_blocks) { return quantize_acts_struct(a_dev, m, k, dev_blocks, true); }
int fq_quantize_acts_q8_0_dev(const float* a_dev, size_t m, size_t k, void* dev_blocks) { return quantize_acts_struct(a_dev, m, k, dev_blocks, false); }

// ---- gates (backend/cuda.zig:2494-2554) --------------------------------------
static int gate(bool pass) {
    if (pass) g_trace.gate_pass++; else g_trace.gate_fail++;
    return pass ? 1 : 0;
}
int fq_should_use_gpu_qmoe(uint64_t total_work) {
    ensure_config();
    return gate(g_cfg.gpu_enabled && total_work >= g_cfg.min_work_qmoe);
}
int fq_qmoe_fill_acceptable(size_t rows, size_t n_tiles) {
    ensure_config();
    if (n_tiles == 0) return 0;
    return (uint64_t)rows * 100 >= (uint64_t)n_tiles * 32 * g_cfg.qmoe_min_fill_pct;
}
int fq_should_use_gpu_dense_quant(int fmt, uint64_t total_work) {
    ensure_config();
    uint64_t floor_;
    switch (fmt) {
        case FQ_Q5_K: floor_ = g_cfg.min_work_packed_q5; break;
        case FQ_Q4_K: case FQ_Q8_0: floor_ = g_cfg.min_work_dense; break;
        default: floor_ = g_cfg.min_work_packed_q8; break;
    }
    return gate(g_cfg.gpu_enabled && format_info(fmt).block_elems && total_work >= floor_);
}
int fq_should_use_gpu_dense_quant_packed(int fmt, uint64_t total_work) {
    ensure_config();
    uint64_t floor_;
    switch (fmt) {
        case FQ_Q4_K: floor_ = g_cfg.min_work_packed_q4; break;
        case FQ_Q5_K: floor_ = g_cfg.min_work_packed_q5; break;
        default: floor_ = g_cfg.min_work_packed_q8; break;
    }
    return gate(g_cfg.gpu_enabled && format_info(fmt).block_elems && total_work >= floor_);
}
int fq_should_use_gpu_quant_decode(int fmt, size_t m, size_t n, size_t k) {
    ensure_config();
    if (!g_cfg.gpu_enabled || !g_cfg.decode_enabled || !format_info(fmt).block_elems) return 0;
    const unsigned __int128 work = (unsigned __int128)m * n * k;
    return gate(work >= (fmt == FQ_Q5_K ? g_cfg.min_work_decode_q5 : g_cfg.min_work_decode));
}
void fq_set_min_work_qmoe_for_test(uint64_t v) {
    ensure_config();
    g_cfg.min_work_qmoe = v;
}
void fq_set_decode_for_test(int enabled) {
    ensure_config();
    g_cfg.decode_enabled = enabled != 0;
}

// ---- trace -------------------------------------------------------------------
int fq_trace_enabled(void) {
    ensure_config();
    return g_trace_on ? 1 : 0;
}
void fq_trace_reset(void) {
    g_trace.calls = g_trace.launches = g_trace.h2d_bytes = g_trace.d2h_bytes = 0;
    g_trace.resident_hits = g_trace.resident_adopts = g_trace.gate_pass = g_trace.gate_fail = 0;
}
void fq_trace_counters(uint64_t out[8]) {
    if (!out) return;
    out[0] = g_trace.calls, out[1] = g_trace.launches, out[2] = g_trace.h2d_bytes, out[3] = g_trace.d2h_bytes;
    out[4] = g_trace.resident_hits, out[5] = g_trace.resident_adopts, out[6] = g_trace.gate_pass, out[7] = g_trace.gate_fail;
}
// ---- CUDA graphs over the library stream ---------------------------------------
// Decode steps are a handful of microsecond kernels; replaying them as one graph
// removes the per-launch host cost. Only *_dev entries that neither allocate
// nor synchronise may run between begin and end (the decode shapes with m <= 4).
int fq_capture_begin(void) {
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    g_dispatch_lock.lock();  // held until fq_capture_end: nothing else may touch the stream while it captures
    cudaError_t e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) {
        g_dispatch_lock.unlock();
        return cuda_fail(e, "begin capture");
    }
    return FQ_OK;
}
int fq_capture_end(fq_graph** out) {
    Ctx* ctx = context();
    if (!ctx || !out) {
        return fail(FQ_DECLINED_ARGS, "no capture in progress");
    }
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    cudaGraphExec_t exec = nullptr;
    if (e == cudaSuccess) e = cudaGraphInstantiate(&exec, graph, 0);
    if (graph) cudaGraphDestroy(graph);
    g_dispatch_lock.unlock();
    if (e != cudaSuccess) return cuda_fail(e, "end capture");
    *out = reinterpret_cast<fq_graph*>(exec);
    return FQ_OK;
}
int fq_graph_launch(fq_graph* g) {
    Ctx* ctx = context();
    if (!ctx || !g) return fail(FQ_DECLINED_ARGS, "null graph");
    std::lock_guard<std::recursive_mutex> lk(g_dispatch_lock);
    cudaError_t e = cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(g), ctx->stream);
    return e == cudaSuccess ? FQ_OK : cuda_fail(e, "graph launch");
}
void fq_graph_destroy(fq_graph* g) {
    if (g && context()) cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(g));
}

void fq_trace_kernel_timing(int enable) {
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    g_ktime_on = enable != 0;
}
int fq_trace_kernel_times(double* total_ms, uint64_t* launches) {
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    std::lock_guard<std::recursive_mutex> g(g_dispatch_lock);
    double sum = 0.0;
    uint64_t n = 0;
    for (auto& pr : g_ktime_events) {
        float ms = 0.0f;
        if (cudaEventSynchronize(pr.second) == cudaSuccess && cudaEventElapsedTime(&ms, pr.first, pr.second) == cudaSuccess) {
            sum += ms;
            ++n;
        }
        g_ktime_pool.push_back(pr.first);
        g_ktime_pool.push_back(pr.second);
    }
    g_ktime_events.clear();
    cudaGetLastError();
    if (total_ms) *total_ms = sum;
    if (launches) *launches = n;
    return FQ_OK;
}
void fq_trace_dump(void) {
    uint64_t c[8];
    fq_trace_counters(c);
    fprintf(stderr,
            "[fucina_b200] calls=%llu launches=%llu h2d=%llu B d2h=%llu B resident hits=%llu adopts=%llu gate pass=%llu fail=%llu "
            "resident=%zu B device cache=%zu B\n",
            (unsigned long long)c[0], (unsigned long long)c[1], (unsigned long long)c[2], (unsigned long long)c[3],
            (unsigned long long)c[4], (unsigned long long)c[5], (unsigned long long)c[6], (unsigned long long)c[7],
            fq_resident_bytes(), g_dev_cache.total());
}

}  // extern "C"
