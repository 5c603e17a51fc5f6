// GGUF file -> device-resident weights.
//
// The reference parses GGUF in src/gguf.zig (header, metadata, tensor table, data section aligned to
// `general.alignment`) and turns quantized tensors into resident GPU bytes in src/weights.zig:2621-2816
// (`allocResidentBytes` + memcpy of the mapped blocks). Here the mapped blocks go straight to the repacked device
// layouts ("gpu_formats" planes): a tensor is cut into row chunks that travel through two page-locked staging
// buffers, so reading the file (page faults on the mapping), the host-to-device copies and the repack kernels of
// consecutive chunks overlap. A row range and an expert range select the shard a rank owns (column-sharded linears,
// expert-parallel stacks). PTQTP models store one TQ2_0 tensor per trit plane, `<name>.ptqtp0/1/2`
// (src/ptqtp_gguf.zig:1-30, :95-98): fq_gguf_load_ptqtp_planes loads the planes that exist, in order.
//
// Parsing needs no GPU; loading needs fq_init.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <string>
#include <vector>

#include "internal.h"
#include "runtime.h"

namespace fq {

// ggml_type ids of the formats this library serves (ggml.h; src/gguf.zig:60-111)
static int fmt_of_ggml_type(int t) {
    switch (t) {
        case 8: return FQ_Q8_0;
        case 12: return FQ_Q4_K;
        case 13: return FQ_Q5_K;
        case 14: return FQ_Q6_K;
        case 35: return FQ_TQ2_0;
        default: return -1;
    }
}
// bytes of one row of `k` elements for the plain types, 0 when unknown here
static size_t plain_row_bytes(int t, uint64_t k) {
    switch (t) {
        case 0: return k * 4;   // f32
        case 1: return k * 2;   // f16
        case 30: return k * 2;  // bf16
        case 24: return k;      // i8
        case 25: return k * 2;  // i16
        case 26: return k * 4;  // i32
        case 27: return k * 8;  // i64
        case 28: return k * 8;  // f64
        default: return 0;
    }
}

struct MetaValue {
    uint32_t type;      // GGUF value type (0..12)
    const uint8_t* at;  // first byte of the value inside the mapping
};
struct TensorEntry {
    std::string name;
    int ggml_type, fmt, n_dims;
    uint64_t dims[4];
    uint64_t offset, bytes;  // offset from the start of the data section
};

}  // namespace fq

struct fq_gguf {
    int fd = -1;
    const uint8_t* map = nullptr;
    size_t len = 0;
    uint32_t version = 0;
    uint64_t alignment = 32;
    uint64_t data_start = 0;
    std::vector<std::pair<std::string, fq::MetaValue>> meta;
    std::vector<fq::TensorEntry> tensors;
};

namespace fq {

namespace {

struct Cursor {
    const uint8_t* p;
    const uint8_t* end;
    bool ok = true;
    template <class T>
    T get() {
        T v{};
        if ((size_t)(end - p) < sizeof(T)) {
            ok = false;
            return v;
        }
        memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    bool skip(uint64_t n) {
        if ((uint64_t)(end - p) < n) return ok = false;
        p += n;
        return true;
    }
    bool str(std::string* out) {
        const uint64_t n = get<uint64_t>();
        if (!ok || (uint64_t)(end - p) < n) return ok = false;
        if (out) out->assign((const char*)p, (size_t)n);
        p += n;
        return true;
    }
};

// bytes of a scalar metadata value, 0 for strings and arrays
size_t scalar_bytes(uint32_t t) {
    switch (t) {
        case 0: case 1: case 7: return 1;
        case 2: case 3: return 2;
        case 4: case 5: case 6: return 4;
        case 10: case 11: case 12: return 8;
        default: return 0;
    }
}
bool skip_value(Cursor& c, uint32_t t, int depth) {
    if (t == 8) return c.str(nullptr);
    if (t == 9) {
        if (depth > 4) return c.ok = false;
        const uint32_t et = c.get<uint32_t>();
        const uint64_t count = c.get<uint64_t>();
        if (!c.ok) return false;
        if (const size_t sb = scalar_bytes(et)) {
            if (count > (uint64_t)(c.end - c.p) / sb) return c.ok = false;
            return c.skip(count * sb);
        }
        if (et != 8 && et != 9) return c.ok = false;
        for (uint64_t i = 0; i < count && c.ok; ++i) skip_value(c, et, depth + 1);
        return c.ok;
    }
    const size_t sb = scalar_bytes(t);
    if (!sb) return c.ok = false;
    return c.skip(sb);
}

const MetaValue* find_meta(const fq_gguf* g, const char* key) {
    for (auto& kv : g->meta)
        if (kv.first == key) return &kv.second;
    return nullptr;
}

int parse(fq_gguf* g) {
    Cursor c{g->map, g->map + g->len};
    const uint32_t magic = c.get<uint32_t>();
    if (!c.ok || magic != 0x46554747u) return fail(FQ_DECLINED_ARGS, "not a GGUF file (magic %08x)", magic);
    g->version = c.get<uint32_t>();
    if (g->version < 2 || g->version > 3) return fail(FQ_DECLINED_ARGS, "GGUF version %u is not read here (2 and 3 are)", g->version);
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    if (!c.ok || n_tensors > (1u << 24) || n_kv > (1u << 24)) return fail(FQ_DECLINED_ARGS, "GGUF header is truncated or implausible");
    for (uint64_t i = 0; i < n_kv; ++i) {
        std::string key;
        c.str(&key);
        const uint32_t t = c.get<uint32_t>();
        const uint8_t* at = c.p;
        if (!c.ok || !skip_value(c, t, 0)) return fail(FQ_DECLINED_ARGS, "GGUF metadata entry %llu is truncated or malformed", (unsigned long long)i);
        g->meta.emplace_back(std::move(key), MetaValue{t, at});
    }
    if (const MetaValue* a = find_meta(g, "general.alignment")) {
        uint32_t v = 0;
        if (a->type == 4) memcpy(&v, a->at, 4);
        if (v == 0 || (v & (v - 1)) != 0) return fail(FQ_DECLINED_ARGS, "general.alignment must be a power of two");
        g->alignment = v;
    }
    g->tensors.reserve((size_t)n_tensors);
    for (uint64_t i = 0; i < n_tensors; ++i) {
        TensorEntry t;
        c.str(&t.name);
        t.n_dims = (int)c.get<uint32_t>();
        if (!c.ok || t.n_dims < 1 || t.n_dims > 4) return fail(FQ_DECLINED_ARGS, "GGUF tensor %llu has %d dimensions", (unsigned long long)i, t.n_dims);
        for (int d = 0; d < 4; ++d) t.dims[d] = d < t.n_dims ? c.get<uint64_t>() : 1;
        t.ggml_type = (int)c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        if (!c.ok) return fail(FQ_DECLINED_ARGS, "GGUF tensor table is truncated");
        t.fmt = fmt_of_ggml_type(t.ggml_type);
        uint64_t rows = 1;
        for (int d = 1; d < 4; ++d) {
            if (t.dims[d] != 0 && rows > UINT64_MAX / t.dims[d]) return fail(FQ_DECLINED_ARGS, "GGUF tensor '%s' overflows", t.name.c_str());
            rows *= t.dims[d];
        }
        size_t row = 0;
        if (t.fmt >= 0) {
            const FormatInfo f = format_info(t.fmt);
            if (t.dims[0] % f.block_elems != 0) return fail(FQ_DECLINED_ARGS, "GGUF tensor '%s': %llu columns are not whole blocks", t.name.c_str(), (unsigned long long)t.dims[0]);
            row = (size_t)(t.dims[0] / f.block_elems) * f.block_bytes;
        } else {
            row = plain_row_bytes(t.ggml_type, t.dims[0]);
        }
        if (row != 0 && rows > UINT64_MAX / row) return fail(FQ_DECLINED_ARGS, "GGUF tensor '%s' overflows", t.name.c_str());
        t.bytes = (uint64_t)row * rows;  // 0 for a type this reader cannot size (the entry is still listed)
        g->tensors.push_back(std::move(t));
    }
    const uint64_t pos = (uint64_t)(c.p - g->map);
    g->data_start = (pos + g->alignment - 1) / g->alignment * g->alignment;
    for (auto& t : g->tensors) {
        if (t.offset % g->alignment != 0) return fail(FQ_DECLINED_ARGS, "GGUF tensor '%s' is not aligned to %llu bytes", t.name.c_str(), (unsigned long long)g->alignment);
        if (g->data_start + t.offset > g->len || t.bytes > g->len - g->data_start - t.offset)
            return fail(FQ_DECLINED_ARGS, "GGUF tensor '%s' runs past the end of the file", t.name.c_str());
    }
    return FQ_OK;
}

constexpr size_t kChunkBytes = (size_t)32 << 20;  // staging buffer size: two of these, page-locked

}  // namespace
}  // namespace fq

using namespace fq;

extern "C" {

int fq_gguf_open(const char* path, fq_gguf** out) {
    if (!path || !out) return fail(FQ_DECLINED_ARGS, "null pointer");
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(FQ_DECLINED_ARGS, "cannot open '%s'", path);
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) {
        close(fd);
        return fail(FQ_DECLINED_ARGS, "'%s' is too short for a GGUF header", path);
    }
    void* map = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (map == MAP_FAILED) {
        close(fd);
        return fail(FQ_DECLINED_ARGS, "cannot map '%s'", path);
    }
    fq_gguf* g = new fq_gguf();
    g->fd = fd;
    g->map = (const uint8_t*)map;
    g->len = (size_t)st.st_size;
    const int rc = parse(g);
    if (rc != FQ_OK) {
        fq_gguf_close(g);
        return rc;
    }
    *out = g;
    return FQ_OK;
}

void fq_gguf_close(fq_gguf* g) {
    if (!g) return;
    if (g->map) munmap((void*)g->map, g->len);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

size_t fq_gguf_tensor_count(const fq_gguf* g) { return g ? g->tensors.size() : 0; }

int fq_gguf_tensor_at(const fq_gguf* g, size_t i, fq_gguf_tensor* out) {
    if (!g || !out || i >= g->tensors.size()) return fail(FQ_DECLINED_ARGS, "tensor index out of range");
    const TensorEntry& t = g->tensors[i];
    out->name = t.name.c_str();
    out->ggml_type = t.ggml_type;
    out->fmt = t.fmt;
    out->n_dims = t.n_dims;
    for (int d = 0; d < 4; ++d) out->dims[d] = t.dims[d];
    out->offset = g->data_start + t.offset;
    out->bytes = t.bytes;
    return FQ_OK;
}

int fq_gguf_find(const fq_gguf* g, const char* name) {
    if (!g || !name) return -1;
    for (size_t i = 0; i < g->tensors.size(); ++i)
        if (g->tensors[i].name == name) return (int)i;
    return -1;
}

const void* fq_gguf_tensor_data(const fq_gguf* g, size_t i) {
    if (!g || i >= g->tensors.size()) return nullptr;
    return g->map + g->data_start + g->tensors[i].offset;
}

int fq_gguf_meta_u64(const fq_gguf* g, const char* key, uint64_t* out) {
    if (!g || !key || !out) return fail(FQ_DECLINED_ARGS, "null pointer");
    const MetaValue* v = find_meta(g, key);
    if (!v) return fail(FQ_DECLINED_ARGS, "no metadata key '%s'", key);
    uint64_t r = 0;
    switch (v->type) {
        case 0: case 7: r = *v->at; break;
        case 2: { uint16_t x; memcpy(&x, v->at, 2); r = x; break; }
        case 4: { uint32_t x; memcpy(&x, v->at, 4); r = x; break; }
        case 10: memcpy(&r, v->at, 8); break;
        case 1: { int8_t x; memcpy(&x, v->at, 1); if (x < 0) return fail(FQ_DECLINED_ARGS, "'%s' is negative", key); r = (uint64_t)x; break; }
        case 3: { int16_t x; memcpy(&x, v->at, 2); if (x < 0) return fail(FQ_DECLINED_ARGS, "'%s' is negative", key); r = (uint64_t)x; break; }
        case 5: { int32_t x; memcpy(&x, v->at, 4); if (x < 0) return fail(FQ_DECLINED_ARGS, "'%s' is negative", key); r = (uint64_t)x; break; }
        case 11: { int64_t x; memcpy(&x, v->at, 8); if (x < 0) return fail(FQ_DECLINED_ARGS, "'%s' is negative", key); r = (uint64_t)x; break; }
        default: return fail(FQ_DECLINED_ARGS, "'%s' is not an integer", key);
    }
    *out = r;
    return FQ_OK;
}

int fq_gguf_meta_str(const fq_gguf* g, const char* key, char* buf, size_t len) {
    if (!g || !key || !buf || len == 0) return fail(FQ_DECLINED_ARGS, "null pointer");
    const MetaValue* v = find_meta(g, key);
    if (!v || v->type != 8) return fail(FQ_DECLINED_ARGS, "no string metadata key '%s'", key);
    uint64_t n;
    memcpy(&n, v->at, 8);
    const size_t take = n < len - 1 ? (size_t)n : len - 1;
    memcpy(buf, v->at + 8, take);
    buf[take] = 0;
    return FQ_OK;
}

// Even split of `n` rows over `n_ranks` in steps of `align` rows (32 keeps a shard of tile-major weights on tile
// boundaries): rank r owns rows [*row0, *row0 + *rows). The last ranks may own fewer rows or none.
int fq_gguf_shard_rows(size_t n, int n_ranks, int rank, size_t align, size_t* row0, size_t* rows) {
    if (!row0 || !rows || n_ranks < 1 || rank < 0 || rank >= n_ranks || align == 0) return fail(FQ_DECLINED_ARGS, "bad shard arguments");
    const size_t units = (n + align - 1) / align, per = (units + n_ranks - 1) / n_ranks;
    const size_t b = per * rank * align, e = per * (rank + 1) * align;
    *row0 = b < n ? b : n;
    *rows = (e < n ? e : n) - *row0;
    return FQ_OK;
}

int fq_gguf_load_weights(const fq_gguf* g, size_t i, size_t row0, size_t rows, size_t mat0, size_t mats, fq_weights** out) {
    if (!g || !out || i >= g->tensors.size()) return fail(FQ_DECLINED_ARGS, "tensor index out of range");
    *out = nullptr;
    const TensorEntry& t = g->tensors[i];
    if (t.fmt < 0) return fail(FQ_DECLINED_ARGS, "tensor '%s' has ggml type %d, which is not a served quantized format", t.name.c_str(), t.ggml_type);
    if (t.n_dims < 2 || t.dims[3] != 1) return fail(FQ_DECLINED_ARGS, "tensor '%s' is not a matrix or a stack of matrices", t.name.c_str());
    const size_t k = (size_t)t.dims[0], n_all = (size_t)t.dims[1], e_all = (size_t)t.dims[2];
    if (rows == 0) rows = n_all - (row0 < n_all ? row0 : n_all);
    if (mats == 0) mats = e_all - (mat0 < e_all ? mat0 : e_all);
    if (rows == 0 || mats == 0 || row0 + rows > n_all || mat0 + mats > e_all)
        return fail(FQ_DECLINED_ARGS, "rows [%zu, +%zu) of matrices [%zu, +%zu) lie outside tensor '%s' (%zu rows, %zu matrices)", row0, rows, mat0, mats,
                    t.name.c_str(), n_all, e_all);
    Ctx* ctx = context();
    if (!ctx) return FQ_DECLINED_NO_GPU;
    if (!gpu_enabled()) return fail(FQ_DECLINED_GATE, "disabled by FUCINA_GPU=0");
    std::lock_guard<std::recursive_mutex> lock(g_dispatch_lock);
    const size_t nb01 = fq_row_bytes(t.fmt, k), nb02 = nb01 * n_all;
    fq_weights* w = nullptr;
    if (int rc = weights_alloc_layout(ctx, t.fmt, rows, k, mats, true, &w)) return rc;
    // chunks of whole 32-row groups through two page-locked buffers and two raw device buffers
    size_t chunk_rows = kChunkBytes / nb01 / 32 * 32;
    if (chunk_rows == 0) chunk_rows = 32;
    const size_t chunk_bytes = chunk_rows * nb01;
    uint8_t* pin[2] = {(uint8_t*)pin_alloc(chunk_bytes), (uint8_t*)pin_alloc(chunk_bytes)};
    uint8_t* raw[2] = {(uint8_t*)dev_alloc(chunk_bytes), (uint8_t*)dev_alloc(chunk_bytes)};
    cudaEvent_t done[2] = {nullptr, nullptr};
    int rc = FQ_OK;
    if (!pin[0] || !pin[1] || !raw[0] || !raw[1]) rc = fail(FQ_DECLINED_BUDGET, "staging buffers could not be allocated");
    for (int b = 0; b < 2 && rc == FQ_OK; ++b)
        if (cudaEventCreateWithFlags(&done[b], cudaEventDisableTiming) != cudaSuccess) rc = cuda_fail(cudaGetLastError(), "event");
    const uint8_t* src0 = g->map + g->data_start + t.offset;
    size_t piece = 0;
    for (size_t m = 0; m < mats && rc == FQ_OK; ++m) {
        for (size_t r = 0; r < rows && rc == FQ_OK; r += chunk_rows, ++piece) {
            const int b = (int)(piece & 1);
            const size_t nr = rows - r < chunk_rows ? rows - r : chunk_rows;
            if (piece >= 2) cudaEventSynchronize(done[b]);  // the repack that read this pair of buffers has finished
            memcpy(pin[b], src0 + (mat0 + m) * nb02 + (row0 + r) * nb01, nr * nb01);  // faults the mapped pages in
            cudaError_t e = cudaMemcpyAsync(raw[b], pin[b], nr * nb01, cudaMemcpyHostToDevice, ctx->stream);
            g_trace.h2d_bytes += nr * nb01;
            DevWeights view = w->dw;
            view.base = w->dw.base + m * w->dw.mat_stride + (w->dw.tile_rows ? (r / 32) * ((size_t)32 * w->dw.row_stride) : r * w->dw.row_stride);
            view.n = (int)nr;
            view.n_mats = 1;
            if (e == cudaSuccess) e = launch_repack(view, raw[b], nb01, nb01 * nr, true, ctx->stream);
            g_trace.launches++;
            if (e == cudaSuccess) e = cudaEventRecord(done[b], ctx->stream);
            if (e != cudaSuccess) rc = cuda_fail(e, "GGUF tensor upload");
        }
    }
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess && rc == FQ_OK) rc = cuda_fail(cudaGetLastError(), "GGUF tensor upload");
    for (int b = 0; b < 2; ++b) {
        if (done[b]) cudaEventDestroy(done[b]);
        dev_free_idle(raw[b]);
        pin_free(pin[b]);
    }
    if (rc != FQ_OK) {
        fq_weights_free(w);
        return rc;
    }
    *out = w;
    return FQ_OK;
}

int fq_gguf_load_ptqtp_planes(const fq_gguf* g, const char* base, size_t row0, size_t rows, size_t mat0, size_t mats, fq_weights* planes_out[3],
                              int* n_planes) {
    if (!g || !base || !planes_out || !n_planes) return fail(FQ_DECLINED_ARGS, "null pointer");
    *n_planes = 0;
    for (int p = 0; p < 3; ++p) planes_out[p] = nullptr;
    uint64_t version = 0;
    if (find_meta(g, "fucina.ptqtp.version") && fq_gguf_meta_u64(g, "fucina.ptqtp.version", &version) == FQ_OK && version > 1)
        return fail(FQ_DECLINED_ARGS, "fucina.ptqtp.version %llu is newer than this build reads", (unsigned long long)version);
    int idx[3];
    for (int p = 0; p < 3; ++p) idx[p] = fq_gguf_find(g, (std::string(base) + ".ptqtp" + (char)('0' + p)).c_str());
    if (idx[0] < 0) return fail(FQ_DECLINED_ARGS, "no tensor '%s.ptqtp0'", base);
    if (idx[2] >= 0 && idx[1] < 0) return fail(FQ_DECLINED_ARGS, "'%s.ptqtp2' without '%s.ptqtp1': planes fill in order", base, base);
    for (int p = 0; p < 3 && idx[p] >= 0; ++p) {
        const TensorEntry& t = g->tensors[(size_t)idx[p]];
        const TensorEntry& t0 = g->tensors[(size_t)idx[0]];
        int rc = FQ_OK;
        if (t.fmt != FQ_TQ2_0) rc = fail(FQ_DECLINED_ARGS, "'%s' is not a TQ2_0 tensor", t.name.c_str());
        else if (t.dims[0] != t0.dims[0] || t.dims[1] != t0.dims[1] || t.dims[2] != t0.dims[2]) rc = fail(FQ_DECLINED_ARGS, "'%s' and '%s' differ in shape", t.name.c_str(), t0.name.c_str());
        else rc = fq_gguf_load_weights(g, (size_t)idx[p], row0, rows, mat0, mats, &planes_out[p]);
        if (rc != FQ_OK) {
            for (int q = 0; q < p; ++q) fq_weights_free(planes_out[q]), planes_out[q] = nullptr;
            *n_planes = 0;
            return rc;
        }
        *n_planes = p + 1;
    }
    return FQ_OK;
}

}  // extern "C"
