/*
 * fucina_b200 -- C ABI of the B200 (sm_100a) quantized-matmul provider.
 *
 * Drop-in for the GPU-offload seam of fucina's `src/backend/cuda.zig`
 * (selected through `src/backend/gpu.zig:14-21`): the Zig host keeps calling
 * the same provider functions, which forward to these entry points. Each
 * declaration cites the reference interface it replaces (paths are relative
 * to the reference project root).
 *
 * Conventions (same as the reference, backend/cuda.zig:2236-2243):
 *   - RHS weights are row-major [n][k/B] raw GGUF blocks; `nb01` is the byte
 *     stride between weight rows, `nb02` between stacked matrices (experts).
 *   - c[m, n] = a[m, k] . dequant(W)^T, f32, "NT" product.
 *   - return 0  : the GPU ran and the outputs are valid,
 *     return >0 : declined before any side effect (the Zig `false`); nothing
 *                 was written, see fq_last_error(),
 *     return <0 : a CUDA error after submission (a failed accelerator.Work).
 *   - There is no CPU fallback inside the library.
 *   - Callable from any thread; entries serialise on one dispatch lock and
 *     make the device current first (backend/cuda.zig:896, :1776-1779).
 */
#ifndef FUCINA_B200_H
#define FUCINA_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define FQ_API __attribute__((visibility("default")))
#else
#define FQ_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* backend/cuda.zig:1486-1499 `QFormat` (values 0..3 kept). The ternary
 * formats have no CUDA counterpart in the reference (`has_tq2_0_quant =
 * false`, backend/cuda.zig:69-71); their values stay clear of both
 * providers' enums (backend/metal.zig:1275-1280 reuses 3 and 4). */
typedef enum {
    FQ_Q8_0 = 0,
    FQ_Q6_K = 1, /* 256 per block, 210 bytes (src/dtype.zig:141-146); streaming decode (m <= 8, k >= 2048), integer and tensor kernels */
    FQ_Q4_K = 2,
    FQ_Q5_K = 3,
    FQ_TQ2_0 = 16,        /* dtype.zig:215-218, one PTQTP plane */
    FQ_TQ2_0_FOLDED = 17, /* backend/quant/types.zig:177-180, tie-fitted K=2 fold */
    FQ_Q2_0 = 18          /* dtype.zig:78-81, 128-element ternary groups */
} fq_format;

/* Status codes (>0 = declined, <0 = device failure). */
enum {
    FQ_OK = 0,
    FQ_DECLINED_ARGS = 1,    /* shape / alignment / format rule violated */
    FQ_DECLINED_NO_GPU = 2,  /* no device or initialisation failed */
    FQ_DECLINED_BUDGET = 3,  /* resident budget or registry exhausted */
    FQ_DECLINED_GATE = 4,    /* disabled by FUCINA_GPU=0 */
    FQ_DECLINED_BUSY = 5,    /* all async slots in flight */
    FQ_ERR_CUDA = -1,
    FQ_ERR_TIMEOUT = -2,     /* a bounded device-side wait gave up */
    FQ_ERR_CAPACITY = -3     /* the routing sent more rows to a GPU than its exchange arena holds */
};

/* backend/ops.zig:89-107 `GatedOp`: g = source(up) * activation(gate) (ops.zig:150-190).
 * swiglu up * gate*sigmoid(gate); geglu up * gelu_tanh(gate) (Gemma); swiglu_clamp10 clamp(up, +-10) *
 * silu(min(gate, 10)) (DeepSeek V4); glu up * sigmoid(gate); situ 25 tanh(up/25) * 4 tanh(gate/4) sigmoid(gate). */
enum { FQ_GATED_SWIGLU = 0, FQ_GATED_GEGLU = 1, FQ_GATED_SWIGLU_CLAMP10 = 2, FQ_GATED_GLU = 3, FQ_GATED_SITU = 4 };

/* backend/cuda.zig:1503-1508 `QMMTile`: one 32-row output tile of one expert's group of panel rows, with the
 * reference's field meaning (filled at llm/gemma/moe.zig:773-787, read at backend/cuda/kernels.cu:322-327): the
 * tile covers panel rows [base_row + 32 * tile_m, base_row + min(m, 32 * tile_m + 32)). */
typedef struct {
    int32_t expert;   /* which matrix of the stack */
    int32_t base_row; /* first panel row of the expert's group */
    int32_t m;        /* rows of the whole group */
    int32_t tile_m;   /* index of this tile inside the group */
} fq_qmm_tile;

/* ---- provider lifetime (backend/cuda.zig:412-508 `context`/`initOnce`,
 *      :510 `deviceName`) ---- */
FQ_API int fq_init(int device); /* idempotent; device <0 = current/0 */
FQ_API int fq_device_count(void);
FQ_API const char* fq_device_name(void);
FQ_API int fq_sm_count(void);
FQ_API int fq_last_error(char* buf, size_t len);
/* The library's compute stream as a cudaStream_t, for callers that own
 * device buffers and want to order their own work after ours. */
FQ_API void* fq_stream(void);
FQ_API int fq_synchronize(void);

/* ---- block geometry (dtype.zig:230-239 size asserts) ---- */
FQ_API size_t fq_block_elems(int fmt);
FQ_API size_t fq_block_bytes(int fmt);
FQ_API size_t fq_row_bytes(int fmt, size_t k); /* GGUF bytes of one weight row */

/* ---- weight residency (backend/cuda.zig:1733 `allocResidentBytes`, :1780
 *      `freeResidentBytes`, :1550-1611 `residentDevPtr`) ----
 * fq_alloc_resident returns page-locked host bytes the loader fills; the
 * device copy (in the gpu_formats layout) is made on first use.
 * rhs pointers passed with cacheable=1 are adopted by source address: the
 * caller promises they stay mapped and unchanged for the process lifetime
 * (exec/quant_matmul.zig:22-36). fq_evict_resident drops one adopted range. */
FQ_API void* fq_alloc_resident(size_t len);
FQ_API void fq_free_resident(const void* p);
FQ_API int fq_evict_resident(const void* host_ptr);
FQ_API size_t fq_resident_bytes(void);
/* Page-lock a range of the caller's tensor storage once, for its lifetime (backend/cuda.zig:1047-1082
 * `ensureHostRegistered`): activations inside it are copied by DMA without a staging copy, and decode-sized
 * results inside it are written by the kernel in place. fq_host_unregister takes the range's start address and
 * waits for the library stream first. Ranges already covered are accepted again at no cost. */
FQ_API int fq_host_register(void* host_ptr, size_t len);
FQ_API int fq_host_unregister(void* host_ptr);
FQ_API int fq_set_vram_budget(size_t bytes); /* FUCINA_GPU_VRAM_BUDGET twin; test seam of backend/cuda.zig:3639 */

/* ---- gpu_formats: explicit device-resident weights ----
 * Upload raw GGUF blocks once, repack to the device layout, and get a handle
 * usable by the *_dev entries. `n_mats` stacked matrices (experts) of n rows.
 * The reference reads raw blocks in place (backend/cuda.zig:2051); this is
 * the new packing stage. */
typedef struct fq_weights fq_weights;
FQ_API int fq_weights_upload(int fmt, const void* host_blocks, size_t nb01, size_t nb02, size_t n, size_t k,
                      size_t n_mats, fq_weights** out);
FQ_API int fq_weights_from_device(int fmt, const void* dev_blocks, size_t nb01, size_t nb02, size_t n, size_t k,
                           size_t n_mats, fq_weights** out); /* raw blocks already in HBM */
/* Rows [row0, row0 + rows) of every stacked matrix as weights of their own: no copy, the parent must outlive the
 * view, both are freed with fq_weights_free. The two halves of a fused gate_up expert tensor
 * [E][2 * out_pe][hidden] (llm/gemma/moe.zig:717) and the column shards of a resident matrix are such views. (New.) */
FQ_API int fq_weights_view(const fq_weights* w, size_t row0, size_t rows, fq_weights** out);
FQ_API void fq_weights_free(fq_weights* w);
FQ_API size_t fq_weights_device_bytes(const fq_weights* w);
/* inverse of the repack, for round-trip checks: device layout -> GGUF bytes (host) */
FQ_API int fq_weights_download_gguf(const fq_weights* w, void* host_blocks, size_t len);
/* dequantise rows [row0, row0+rows) of matrix `mat` to f32 on the host or the
 * device (kernels.cu:72-159 `dequant_*`; values are bit-identical to the CPU
 * decoders q4_k.zig:1954-1972, q5_k.zig:1154-1167, q8k.zig:95-114,
 * cold.zig:651-670, :289-301, ternary.zig:850-876). */
FQ_API int fq_dequantize_rows(const fq_weights* w, size_t mat, size_t row0, size_t rows, float* host_out);
FQ_API int fq_dequantize_rows_dev(const fq_weights* w, size_t mat, size_t row0, size_t rows, float* dev_out);
/* Weight encoders on the device (q8k.zig:49-69, q4_k.zig:1977-2048,
 * q5_k.zig:1172-1257, ternary.zig:79-144, cold.zig:309-332): f32 rows in HBM
 * -> raw GGUF blocks in HBM, byte-identical to the CPU encoders. */
FQ_API int fq_quantize_rows_dev(int fmt, const float* dev_src, size_t n, size_t k, void* dev_blocks);

/* ---- streaming attention forward (the step on the other side of the linear layers in a decode token) ----
 * The contract of attnFwdHostImpl / attnPrefillF16 (backend/cuda.zig:2601-2736) and of the kernels
 * fucina_attn_fwd_{f16,f32} (backend/cuda/kernels.cu:574-681): q [q_seq][heads][d] f32, k and v [kv_seq][kv_heads][d]
 * f16 (kv_is_f16 != 0) or f32, out [q_seq][heads][d] f32, optional stats [heads][q_seq][2] = {row max, sum exp},
 * kv_head_for_head [heads]; query row i sits at absolute position source_offset + i; causal (keys up to that
 * position, the last `window` of them when window > 0) or bidirectional; scores are scaled by `scale`.
 * d <= 256 and a multiple of 8 (f16) or 4 (f32); heads <= 512; device pointers 16-byte aligned; every map entry must
 * name a kv head (the host form checks it, the device form cannot). Online softmax in f32; the key range of a row is
 * cut into splits merged by a second kernel, in a fixed order; the K and V rows of a step are staged in shared memory
 * once for all the heads that share the kv head. Device-buffer and blocking host-buffer forms. */
FQ_API int fq_attn_fwd_dev(const float* q_dev, const void* k_dev, const void* v_dev, int kv_is_f16, float* out_dev, float* stats_dev,
                           const int32_t* kv_head_for_head_dev, size_t q_seq, size_t kv_seq, size_t heads, size_t kv_heads, size_t d,
                           size_t source_offset, float scale, size_t window, int causal, void* stream);
FQ_API int fq_attn_fwd(const float* q, const void* k, const void* v, int kv_is_f16, float* out, float* stats,
                       const int32_t* kv_head_for_head, size_t q_seq, size_t kv_seq, size_t heads, size_t kv_heads, size_t d,
                       size_t source_offset, float scale, size_t window, int causal);

/* ---- GGUF file -> device-resident weights (new on the GPU side). The reference parses GGUF in src/gguf.zig
 *      (:214-452: header, metadata, tensor table, data section aligned to general.alignment) and makes quantized
 *      tensors GPU-resident in src/weights.zig:2621-2816; here the mapped blocks of a row / expert range go straight
 *      to the repacked device layouts through two page-locked staging buffers, so file reads, copies and repack
 *      kernels overlap. Opening and querying need no GPU. ---- */
typedef struct fq_gguf fq_gguf;
typedef struct {
    const char* name;   /* valid until fq_gguf_close */
    int ggml_type;      /* ggml_type id as stored */
    int fmt;            /* FQ_* format id, or -1 when the type is not a served quantized format */
    int n_dims;         /* 1..4; dims[0] is the row length (k), dims[1] the rows, dims[2] the matrices (experts) */
    uint64_t dims[4];
    uint64_t offset;    /* from the start of the file */
    uint64_t bytes;     /* 0 when this reader cannot size the type */
} fq_gguf_tensor;
FQ_API int fq_gguf_open(const char* path, fq_gguf** out);
FQ_API void fq_gguf_close(fq_gguf* g);
FQ_API size_t fq_gguf_tensor_count(const fq_gguf* g);
FQ_API int fq_gguf_tensor_at(const fq_gguf* g, size_t i, fq_gguf_tensor* out);
FQ_API int fq_gguf_find(const fq_gguf* g, const char* name);        /* index, or -1 (src/gguf.zig:546 maybeGet) */
FQ_API const void* fq_gguf_tensor_data(const fq_gguf* g, size_t i); /* the tensor's bytes inside the mapping */
FQ_API int fq_gguf_meta_u64(const fq_gguf* g, const char* key, uint64_t* out);            /* src/gguf.zig:511 getInt */
FQ_API int fq_gguf_meta_str(const fq_gguf* g, const char* key, char* buf, size_t len);    /* NUL-terminated, cut to len - 1 */
/* Rows [row0, row0 + rows) of matrices [mat0, mat0 + mats) of tensor i as resident weights (rows == 0 / mats == 0:
 * to the end): the shard a rank owns of a column-sharded linear or of an expert stack. */
FQ_API int fq_gguf_load_weights(const fq_gguf* g, size_t i, size_t row0, size_t rows, size_t mat0, size_t mats, fq_weights** out);
/* The trit planes `<base>.ptqtp0/1/2` of a PTQTP model (src/ptqtp_gguf.zig:95-98): every plane present, in order. */
FQ_API int fq_gguf_load_ptqtp_planes(const fq_gguf* g, const char* base, size_t row0, size_t rows, size_t mat0, size_t mats,
                                     fq_weights* planes_out[3], int* n_planes);
/* Even split of n rows over n_ranks in steps of `align` rows (32 keeps tile-major shards on tile boundaries). */
FQ_API int fq_gguf_shard_rows(size_t n, int n_ranks, int rank, size_t align, size_t* row0, size_t* rows);

/* ---- dense quantized matmul, host buffers ----
 * backend/cuda.zig:2398-2435 `gemmQuantNt` (blocking), :2441-2492
 * `gemmQuantNtSharedABatch`. `rhs_len` is the byte length of the rhs range. */
FQ_API int fq_gemm_quant_nt(int fmt, const void* rhs, size_t rhs_len, int cacheable, size_t nb01, const float* a,
                     float* c, size_t m, size_t n, size_t k);
FQ_API int fq_gemm_quant_nt_shared_a_batch(int fmt, const void* rhs, size_t rhs_len, int cacheable, size_t nb01,
                                    size_t nb02, const float* a, float* c, size_t batch, size_t m, size_t n,
                                    size_t k);

/* ---- eager async submit + completion token ----
 * backend/cuda.zig:2001-2175 `gemmQuantNtAsync`; the token is the C twin of
 * accelerator.Work's vtable {finish, device_ptr, destroy}
 * (accelerator.zig:22-133, backend/cuda.zig:1145-1218). `a_dep` chains a
 * pending producer's device output without a host round trip
 * (backend/cuda.zig:1224-1230 `pendingDeviceInput`); pass NULL to read `a`.
 * c_host belongs to the token from the submit until fq_work_finish returns: decode-sized results are copied
 * out behind the product (on a transfer stream of their own), so they may land there before finish is called. */
typedef struct fq_work fq_work;
FQ_API int fq_gemm_quant_nt_async(int fmt, const void* rhs, size_t rhs_len, int cacheable, size_t nb01, size_t nb02,
                           const float* a, fq_work* a_dep, float* c_host, size_t batch, size_t m, size_t n,
                           size_t k, fq_work** out_work);
FQ_API int fq_work_finish(fq_work* w, int copy_to_host); /* 0 ok; <0 failed */
FQ_API uintptr_t fq_work_device_ptr(fq_work* w);
FQ_API void fq_work_destroy(fq_work* w);

/* ---- dense quantized matmul, device buffers (activation chaining and
 *      kernel-only timing); a_dev/c_dev are f32 in HBM. Runs on `stream`
 *      (NULL = the library stream). mode: see FQ_MODE_*. ---- */
enum {
    FQ_MODE_AUTO = 0,   /* m <= 16: integer decode kernel; larger: tensor cores */
    FQ_MODE_INT8 = 1,   /* activations quantised like the CPU kernels (native.zig:427-490), dp4a dots */
    FQ_MODE_TENSOR = 2  /* weights and activations rounded to bf16, tcgen05 MMA, f32 accumulate */
};
FQ_API int fq_gemm_quant_nt_dev(const fq_weights* w, size_t mat, const float* a_dev, float* c_dev, size_t m, int mode,
                         void* stream);
/* The fused neighbours of the CPU path: a row operation applied to the activations on their way into the
 * quantiser, so the [m, k] intermediate is never written (src/exec/quant_matmul.zig:480-757,
 * src/exec/row_ops.zig:39-137; the reference has them on the CPU only).
 *   FQ_PRE_RMS_NORM_MUL  a_dev [m][k], pre_w_dev [k]: (x * scale) * weight with
 *                        scale = 1 / sqrt(sum(x^2) / k + eps)                            (row_ops.zig:96-106)
 *   FQ_PRE_SPLIT_SWIGLU  a_dev [m][2k] = gate | up per row: (up * gate) * (1 / (1 + exp(-gate)))  (row_ops.zig:711-728)
 * k must be a multiple of 256. Decode shapes (m <= 4, the formats and sizes of the copy-engine kernel) run the
 * operation inside that kernel's prologue; every other shape runs fq_act_prologue_dev into scratch and then the
 * plain product. Both forms use one arithmetic order, so the results are bit-identical to
 * fq_act_prologue_dev followed by fq_gemm_quant_nt_dev. The sum of squares adds 256-element block sums in block
 * order (the reference's scalar loop adds element by element: scale agrees to f32 round-off, not bit for bit). */
enum { FQ_PRE_NONE = 0, FQ_PRE_RMS_NORM_MUL = 1, FQ_PRE_SPLIT_SWIGLU = 2 };
FQ_API int fq_gemm_quant_nt_pre_dev(const fq_weights* w, size_t mat, int pre_op, const float* a_dev, const float* pre_w_dev,
                                    float eps, float* c_dev, size_t m, int mode, void* stream);
/* The row operation alone: out_dev [m][k] f32. */
FQ_API int fq_act_prologue_dev(int pre_op, const float* a_dev, const float* pre_w_dev, float eps, float* out_dev, size_t m,
                               size_t k, void* stream);
/* Allocation-free small-batch product. No counterpart in the reference (its
 * provider grows device buffers on demand, backend/cuda.zig:873-890). For
 * hosts that must not allocate device memory once they are serving -- VRAM
 * fully budgeted at start-up, a decode loop that cannot afford the device-wide
 * stall of a cudaMalloc, memory owned by an external pool. Same result as
 * fq_gemm_quant_nt_dev in FQ_MODE_INT8 for m <= 16, but the int8 activation
 * records live in a fixed 512 KiB array inside the library image instead of
 * the caching allocator. Two bounds, both checked before anything is launched
 * or written: the records of the m rows must fit the array (a record is about
 * 1.1 * k bytes, 1.4 * k for Q8_0), and the kernel keeps the rows -- padded to
 * 1, 2, 4, 8 or 16 -- in shared memory, so pad(m) records must fit 227 KiB
 * (fq_small_batch_max_rows gives the largest m for a format and k); otherwise
 * the call is declined. Every GPU that loads the library holds the
 * array until exit. All calls share it, so calls that overlap on the GPU
 * race; order them on one stream. The first call on a device resolves the
 * array's address: make it before any stream capture. fq_init must have been
 * called; this entry creates nothing. */
FQ_API int fq_gemm_quant_nt_dev_noalloc(const fq_weights* w, size_t mat, const float* a_dev, float* c_dev, size_t m,
                                        void* stream);
/* Largest number of activation rows one launch of the small-batch integer
 * kernel takes for this format and k: 16, 8, 4, 2, 1, or 0 when not even one
 * row's int8 records fit a CTA's shared memory. Larger batches are served in
 * chunks of this size by fq_gemm_quant_nt_dev; needs no device. (New.) */
FQ_API int fq_small_batch_max_rows(int fmt, size_t k);
/* K planes of one PTQTP weight summed per element in plane order
 * (weights.zig:204-300 `linearSeqPtqtpFused`). */
FQ_API int fq_gemm_ptqtp_dev(const fq_weights* const* planes, int n_planes, const float* a_dev, float* c_dev, size_t m,
                      void* stream);
/* Activation quantisers on the device (q8k.zig:268-313 Q8_K, :49-69 Q8_0);
 * outputs are the reference block structs (dtype.zig:148-152, :83-86). */
FQ_API int fq_quantize_acts_q8_k_dev(const float* a_dev, size_t m, size_t k, void* dev_blocks);
FQ_API int fq_quantize_acts_q8_0_dev(const float* a_dev, size_t m, size_t k, void* dev_blocks);

/* ---- CUDA graphs over the library stream (new; the reference is eager and
 *      pays 4-17 us of submit time per call, docs/GPU-OFFLOAD.md:376-390) ----
 * Between fq_capture_begin and fq_capture_end only *_dev entries that neither
 * allocate nor synchronise may be called from the capturing thread: the dense
 * decode shapes with m <= 4 on the library stream (stream = NULL). The
 * captured step replays with one launch. */
typedef struct fq_graph fq_graph;
FQ_API int fq_capture_begin(void);
FQ_API int fq_capture_end(fq_graph** out);
FQ_API int fq_graph_launch(fq_graph* g);
FQ_API void fq_graph_destroy(fq_graph* g);

/* ---- grouped MoE GEMM over a CPU-built tile table ----
 * backend/cuda.zig:2181 `qmoe_lock`, :2221 `qmoeStage`, :2244-2333
 * `gemmQGroupedNt`. The stage's host panels are owned by the library. */
FQ_API void fq_qmoe_lock(void);
FQ_API void fq_qmoe_unlock(void);
FQ_API int fq_qmoe_stage(size_t in_bytes, size_t out_bytes, float** in, float** out);
FQ_API int fq_gemm_q_grouped_nt(int fmt, const void* rhs, size_t rhs_len, int cacheable, size_t nb01, size_t nb02,
                         size_t n_out, size_t k, const fq_qmm_tile* tiles, size_t n_tiles);
/* Tiles of one expert over adjoining rows are merged into runs (the expert's weights stream once per run). Runs of
 * 17 rows or more multiply on the tensor cores over bf16-rounded operands (the reference's grouped kernel rounds
 * its operands to f16, backend/cuda/kernels.cu:340-379), shorter runs keep the CPU kernels' int8 arithmetic.
 * Test seam in the spirit of setQuantMmaForTest (backend/cuda.zig:2563): -1 by run length, 0 integer arm only,
 * 1 tensor cores for every run the format allows. */
FQ_API void fq_set_grouped_tensor_for_test(int mode);

/* ---- fused, device-resident MoE expert layer (new) ----
 * Argument-for-argument twin of ExecContext.moeExpertFfn / moeExpertFfnBatch
 * (exec/moe.zig:1135-1298, :1865-2088): x [seq, hidden], selected/weights
 * [seq*top_k] row-major per token, out [seq, hidden]; gate/up are
 * [E][out_pe][hidden], down is [E][hidden][out_pe]. gated_op is one of FQ_GATED_*
 * (backend/ops.zig:150-190). gate and up share one format; down may come in another (Gemma pairs Q4_K
 * gate/up with Q8_0 down, llm/gemma/moe.zig:696-901); a fused [2 * out_pe] gate_up tensor is passed as the two
 * row views fq_weights_view makes of it. Host-buffer and device-buffer forms. */
FQ_API int fq_moe_layer(const fq_weights* gate, const fq_weights* up, const fq_weights* down, const float* x, size_t seq,
                 size_t top_k, const int64_t* selected, const float* weights, int gated_op, float* out);
FQ_API int fq_moe_layer_dev(const fq_weights* gate, const fq_weights* up, const fq_weights* down, const float* x_dev,
                     size_t seq, size_t top_k, const int32_t* selected_dev, const float* weights_dev,
                     int gated_op, float* out_dev, void* stream);
/* The same layer over multi-plane ternary (PTQTP) experts (exec/moe.zig:51-78 `MoePtqtpRhs`, :591-631
 * `moePtqtpTileDotRange`): arrays of n_planes (1..3) TQ2_0 expert stacks per projection; every product is the
 * plane dots summed per element in plane order, as the dense fused PTQTP linear sums them. Integer arm. */
FQ_API int fq_moe_layer_ptqtp_dev(const fq_weights* const* gate_planes, const fq_weights* const* up_planes,
                                  const fq_weights* const* down_planes, int n_planes, const float* x_dev, size_t seq, size_t top_k,
                                  const int32_t* selected_dev, const float* weights_dev, int gated_op, float* out_dev, void* stream);
/* Expert-parallel shard of the same layer (the reference is single-device, backend/cuda.zig:439,
 * so this has no counterpart there). gate/up/down hold experts [expert_base, expert_base + E_local)
 * of the full layer; `selected_dev` carries GLOBAL expert ids. Pairs routed to other shards are
 * skipped, and partial_dev [seq, hidden] receives, per token, the slot-ordered weighted sum over the
 * pairs this shard serves (all zero when it serves none). Summing the shards' partial outputs gives
 * the layer output; a reduce-scatter does that when tokens are sharded too. */
FQ_API int fq_moe_layer_ep_dev(const fq_weights* gate, const fq_weights* up, const fq_weights* down, const float* x_dev,
                        size_t seq, size_t top_k, const int32_t* selected_dev, const float* weights_dev,
                        int expert_base, int gated_op, float* partial_dev, void* stream);
/* ---- several GPUs of one node, one process per GPU (new: the reference takes device 0 only,
 *      backend/cuda.zig:439) ----
 * Rank 0 makes a 128-byte rendezvous id (fq_tp_unique_id); the host carries it to the other processes; every
 * rank then calls fq_tp_init (collective). It creates an NCCL communicator (libnccl.so.2 is loaded at run
 * time) and an exchange arena of `arena_bytes` (0 = 1 GiB) per rank whose CUDA IPC handle every peer opens,
 * so kernels store into other GPUs' memory over NVLink. fq_tp_peer_access tells whether that mapping
 * succeeded; without it only the NCCL forms run. fq_init must name this process's GPU first. */
#define FQ_TP_ID_BYTES 128
FQ_API int fq_tp_unique_id(void* id128);
FQ_API int fq_tp_init(int n_ranks, int rank, const void* id128, size_t arena_bytes);
FQ_API int fq_tp_shutdown(void);
FQ_API int fq_tp_ranks(void);       /* 0 before fq_tp_init */
FQ_API int fq_tp_rank(void);        /* -1 before fq_tp_init */
FQ_API int fq_tp_peer_access(void); /* 1 when every peer's arena is mapped */
/* Column-sharded (tensor-parallel) product: `w_shard` holds this rank's contiguous slice of the weight rows
 * (every rank the same number), the activations are replicated, and one all-gather assembles
 * c_dev [rank][m][n_shard] on every rank. No reduction crosses ranks: each element is computed exactly as on
 * one GPU (fq_gemm_quant_nt_dev semantics for a_dev, mode and stream). Collective. */
FQ_API int fq_gemm_quant_nt_tp(const fq_weights* w_shard, const float* a_dev, float* c_dev, size_t m, int mode, void* stream);
/* Expert-parallel MoE layer. gate/up/down hold experts [rank * E_local, (rank + 1) * E_local) of the layer;
 * x_dev [seq, hidden] are THIS rank's tokens, selected_dev carries global expert ids, out_dev [seq, hidden].
 * Collective: every rank calls it once per layer (seq may differ between ranks in the fused form).
 * flags: 0 = the fused form when the peers' arenas are mapped (token rows are stored straight into the
 * owning GPU's panel by the gather kernel, the down product's epilogue stores result rows straight into the
 * home GPU's return panel, flags with bounded waits order the phases; bf16 tensor-core arithmetic for every
 * batch size, bit-identical to the one-GPU tensor arm), else the baseline; FQ_EP_NCCL = the baseline (NCCL
 * all-gather of tokens and routing, partial sums per rank, NCCL reduce-scatter; needs the same seq on every
 * rank); FQ_EP_FUSED = the fused form or a decline. A routing that sends a rank more rows than its arena
 * holds ends the layer with FQ_ERR_CAPACITY at the next synchronisation (size the arena for
 * n_ranks * seq * top_k rows of 2 * hidden + 8 bytes, plus seq * top_k * hidden * 4). */
enum { FQ_EP_AUTO = 0, FQ_EP_NCCL = 1, FQ_EP_FUSED = 2 };
FQ_API int fq_moe_layer_ep(const fq_weights* gate, const fq_weights* up, const fq_weights* down, const float* x_dev, size_t seq,
                           size_t top_k, const int32_t* selected_dev, const float* weights_dev, int gated_op, float* out_dev,
                           int flags, void* stream);
/* Test seam: `world` ranks of the fused form emulated on ONE GPU (arrays of `world` pointers; every rank
 * has `seq` tokens). The phases run in lockstep on the library stream, so every wait finds its flags posted
 * by kernels that have already finished. Runs `layers` layers back to back over the same arenas and waits.
 * layers < 0: one layer in which the last rank's count publication is dropped, so every rank's bounded wait
 * runs out (about a second each) and the call returns FQ_ERR_TIMEOUT with the context still usable. */
FQ_API int fq_ep_emulate_for_test(int world, const fq_weights* const* gate, const fq_weights* const* up,
                                  const fq_weights* const* down, const float* const* x_dev, size_t seq, size_t top_k,
                                  const int32_t* const* selected_dev, const float* const* weights_dev, float* const* out_dev,
                                  size_t arena_bytes, int layers);
/* exec/topk.zig:21-86 `routerTopK` on the device: logits [seq, E] -> selected/weights [seq, top_k]. */
FQ_API int fq_router_topk_dev(const float* logits_dev, size_t seq, size_t n_expert, size_t top_k, int normalize,
                       int32_t* selected_dev, float* weights_dev, void* stream);

/* ---- gates (backend/cuda.zig:2494-2554) and test seams (:2537-2571) ---- */
FQ_API int fq_should_use_gpu_dense_quant(int fmt, uint64_t total_work);
FQ_API int fq_should_use_gpu_dense_quant_packed(int fmt, uint64_t total_work);
FQ_API int fq_should_use_gpu_quant_decode(int fmt, size_t m, size_t n, size_t k);
FQ_API int fq_should_use_gpu_qmoe(uint64_t total_work);
FQ_API int fq_qmoe_fill_acceptable(size_t rows, size_t n_tiles);
FQ_API void fq_set_min_work_qmoe_for_test(uint64_t v);
FQ_API void fq_set_decode_for_test(int enabled);
/* Arm selection of the fused MoE layer, in the spirit of setQuantMmaForTest (backend/cuda.zig:2563):
 * -1 automatic (tensor cores once a batch averages >= 20 rows per expert, else the int8 decode
 * arm), 0 always the int8 arm, 1 the tensor-core arm whenever the format has one. */
FQ_API void fq_set_moe_tensor_for_test(int mode);
/* The integer arm of fq_moe_layer_dev with its two intermediates copied out in pair order
 * (row p = token p / top_k, slot p % top_k): g_pairs_dev [seq*top_k, out_pe] receives
 * swiglu(gate . qx, up . qx) (exec/moe.zig:890-920 before the requantisation of g) and
 * down_pairs_dev [seq*top_k, hidden] the unweighted down rows; either may be NULL. Lets a test hold
 * each stage to the f32 tolerance on its own. Library stream. */
FQ_API int fq_moe_layer_stages_for_test(const fq_weights* gate, const fq_weights* up, const fq_weights* down, const float* x_dev,
                                        size_t seq, size_t top_k, const int32_t* selected_dev, const float* weights_dev,
                                        float* g_pairs_dev, float* down_pairs_dev, float* out_dev);
/* Grouped integer launches put one table entry per grid row and stride over tables longer than the
 * grid's y limit (65535); this lowers the limit so a small case walks the striding path (<= 0 restores it). */
FQ_API void fq_set_group_grid_limit_for_test(int limit);
/* Failure-detection seam (no counterpart in the reference): every device-side wait in this library is
 * bounded and reports FQ_ERR_TIMEOUT through a status word instead of hanging. This launches one warp that
 * polls `limit` times (1..2^20) a barrier nothing completes, gives up the same way and returns normally; the
 * next fq_synchronize or blocking entry then returns FQ_ERR_TIMEOUT once, and the context stays usable. */
FQ_API int fq_selftest_bounded_wait(unsigned limit);

/* ---- trace counters (backend/cuda.zig:191-317) ---- */
FQ_API int fq_trace_enabled(void);
FQ_API void fq_trace_reset(void);
FQ_API void fq_trace_dump(void);
/* counter snapshot: calls, kernel launches, h2d bytes, d2h bytes, resident hits, resident adopts, gate pass, gate fail */
FQ_API void fq_trace_counters(uint64_t out[8]);
/* Device time of the decode kernel (CUDA events around each launch while
 * enabled), the per-kind timing of backend/cuda.zig:231-257 taken on the
 * device instead of the host clock. fq_trace_kernel_times waits for the
 * recorded launches, returns their summed duration and count, and clears. */
FQ_API void fq_trace_kernel_timing(int enable);
FQ_API int fq_trace_kernel_times(double* total_ms, uint64_t* launches);

#ifdef __cplusplus
}
#endif
#endif /* FUCINA_B200_H */
