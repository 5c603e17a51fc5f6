// Launchers shared between the translation units of libfucina_b200.so.
#pragma once
#include <cstdlib>
#include "common.cuh"

namespace fq {

// formats.cu
cudaError_t launch_repack(const DevWeights& w, const uint8_t* gguf_dev, size_t nb01, size_t nb02, bool to_device,
                          cudaStream_t st);
cudaError_t launch_dequant_rows(const DevWeights& w, int mat, int row0, int rows, float* out, cudaStream_t st);
// row r of the output is quantised from source row (src_rows ? src_rows[r] / src_div : r)
cudaError_t launch_quantize_acts_layout(const float* a, const int* src_rows, int src_div, int m, int k, int fmt, uint8_t* out,
                                        cudaStream_t st);
cudaError_t launch_quantize_acts_struct(const float* a, int m, int k, bool q8k, uint8_t* out, cudaStream_t st);
cudaError_t launch_quantize_weights(int fmt, const float* src, size_t n, size_t k, uint8_t* dst, cudaStream_t st);

// gemv.cu -- decode kernels over int8 activations in the acts.cuh layout.
//
// Plain form: `acts` holds m <= 16 rows of act_sizes(fmt,k).row bytes; all n
// rows of matrix `mat` are multiplied; c is [m][ldc]. accumulate != 0 adds to
// c instead of storing (PTQTP plane sums).
//
// Grouped form (table != nullptr): blockIdx.y walks a device-built table of
// row groups; group g multiplies activation rows [row0, row0+m) -- and writes
// the same rows of c -- with matrix `mat` of the expert stack. Entries at or
// beyond *n_desc are skipped, so the host can launch an upper bound.
//
// Gated form (w2.base != nullptr): row j of `w` (gate) and row j of `w2` (up)
// are dotted with the same activations and c receives
// up * (gate * 1/(1+exp(-gate))) (reference backend/ops.zig:150-190, swiglu).
struct TcTile;
struct GroupDesc {
    int mat;
    int row0;
    int m;
    int pad;
};
struct GemvArgs {
    DevWeights w;
    DevWeights w2;
    int mat;
    const uint8_t* acts;
    float* c;
    int m;
    int ldc;
    int accumulate;
    const GroupDesc* table;
    const int* n_desc;
    int max_desc;
    int gated_op = 0;  // FQ_GATED_* of the gated form
};
cudaError_t launch_gemv(const GemvArgs& a, int sm_count, cudaStream_t st);
size_t gemv_max_rows();  // largest m one launch (or one table entry) handles
// m padded to the row counts the kernel is instantiated for (1, 2, 4, 8, 16), and the largest such count whose
// activation records fit a CTA's shared memory for this format and K (0: not even one row fits)
void set_gemv_grid_y_limit(int limit);  // test seam: cap gridDim.y of grouped launches (<= 0 restores 65535)
int gemv_padded_rows(size_t m);
int gemv_rows_that_fit(int fmt, size_t k);

// Launch with programmatic stream serialisation allowed (see pdl_wait_then_release in common.cuh): the grid may be
// scheduled while the previous kernel of the stream drains. FUCINA_B200_NO_PDL switches it off.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    static const bool no_pdl = getenv("FUCINA_B200_NO_PDL") != nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = no_pdl ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// formats.cu -- natural-order activation records (actquant.cuh)
cudaError_t launch_quantize_acts_natural(const float* a, int m, int k, int q8k, uint8_t* out, cudaStream_t st);

// decode_rows.cu -- row-per-lane decode kernel with TMA-staged weights.
struct RowsArgs {
    DevWeights w;
    int mat;
    const float* a_f32;       // [m][k] f32 activations, quantised in the kernel prologue (fused form)
    const uint8_t* acts_nat;  // or m pre-quantised natural records
    float* c;                 // [m][ldc]
    int m;
    int ldc;
    int slab;    // 256-weight units per row per pipeline step
    int stages;  // pipeline depth per warp
    int* status; // device-visible status word (FQ_ERR_TIMEOUT on a wait that gave up)
    int use_tmap; // weights arrive by 2-D tensor copies (one per warp step) instead of per-lane bulk copies
    int skip_compute; // diagnosis only: stream the weights, skip the arithmetic
    int l2_stream;    // weight copies carry an evict-first L2 hint (tile-major form)
    int rows_per_cta; // 0: rows split evenly over the grid; > 0: CTA b serves rows [b*rows_per_cta, +rows_per_cta);
                      // < 0: whole 32-row storage tiles split evenly over the grid
    int split_n;      // 0, or the rows of ONE matrix when w stacks several that share the activations: weight row r
                      // of token b lands at c[((r / split_n) * m + b) * split_n + r % split_n] (the [batch][m][n] layout)
    PreArgs pre;      // activation prologue applied while quantising (fused form only): rms_norm_mul or split_swiglu
    int accumulate;   // add to c instead of overwriting it (TQ2_0 form: the planes of a PTQTP product)
};
// Grouped expert form of the row-per-lane kernel (MoE decode): a device-built table of (expert, run of
// <= 8 activation rows) entries over a row-major expert stack; the f32 activation rows are quantised
// by the kernel itself. With w2 the gate (w) and up (w2) matrices are multiplied together and the
// SwiGLU product is stored.
struct ExpertArgs {
    DevWeights w, w2;
    const float* src;       // f32 rows: token rows (src_index set) or one row per sorted pair position
    const int* src_index;   // sorted position -> pair id; the token row is pair / top_k
    int top_k;
    float* out;             // [pairs][n]
    const GroupDesc* table;
    const int* n_desc;
    int max_desc;
    int tiles_per_item;     // 1, 2, 4 or 8 tiles of 32 rows per work item; 8 / tiles_per_item warps split K
    int stages;
    int* status;
    int gated_op;           // FQ_GATED_* of the gate/up pair (w2 set)
    int chain;              // launch with programmatic stream serialisation (short tables)
};
// one warp runs a bounded wait on a barrier nothing completes and reports through the status word
cudaError_t launch_bounded_wait_probe(int* status, unsigned limit, cudaStream_t st);
int expert_rows_max_group();
bool expert_rows_eligible(const DevWeights& w, const DevWeights* w2, int group_rows);
cudaError_t launch_expert_rows(const DevWeights& w, const DevWeights* w2, const float* src, const int* src_index, int top_k, float* out,
                               const GroupDesc* table, const int* n_desc, int max_desc, int group_rows, int sm_count, int* status,
                               cudaStream_t st, int gated_op = 0);
// true when the shape is one the kernel serves (format, K, m, shared memory)
bool decode_rows_eligible(const DevWeights& w, size_t m);
// bytes of natural-record scratch the non-fused form needs (0 for the fused form)
size_t decode_rows_scratch_bytes(const DevWeights& w, size_t m);
// `pre` (optional): an activation prologue fused into the kernel's quantiser; only where decode_rows_fuses_prologue
cudaError_t launch_decode_rows(const DevWeights& w, int mat, const float* a_dev, uint8_t* scratch, float* c, int m, int ldc,
                               int sm_count, int* status, cudaStream_t st, int split_n = 0, const PreArgs* pre = nullptr, int accumulate = 0);
bool decode_rows_fuses_prologue(const DevWeights& w, size_t m);
// formats.cu -- the stand-alone form of the activation prologues: out[m][k] (split_swiglu reads 2k values per row)
cudaError_t launch_act_prologue(const PreArgs& pre, const float* a, float* out, int m, int k, cudaStream_t st);

// gemm_tc.cu -- tcgen05 prefill GEMM. One output tile of the grouped (MoE) form: weight rows
// [rt*128, +128) of expert matrix `mat` times the consecutive activation rows [tok0, tok0+ntok).
struct TcTile {
    int mat, rt, tok0, ntok;
};
// Optional multi-GPU hooks of the grouped tensor-core GEMM (expert parallelism over peer memory).
//  * wait_flags: the token-tile producer does not issue its first load before wait_flags[i] >= wait_value for
//    every i < n_wait (other ranks' dispatch kernels post these after writing their token rows into this GPU's
//    panel). The wait is bounded; a timeout aborts the CTA and records FQ_ERR_TIMEOUT.
//  * row_meta: the f32 epilogue does not write c[row][col] but dst_base[meta.x][meta.y * ldc + col]: each output
//    row goes straight to the panel of the rank that owns its token (plain peer stores over NVLink).
constexpr int kMaxPeers = 8;
struct TcPeer {
    const int* wait_flags = nullptr;
    int n_wait = 0;
    int wait_value = 0;
    const int2* row_meta = nullptr;
    float* dst_base[kMaxPeers] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    //  * signal: the last CTA of the grid to finish (counted in *done_counter, which the caller zeroes) stores
    //    signal_value into signal_flag[i], i < n_signal, after a system-wide fence: "my result rows are in your panel".
    int* done_counter = nullptr;
    int* signal_flag[kMaxPeers] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    int n_signal = 0;
    int signal_value = 0;
};
cudaError_t launch_add_f32(float* c, const float* t, size_t n, cudaStream_t st);
cudaError_t launch_f32_to_bf16(const float* src, void* dst, size_t n, cudaStream_t st);

}  // namespace fq
