// Multi-GPU context shared by multi.cu (communicator, peer-mapped arena, column-sharded product) and ep.cu
// (expert-parallel MoE layer). One process per GPU; the reference is single-device (src/backend/cuda.zig:439).
#pragma once
#include "internal.h"
#include "runtime.h"

namespace fq {

struct TpCtx {
    int world = 0;
    int rank = -1;
    void* comm = nullptr;              // ncclComm_t
    uint8_t* arena = nullptr;          // this rank's exchange arena (cudaMalloc, exported to the peers)
    size_t arena_bytes = 0;
    uint8_t* peer[kMaxPeers] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};  // peer[r]: rank r's arena as mapped here
    bool peer_ok = false;              // every peer's arena is mapped (same node, peer access granted)
    int epoch = 0;                     // expert-parallel layers served so far (flag values)
};

// The context fq_tp_init created, or nullptr.
TpCtx* tp_context();

// NCCL wrappers on the communicator of tp_context(); FQ_OK or a negative status with fq_last_error set.
int tp_all_gather(const void* send, void* recv, size_t bytes_per_rank, cudaStream_t st);
int tp_reduce_scatter_f32(const float* send, float* recv, size_t count_per_rank, cudaStream_t st);

// moe.cu: one expert shard of the layer (experts [expert_base, expert_base + E_local) of the full layer, global ids
// in selected_dev, other shards' pairs skipped): partial sums per token.
int moe_layer_shard_dev(Ctx* ctx, const DevWeights& gate, const DevWeights& up, const DevWeights& down, const float* x_dev, int seq,
                        int top_k, const int* selected_dev, const float* weights_dev, int expert_base, float* partial_dev, cudaStream_t st,
                        int gated_op = 0);

// ep.cu: print and clear the per-phase device times gathered under FUCINA_B200_EP_TRACE
void ep_trace_dump(int rank);

}  // namespace fq
