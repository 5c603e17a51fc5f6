// Prefill-shaped quantized GEMM on the 5th-generation tensor cores (tcgen05,
// accumulators in TMEM). Placeholder translation unit: until the kernel lands
// every shape is declined and callers use the integer decode kernel.
#include "internal.h"
#include "runtime.h"

namespace fq {

int gemm_tensor_dev(Ctx*, const DevWeights&, int, const float*, float*, size_t, size_t, cudaStream_t) {
    return fail(FQ_DECLINED_ARGS, "tensor-core path not built");
}

}  // namespace fq
