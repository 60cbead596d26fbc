// Placeholder translation unit: the tensor-core decode kernel is not built yet, so the
// dispatcher routes short-query problems to the CUDA-core split-KV kernel.
#include "sdpa_common.cuh"

namespace pb {

bool sdpa_decode_supported(const Gpu*, const paras_sdpa_args&, const char** why) {
    *why = "decode kernel not built";
    return false;
}
int sdpa_decode_pick_splits(const Gpu*, const paras_sdpa_args&) { return 1; }
int sdpa_decode_launch(Gpu*, const paras_sdpa_args&, float, const SplitWorkspace&, cudaStream_t) {
    return fail(PARAS_E_UNSUPPORTED, "paras sdpa: decode kernel not built");
}

}  // namespace pb
