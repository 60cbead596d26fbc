// Internal interfaces shared by the SDPA kernels and their dispatcher.
#pragma once

#include "common.cuh"

namespace pb {

// Split-KV partial results: o_part[split][row][D] (unnormalised, relative to m),
// ml_part[split][row] = {running max of scaled scores, running sum of exp}.
// row = (b*Hq + h)*Lq + qi.
struct SplitWorkspace {
    float* o_part = nullptr;
    float2* ml_part = nullptr;
    int splits = 1;
};

// Layout: ml_part first (8-byte entries), then o_part at the next multiple of 16 bytes.  With
// the base 16-byte aligned both parts are aligned for their access width (float2 / float)
// whatever rows, D and splits are -- odd D with an odd number of splits included.
inline size_t split_ml_bytes(int64_t rows, int splits) {
    return (size_t(splits) * size_t(rows) * sizeof(float2) + 15u) & ~size_t(15);
}

inline size_t split_workspace_bytes(int64_t rows, int D, int splits) {
    if (splits <= 1) return 0;
    return split_ml_bytes(rows, splits) + size_t(splits) * size_t(rows) * size_t(D) * sizeof(float);
}

inline SplitWorkspace carve_workspace(void* base, int64_t rows, int D, int splits) {
    SplitWorkspace w;
    w.splits = splits;
    (void)D;
    if (splits > 1) {
        w.ml_part = static_cast<float2*>(base);
        w.o_part = reinterpret_cast<float*>(static_cast<char*>(base) + split_ml_bytes(rows, splits));
    }
    return w;
}

// Generic CUDA-core flash kernel: any dtype, D <= 256, masks, any strides.
int sdpa_simt_launch(Gpu* g, const paras_sdpa_args& a, float scale, const SplitWorkspace& ws,
                     cudaStream_t s);
int sdpa_simt_pick_splits(const Gpu* g, const paras_sdpa_args& a);

// Merges split-KV partials into out (and lse).
int sdpa_combine_launch(Gpu* g, const paras_sdpa_args& a, const SplitWorkspace& ws,
                        cudaStream_t s);

// tcgen05/TMEM/TMA kernel: bf16/f16, D == 128 or 64.  `rope` (optional, D == 128, no mask tensor):
// the queries are rotated in the kernel's prologue with these tables ([rows, 128] in the tensors'
// dtype, row = pos0 + query index).
struct RopeTables {
    const void* cos;
    const void* sin;
    int64_t pos0;
};
bool sdpa_tc_supported(const Gpu* g, const paras_sdpa_args& a, const char** why);
// `variant` (optional) receives the name of the route taken: "tcgen05", "tcgen05_split" (key range in pieces),
// "tcgen05_packed" (the heads of a GQA group in one item), "tcgen05_packed_split", "tcgen05_rope"
int sdpa_tc_launch(Gpu* g, const paras_sdpa_args& a, float scale, cudaStream_t s, const RopeTables* rope = nullptr,
                   const char** variant = nullptr);
int sdpa_mask_is_causal(Gpu* g, int gpu, const void* mask, int mask_kind, int dtype, int64_t row_stride, int Lq, int Lk,
                        float scale, cudaStream_t s, int* result);
// scratch of the split-key route (few query blocks, many keys); 0 when the route is not taken
size_t sdpa_tc_workspace_bytes(const Gpu* g, const paras_sdpa_args& a);

// Tensor-core split-KV decode kernel: 16-bit, D == 128, short Lq, no mask tensor.
bool sdpa_decode_supported(const Gpu* g, const paras_sdpa_args& a, const char** why);
int sdpa_decode_pick_splits(const Gpu* g, const paras_sdpa_args& a);
int sdpa_decode_launch(Gpu* g, const paras_sdpa_args& a, float scale, const SplitWorkspace& ws,
                       cudaStream_t s);

// Dropout on the weights / a given dropout mask / the weights as an output (sdpa_weights.cu).
bool sdpa_wants_weights(const paras_sdpa_args& a);
int sdpa_weights_launch(Gpu* g, const paras_sdpa_args& a, float scale, cudaStream_t s);

// Philox2x32 with 10 rounds, key schedule and counter layout of csrc/ops/random_ops.cpp:27-47.
__device__ __forceinline__ uint32_t philox2x32_r0(uint64_t seed, uint64_t sequence, uint64_t idx) {
    uint32_t c0 = uint32_t(idx);
    uint32_t c1 = uint32_t(sequence + (idx >> 32));
    uint32_t k0 = uint32_t(seed);
#pragma unroll
    for (int i = 0; i < 10; ++i) {
        const uint64_t prod = uint64_t(0xD256D193u) * c0;
        const uint32_t n0 = uint32_t(prod >> 32) ^ k0 ^ c1;
        c1 = uint32_t(prod);
        c0 = n0;
        k0 += 0x9E3779B9u;
    }
    return c0;
}

// The softmax scale as the kernels use it (rounded to the tensors' dtype with PARAS_SDPA_REF_SCALE).
float effective_scale(const paras_sdpa_args& a);

// Fused tcgen05 attention backward (sdpa_bwd_tc.cu): 16-bit, D == 128 or 64, dense tensors.
bool sdpa_bwd_tc_supported(const Gpu* g, const paras_sdpa_bwd_args& a);
size_t sdpa_bwd_tc_scratch_bytes(const paras_sdpa_bwd_args& a);
int sdpa_bwd_tc_launch(Gpu* g, const paras_sdpa_bwd_args& a, float* scratch, cudaStream_t s);

}  // namespace pb
