// Internal entry to the tcgen05 GEMM for callers inside the library that need an epilogue the
// public paras_b200_gemm does not offer (attention backward).
#pragma once

#include "common.cuh"

namespace pb {

struct GemmExtra {
    int epilogue;           // 0: none (only k_skip is used)
                            // 3: C = exp(acc*scale - row_stat[row]), causally masked (col <= row % Lq)
                            // 4: C = prob[row, col] * (acc - row_stat[row]) * scale
    const float* row_stat;  // [batch * M]
    const void* prob;       // [batch * M, prob_ld] in the GEMM's dtype (epilogue 4)
    int64_t prob_ld;
    int Lq;
    int causal;
    float scale;
    int k_skip;             // with causal: skip K steps whose operand slice is entirely masked;
                            // 1: A rows are queries, K runs over keys; 2: A rows are keys, K over stacked queries
    int tile_skip;          // with causal, epilogues 3 and 4: 128 x 256 output tiles all of whose keys follow
                            // all of their queries are not computed and NOT WRITTEN; only for Lk <= Lq, and
                            // only when every reader of C skips the same parts (k_skip does)
};

// The CTA-pair kernel (gemm_tc2.cu): 256 x 256 tiles on two CTAs of a cluster, for the large projections.
bool gemm_tc2_eligible(const Gpu* g, const paras_gemm_args* a);
int gemm_tc2_run(Gpu* g, const paras_gemm_args* a, cudaStream_t s);

// The decode-step kernel (gemm_skinny.cu): at most 128 rows of A against a weight that is read once.
bool gemm_skinny_eligible(const Gpu* g, const paras_gemm_args* a);
int gemm_skinny_run(Gpu* g, const paras_gemm_args* a, cudaStream_t s);

// paras_b200_gemm with `ex` (may be null); A must be [M, K] rows for epilogues 3 and 4.
int gemm_run(const paras_gemm_args* a, const GemmExtra* ex);

}  // namespace pb
