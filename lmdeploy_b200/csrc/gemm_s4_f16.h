// Internal interface between the C ABI (api.cu) and the W4A16 GEMM kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace tmb {

// ---- small-token (HBM-bound) kernel -----------------------------------------------------
struct GemmSmallParams {
    __half*              C;
    const unsigned char* A;  // runtime int4 layout, [K/32][N/32][512 B]
    const unsigned char* X;  // half [T, K]
    const unsigned char* Q;  // half2 [K/128, N]
    float*               workspace;
    int*                 counters;
    unsigned*            status;
    int                  N, T, K;
    int                  fused_silu;
    // filled in by gemm_small_launch from the plan
    int units_per_cta, total_units, slots_per_chunk, n_col_tiles, stages;
};

struct GemmSmallPlan {
    int    nt;             // 8-token MMA tiles per pass (1, 2 or 4)
    int    t_chunks;       // passes over the weight (grid.y)
    int    n_col_tiles;    // 512-column tiles
    int    total_units;    // 64x512 weight units
    int    units_per_cta;
    int    ctas;
    int    slots_per_chunk;  // split-K scratch slots per token chunk (= ctas + n_col_tiles)
    int    stages;
    int    cols_tiles;     // 1 or 2: the column-owner kernel runs instead, on strips of that many 32-column tiles (up to 8 tokens,
                           // at least one strip per SM); 0: the split-K kernel
    size_t smem_bytes;
    size_t workspace_floats;
    size_t counter_ints;
};

size_t        gemm_small_smem_bytes(int nt);
GemmSmallPlan gemm_small_plan(int N, int T, int K, int sm_count, int max_smem, int cols_variant = 1);
cudaError_t   gemm_small_prepare(int max_smem);
cudaError_t   gemm_small_launch(const GemmSmallPlan& plan, GemmSmallParams p, cudaStream_t st, bool pdl = false);

// Residual add + RMSNorm folded into two consecutive tensor-core GEMMs of the decode step (decode driver only).
// Producer side (o_proj, w2): the reducers of the output tiles add the residual, store it, write
// half((residual + y) * norm_weight) as the output and add up every token's sum of squares in 2^-20 fixed point
// (integer atomics: the order of the additions cannot change the result).
// Consumer side (qkv, w13): the rows of the accumulator are scaled by rsqrt(ssq[t] * 2^-20 * inv_n + eps) before the
// output is rounded, which completes the normalisation of its input.
struct GemmNormFusion {
    __half*                   residual    = nullptr;  // [T][N], producer
    const __half*             norm_weight = nullptr;  // [N], producer
    unsigned long long*       ssq_out     = nullptr;  // [T], producer
    const unsigned long long* ssq_in      = nullptr;  // [T], consumer
    float                     inv_n       = 0.f;      // 1 / (length of the normalised row), consumer
    float                     eps         = 0.f;
};

// ---- tensor-core (tcgen05) kernel for more than 16 tokens ---------------------------------
struct GemmTcParams {
    __half*              C;
    const unsigned char* A;
    const unsigned char* X;
    const unsigned char* Q;
    float*               workspace;
    int*                 counters;
    unsigned*            status;
    int                  N, T, K;
    int                  fused_silu;
    // filled in by gemm_tc_launch from the plan
    int units_per_cta, total_units, slots_per_chunk, n_col_tiles, token_tile, x_stages, a_stages, acc_stride, k_split, parts_per_tile;
    long long max_wait_cycles;  // bound of the wait for the partners of a split tile; 0 = the default
    GemmNormFusion norm;        // all null: a plain GEMM
};

struct GemmTcPlan {
    int    token_tile;     // UMMA N: tokens per pass, multiple of 16, <= 128
    int    t_chunks;       // passes over the weight (grid.y), 128 tokens each
    int    n_col_tiles;    // 256-feature tiles
    int    total_units;    // 128x256 weight units
    int    units_per_cta;
    int    parts_per_tile;  // CTAs per column tile (each with up to units_per_cta groups of it); 0 = the flat unit list cut evenly
    int    ctas;
    int    slots_per_chunk;
    size_t smem_bytes;
    size_t workspace_floats;
    size_t counter_ints;
};

size_t      gemm_tc_smem_bytes(int token_tile);
GemmTcPlan  gemm_tc_plan(int N, int T, int K, int sm_count);
// true when every output tile of the plan is reduced by reduce_share (the only place that applies GemmNormFusion)
bool        gemm_tc_all_tiles_split(const GemmTcPlan& plan, int K);
cudaError_t gemm_tc_prepare(int max_smem);
cudaError_t gemm_tc_launch(const GemmTcPlan& plan, GemmTcParams p, cudaStream_t st, bool pdl = false);

}  // namespace tmb
