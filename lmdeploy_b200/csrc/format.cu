// int4 layout conversions (deploy-time helpers), written as gathers: every thread produces
// whole destination words from the closed form of the permutation, so there are no atomics
// and `dst` needs no zero fill.  Behaviour (argument order, layouts, values) follows
// src/turbomind/kernels/gemm_s_f16/format.cu:61-142 of lmdeploy v0.0.9; `m` = output features.
#include "common.cuh"
#include "tm_b200.h"

namespace tmb {
namespace {

// AWQ packing: nibble position p of a word holds column order[p] = {0,2,4,6,1,3,5,7}
// (lmdeploy/pytorch/modules/linear.py:87), so column c sits at position (c & 1) * 4 + (c >> 1).
__device__ __forceinline__ int awq_pos_of_col(int c)
{
    return ((c & 1) << 2) | (c >> 1);
}
__device__ __forceinline__ int awq_col_of_pos(int p)
{
    return ((p & 3) << 1) | (p >> 2);
}

__device__ __forceinline__ uint32_t read_awq(const uint32_t* __restrict__ src, size_t row, int words_per_row, int col)
{
    const uint32_t w = __ldg(src + row * words_per_row + (col >> 3));
    return (w >> (4 * awq_pos_of_col(col & 7))) & 0xfu;
}

// dst word index -> [k/32][m/32][lane][w]; see the closed form in common.cuh (unpack_s4_minus_zero)
__global__ void reformat_s4_k_m8_kernel(uint32_t* __restrict__ dst, const uint32_t* __restrict__ src, int m, int k)
{
    const size_t total = (size_t)k * m / 8;
    const int    mt    = m / 32;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int    w    = i & 3;
        const int    lane = (i >> 2) & 31;
        const size_t tile = i >> 7;
        const int    n32  = tile % mt;
        const size_t k32  = tile / mt;
        uint32_t     out  = 0;
#pragma unroll
        for (int nib = 0; nib < 8; ++nib) {
            const size_t kk = k32 * 32 + (w >> 1) * 16 + ((nib >> 1) & 1) * 8 + (lane & 3) * 2 + (nib >> 2);
            const int    nn = n32 * 32 + (w & 1) * 16 + (nib & 1) * 8 + (lane >> 2);
            out |= read_awq(src, kk, m / 8, nn) << (4 * nib);
        }
        dst[i] = out;
    }
}

// zeros (AWQ packed) -> workspace half[k/g * m] = 64 + z, and Q = {64 + z, scale}
__global__ void merge_q_kernel(__half2* __restrict__ Q,
                               __half* __restrict__ workspace,
                               const __half* __restrict__ scales,
                               const uint32_t* __restrict__ qzeros,
                               size_t n_words)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_words; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t w = __ldg(qzeros + i);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const uint32_t nib  = (w >> (4 * awq_pos_of_col(c))) & 0xfu;
            const __half   z    = __ushort_as_half((unsigned short)(0x5400u | (nib << 4)));  // 64 + nib
            const size_t   e    = i * 8 + c;
            if (workspace) workspace[e] = z;
            Q[e] = __halves2half2(z, scales[e]);
        }
    }
}

__global__ void
transpose_qk_kernel(uint32_t* __restrict__ dst, const uint32_t* __restrict__ src, int m, int k, int size_per_head)
{
    const size_t total = (size_t)k * m / 8;
    const int    wpr   = m / 8;
    const int    half  = size_per_head / 2;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / wpr;
        const int    cw  = i % wpr;
        uint32_t     out = 0;
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            const int f    = cw * 8 + awq_col_of_pos(p);
            const int head = f / size_per_head;
            const int fi   = f % size_per_head;
            const int sf   = head * size_per_head + (fi & 1) * half + (fi >> 1);  // new[2j+h] = old[half*h + j]
            out |= read_awq(src, row, wpr, sf) << (4 * p);
        }
        dst[i] = out;
    }
}

// src [2, k, m/8] (w1 then w3) -> dst [k, 2m/8], features interleaved w1_0, w3_0, w1_1, ...
__global__ void fuse_w1_w3_kernel(uint32_t* __restrict__ dst, const uint32_t* __restrict__ src, int m, int k)
{
    const size_t total = (size_t)k * m / 4;
    const int    wpr   = m / 4;  // destination words per row
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / wpr;
        const int    cw  = i % wpr;
        uint32_t     out = 0;
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            const int f     = cw * 8 + awq_col_of_pos(p);
            const int which = f & 1;
            out |= read_awq(src + (size_t)which * k * (m / 8), row, m / 8, f >> 1) << (4 * p);
        }
        dst[i] = out;
    }
}

__global__ void dequantize_s4_kernel(uint4* __restrict__ dst, const uint32_t* __restrict__ src, size_t count)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t w = __ldg(src + i);
        // halves in nibble order [0,4,1,5,2,6,3,7] (kernels/gemm_s_f16/common.h:70-84), plain 0..15
        __half2 h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            h[j] = __halves2half2(__ushort2half_rn((unsigned short)((w >> (4 * j)) & 0xfu)),
                                  __ushort2half_rn((unsigned short)((w >> (4 * j + 16)) & 0xfu)));
        }
        dst[i] = *reinterpret_cast<uint4*>(h);
    }
}

inline int grid_for(size_t n, int block)
{
    size_t g = (n + block - 1) / block;
    if (g > 4096) g = 4096;  // grid-stride loops: a few thousand blocks fill any device
    if (g < 1) g = 1;
    return (int)g;
}

inline bool aligned16(const void* p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

inline int launch_status()
{
    return cudaGetLastError() == cudaSuccess ? TM_OK : TM_ERR_CUDA;
}

}  // namespace
}  // namespace tmb

using namespace tmb;

extern "C" int tm_reformat_s4_k_m8(uint32_t* dst, const uint32_t* src, int m, int k, void* stream)
{
    if (!dst || !src || dst == src) return TM_ERR_INVALID_ARG;
    if (m <= 0 || k <= 0 || m % 32 || k % 32) return TM_ERR_UNSUPPORTED;
    const size_t total = (size_t)k * m / 8;
    reformat_s4_k_m8_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(dst, src, m, k);
    return launch_status();
}

extern "C" int tm_convert_s4_k_m8(uint32_t*       A_dst,
                                  void*           Q_dst,
                                  void*           workspace,
                                  const uint32_t* A_src,
                                  const void*     scales,
                                  const uint32_t* qzeros,
                                  int             m,
                                  int             k,
                                  int             group_size,
                                  void*           stream)
{
    if (!A_dst || !Q_dst || !A_src || !scales || !qzeros || A_dst == A_src) return TM_ERR_INVALID_ARG;
    if (m <= 0 || k <= 0 || group_size <= 0 || m % 32 || k % 32 || k % group_size) return TM_ERR_UNSUPPORTED;
    const size_t n_words = (size_t)(k / group_size) * m / 8;
    merge_q_kernel<<<grid_for(n_words, 256), 256, 0, (cudaStream_t)stream>>>(
        (__half2*)Q_dst, (__half*)workspace, (const __half*)scales, qzeros, n_words);
    if (cudaGetLastError() != cudaSuccess) return TM_ERR_CUDA;
    return tm_reformat_s4_k_m8(A_dst, A_src, m, k, stream);
}

extern "C" int
tm_transpose_qk_s4_k_m8_hf(uint32_t* dst, const uint32_t* src, int m, int k, int size_per_head, void* stream)
{
    if (!dst || !src || dst == src) return TM_ERR_INVALID_ARG;
    if (m <= 0 || k <= 0 || size_per_head <= 0 || size_per_head % 16 || m % size_per_head) return TM_ERR_UNSUPPORTED;
    const size_t total = (size_t)k * m / 8;
    transpose_qk_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(dst, src, m, k, size_per_head);
    return launch_status();
}

extern "C" int tm_fuse_w1_w3_s4_k_m8(uint32_t* dst, const uint32_t* src, int m, int k, void* stream)
{
    if (!dst || !src || dst == src) return TM_ERR_INVALID_ARG;
    if (m <= 0 || k <= 0 || m % 8) return TM_ERR_UNSUPPORTED;
    const size_t total = (size_t)k * m / 4;
    fuse_w1_w3_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(dst, src, m, k);
    return launch_status();
}

extern "C" int tm_dequantize_s4(void* dst, const uint32_t* src, size_t count, void* stream)
{
    if (count == 0) return TM_OK;
    if (!dst || !src) return TM_ERR_INVALID_ARG;
    if (!aligned16(dst)) return TM_ERR_INVALID_ARG;
    dequantize_s4_kernel<<<grid_for(count, 256), 256, 0, (cudaStream_t)stream>>>((uint4*)dst, src, count);
    return launch_status();
}
