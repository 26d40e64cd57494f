// RMSNorm and fused residual-add + RMSNorm of the decoder loop: one CTA per token row, the row
// kept in registers between the sum-of-squares pass and the scaling pass (one read, one write),
// 128-bit accesses.  Replaces invokeRootMeanSquareNorm (src/turbomind/models/llama/
// llama_kernels.cu:14-79) and invokeFusedAddBiasResidualRMSNorm (src/turbomind/models/llama/
// llama_decoder_kernels.cu:104-160) of lmdeploy v0.0.9, with the same arithmetic: fp32 math,
// the residual stored as fp16, the sum of squares taken before that rounding, the
// normalisation applied to the stored value.
#include "common.cuh"
#include "mmha.h"

namespace tmb {
namespace {

constexpr int kNormThreads = 256;
constexpr int kMaxVec      = 8;  // 8 x 8 halves x 256 threads = rows up to 16384

__device__ __forceinline__ float block_sum(float v, float* red)
{
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = lane < (kNormThreads / 32) ? red[lane] : 0.f;
#pragma unroll
    for (int m = 4; m >= 1; m >>= 1) t += __shfl_xor_sync(0xffffffffu, t, m);
    return __shfl_sync(0xffffffffu, t, 0);
}

template<bool RESIDUAL>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(__half* residual, __half* in_out, const __half* in, const __half* bias, const __half* scale, float eps, int n)
{
    __shared__ float red[kNormThreads / 32];
    pdl_wait();  // the rows come from the kernel before this one
    pdl_launch_dependents();
    const size_t     row  = (size_t)blockIdx.x * n;
    const int        nvec = n / 8;
    uint4            keep[kMaxVec];
    float            ss = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
        const int v = threadIdx.x + i * kNormThreads;
        if (v < nvec) {
            if (RESIDUAL) {
                uint4          r = reinterpret_cast<const uint4*>(residual + row)[v];
                const uint4    x = reinterpret_cast<const uint4*>(in_out + row)[v];
                uint4          b = make_uint4(0, 0, 0, 0);
                if (bias) b = reinterpret_cast<const uint4*>(bias)[v];
                __half2*       rh = reinterpret_cast<__half2*>(&r);
                const __half2* xh = reinterpret_cast<const __half2*>(&x);
                const __half2* bh = reinterpret_cast<const __half2*>(&b);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 a = __half22float2(rh[e]), c = __half22float2(xh[e]), d = __half22float2(bh[e]);
                    const float2 s = make_float2(a.x + c.x + d.x, a.y + c.y + d.y);
                    ss += s.x * s.x + s.y * s.y;
                    rh[e] = __float22half2_rn(s);
                }
                reinterpret_cast<uint4*>(residual + row)[v] = r;
                keep[i]                                     = r;
            }
            else {
                const uint4    x  = reinterpret_cast<const uint4*>(in + row)[v];
                const __half2* xh = reinterpret_cast<const __half2*>(&x);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 a = __half22float2(xh[e]);
                    ss += a.x * a.x + a.y * a.y;
                }
                keep[i] = x;
            }
        }
    }
    const float total = block_sum(ss, red);
    const float inv   = rsqrtf(total / (float)n + eps);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
        const int v = threadIdx.x + i * kNormThreads;
        if (v < nvec) {
            const uint4    s  = reinterpret_cast<const uint4*>(scale)[v];
            const __half2* sh = reinterpret_cast<const __half2*>(&s);
            uint4          o  = keep[i];
            __half2*       oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 a = __half22float2(oh[e]), w = __half22float2(sh[e]);
                // llama_decoder_kernels.cu:58-61: a * s * factor ; llama_kernels.cu:37-38: a * factor * s
                oh[e] = RESIDUAL ? __float22half2_rn(make_float2(a.x * w.x * inv, a.y * w.y * inv)) :
                                   __float22half2_rn(make_float2(a.x * inv * w.x, a.y * inv * w.y));
            }
            reinterpret_cast<uint4*>(in_out + row)[v] = o;
        }
    }
}

}  // namespace

cudaError_t rmsnorm_launch(__half* out, const __half* in, const __half* scale, float eps, int m, int n, cudaStream_t st, bool pdl)
{
    return launch_kernel(rmsnorm_kernel<false>, dim3(m), dim3(kNormThreads), 0, st, pdl, nullptr, out, in, nullptr, scale, eps, n);
}

cudaError_t add_residual_rmsnorm_launch(
    __half* residual, __half* in_out, const __half* bias, const __half* scale, float eps, int m, int n, cudaStream_t st, bool pdl)
{
    return launch_kernel(rmsnorm_kernel<true>, dim3(m), dim3(kNormThreads), 0, st, pdl, residual, in_out, nullptr, bias, scale, eps, n);
}

}  // namespace tmb
