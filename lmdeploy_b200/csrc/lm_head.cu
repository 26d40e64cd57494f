// lm-head of the decode step: logits[b, v] (fp32) = sum_k x[b, k] * w[v, k], fp16 operands, for one rank's slice of the
// vocabulary.  Replaces the cuBLAS call of LlamaV2::postDecodeEmbedding (src/turbomind/models/llama/LlamaV2.cc:312-372;
// there cublas_wrapper_->Gemm(CUBLAS_OP_T, CUBLAS_OP_N, vocab / tp, batch, hidden, ...) with fp32 output).
//
// HBM-bound at decode batch sizes (262 MB of fp16 weight for 32000 x 4096, read once), and a plain dense contraction, so
// it runs on the tcgen05 tensor core with both operands in shared memory:
//   warp 0   one lane feeds a ring of stages with TMA: a [128 vocabulary rows x 64 k] box of the weight and the
//            [token tile x 64 k] box of the activations, 128-byte swizzle (no multicast: every CTA loads for itself)
//   warp 1   allocates TMEM; one lane issues four M128 x N(token tile) x K16 MMAs per stage, accumulator in TMEM,
//            tcgen05.commit hands the stage back to the loader and, at the end, the accumulator to
//   warps 2-5  which read their 32 TMEM lanes (vocabulary rows) and store fp32 logits, 32 consecutive columns per
//            warp and token (128-byte stores).
// One CTA per 128-row tile, whole K range: no partial sums meet anywhere.  Two CTAs are co-resident per SM up to a token
// tile of 128 (250 tiles of the Llama-2 vocabulary then all run at once instead of in two waves).
// Every wait is bounded: a barrier that does not complete sets a status bit and the CTA drains and leaves.
#include "common.cuh"
#include "handle.h"
#include "tm_b200.h"

#include <cuda.h>
#include <cuda_fp16.h>

namespace tmb {
namespace {

constexpr int kLmTileV   = 128;  // vocabulary rows per CTA (UMMA M)
constexpr int kLmKBlock  = 64;   // k per stage: 128 bytes per row, the swizzle span
constexpr int kLmThreads = 6 * 32;
constexpr int kLmMaxStages = 8;

struct LmBars {
    uint64_t full[kLmMaxStages], empty[kLmMaxStages];
    uint64_t acc_full;
    uint32_t tmem_base;
    int      dead;
};

struct LmHeadParams {
    float*    logits;  // [tokens][ld]
    int       ld;
    int       tokens, vocab, hidden;
    int       token_tile;  // UMMA N: tokens rounded up to 16
    int       stages;
    int       tmem_cols;
    unsigned* status;
    long long max_wait_cycles;
};

__device__ __forceinline__ uint64_t lm_desc(uint32_t smem_addr)
{
    // K-major operand, 128-byte swizzle: 8-row groups 1024 B apart, descriptor version 1
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46)
           | ((uint64_t)2 << 61);
}

__device__ __forceinline__ void lm_umma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a),
        "l"(desc_b),
        "r"(idesc),
        "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void lm_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void lm_tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(map)),
                 "r"(x),
                 "r"(y),
                 "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void lm_tmem_ld16(uint32_t taddr, float (&v)[16])
{
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__global__ void __launch_bounds__(kLmThreads, 2)
lm_head_kernel(LmHeadParams p, const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map)
{
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t raw  = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;  // operand tiles sit on 1024-byte boundaries (swizzle = f(address))
    unsigned char* sm   = smem_dyn + (base - raw);

    const int      NT      = p.token_tile;
    const uint32_t w_bytes = kLmTileV * 128;
    const uint32_t x_bytes = (uint32_t)NT * 128;
    const uint32_t stage_b = w_bytes + x_bytes;
    const int      ST      = p.stages;
    LmBars*        bars    = reinterpret_cast<LmBars*>(sm + (size_t)ST * stage_b);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int v0  = blockIdx.x * kLmTileV;
    const int nkb = p.hidden / kLmKBlock;

    if (tid == 0) {
        for (int s = 0; s < kLmMaxStages; ++s) {
            mbar_init(&bars->full[s], 1);
            mbar_init(&bars->empty[s], 1);
        }
        mbar_init(&bars->acc_full, 1);
        bars->dead = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                     "r"(p.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0) {
        // ===================================================================================== loader
        if (lane == 0) {
            // the weight is written by no kernel: its first boxes start before the kernel ahead of this one is known to
            // be complete; the activations follow after that wait, on the same barriers
            const int pre = min(ST, nkb);
            for (int kb = 0; kb < pre; ++kb) {
                mbar_arrive_expect_tx(&bars->full[kb], stage_b);
                lm_tma_2d(base + kb * stage_b, &w_map, kb * kLmKBlock, v0, &bars->full[kb]);
            }
            pdl_wait();
            pdl_launch_dependents();
            for (int kb = 0; kb < pre; ++kb) lm_tma_2d(base + kb * stage_b + w_bytes, &x_map, kb * kLmKBlock, 0, &bars->full[kb]);
            for (int kb = pre; kb < nkb; ++kb) {
                const int s = kb % ST;
                if (!mbar_wait(&bars->empty[s], ((kb / ST) - 1) & 1, p.max_wait_cycles)) {
                    atomicOr(p.status, kStatusGemmPipeWait);
                    *(volatile int*)&bars->dead = 1;
                    break;
                }
                mbar_arrive_expect_tx(&bars->full[s], stage_b);
                lm_tma_2d(base + s * stage_b, &w_map, kb * kLmKBlock, v0, &bars->full[s]);
                lm_tma_2d(base + s * stage_b + w_bytes, &x_map, kb * kLmKBlock, 0, &bars->full[s]);
            }
        }
        else {
            pdl_wait();
            pdl_launch_dependents();
        }
    }
    else if (warp == 1) {
        // ===================================================================================== MMA issuer
        pdl_wait();
        pdl_launch_dependents();
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(kLmTileV >> 4) << 24);
            bool           ok    = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int s = kb % ST;
                if (!mbar_wait(&bars->full[s], (kb / ST) & 1, p.max_wait_cycles)) {
                    atomicOr(p.status, kStatusGemmPipeWait);
                    *(volatile int*)&bars->dead = 1;
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = lm_desc(base + s * stage_b), db = lm_desc(base + s * stage_b + w_bytes);
#pragma unroll
                for (int j = 0; j < 4; ++j) lm_umma_ss(tmem, da + (uint64_t)(2 * j), db + (uint64_t)(2 * j), idesc, (kb | j) ? 1u : 0u);
                lm_commit(&bars->empty[s]);  // the stage is free once these MMAs have read it
            }
            lm_commit(&bars->acc_full);  // arrives when everything issued so far is complete (also on the give-up path)
        }
    }
    else {
        // ===================================================================================== logits out
        pdl_wait();
        pdl_launch_dependents();
        const int  q    = warp & 3;  // the TMEM lane quarter this warp may read
        const int  v    = v0 + q * 32 + lane;
        int        okw  = 1;
        if (lane == 0) okw = mbar_wait(&bars->acc_full, 0, p.max_wait_cycles) ? 1 : 0;
        okw = __shfl_sync(0xffffffffu, okw, 0);
        if (!okw && lane == 0) atomicOr(p.status, kStatusGemmTmemWait);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (okw && *(volatile int*)&bars->dead == 0) {
            for (int c0 = 0; c0 < NT; c0 += 16) {
                if (c0 >= p.tokens) break;
                float acc[16];
                lm_tmem_ld16(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, acc);
                if (v < p.vocab) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        if (c0 + i < p.tokens) p.logits[(size_t)(c0 + i) * p.ld + v] = acc[i];
                    }
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(p.tmem_cols) : "memory");
    }
}

using PFN_encodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                     const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

PFN_encodeTiled lm_lookup_encode_tiled()
{
    void*                           fn = nullptr;
    cudaDriverEntryPointQueryResult q{};
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess
        || q != cudaDriverEntryPointSuccess) {
        return nullptr;
    }
    return reinterpret_cast<PFN_encodeTiled>(fn);
}

bool lm_encode(PFN_encodeTiled encode, CUtensorMap* map, const void* ptr, int rows, int hidden, int box_rows)
{
    const cuuint64_t dims[2]    = {(cuuint64_t)hidden, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)hidden * 2};
    const cuuint32_t box[2]     = {(cuuint32_t)kLmKBlock, (cuuint32_t)box_rows};
    const cuuint32_t estr[2]    = {1u, 1u};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
           == CUDA_SUCCESS;
}

}  // namespace

cudaError_t lm_head_prepare(int max_smem)
{
    return cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
}

// logits[tokens][ld] = x[tokens][hidden] . w[vocab][hidden]^T; tokens <= 256 per launch (longer batches are cut)
int lm_head_launch(float* logits, int ld, const __half* x, const __half* w, int tokens, int vocab, int hidden, unsigned* status,
                   long long max_wait_cycles, int max_smem, cudaStream_t st, bool pdl, unsigned long long* launches)
{
    if (!logits || !x || !w || tokens <= 0 || vocab <= 0 || hidden <= 0) return TM_ERR_INVALID_ARG;
    if (hidden % kLmKBlock || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return TM_ERR_UNSUPPORTED;
    static const PFN_encodeTiled encode = lm_lookup_encode_tiled();
    if (encode == nullptr) return TM_ERR_CUDA;
    for (int t0 = 0; t0 < tokens; t0 += 256) {
        const int    n  = tokens - t0 < 256 ? tokens - t0 : 256;
        LmHeadParams p{};
        p.logits     = logits + (size_t)t0 * ld;
        p.ld         = ld;
        p.tokens     = n;
        p.vocab      = vocab;
        p.hidden     = hidden;
        p.token_tile = (n + 15) / 16 * 16;
        p.tmem_cols  = 32;
        while (p.tmem_cols < p.token_tile) p.tmem_cols *= 2;
        const size_t stage_b = (size_t)kLmTileV * 128 + (size_t)p.token_tile * 128;
        // two CTAs per SM while the accumulators of both fit TMEM side by side and a ring of >= 3 stages fits half the
        // shared memory; one CTA with a deeper ring otherwise
        const size_t budget = (p.token_tile <= 128 ? (size_t)max_smem / 2 : (size_t)max_smem) - 2048;
        int          stages = (int)(budget / stage_b);
        if (stages > kLmMaxStages) stages = kLmMaxStages;
        if (stages < 2) return TM_ERR_UNSUPPORTED;
        p.stages          = stages;
        p.status          = status;
        p.max_wait_cycles = max_wait_cycles > 0 ? max_wait_cycles : kMaxWaitCycles;
        CUtensorMap w_map, x_map;
        if (!lm_encode(encode, &w_map, w, vocab, hidden, kLmTileV)) return TM_ERR_CUDA;
        if (!lm_encode(encode, &x_map, x + (size_t)t0 * hidden, n, hidden, p.token_tile)) return TM_ERR_CUDA;
        const size_t smem = 1024 + (size_t)stages * stage_b + sizeof(LmBars) + 64;
        const dim3   grid((vocab + kLmTileV - 1) / kLmTileV);
        if (launch_kernel(lm_head_kernel, grid, dim3(kLmThreads), smem, st, pdl, p, w_map, x_map) != cudaSuccess) return TM_ERR_CUDA;
        if (launches) ++*launches;
    }
    return TM_OK;
}

}  // namespace tmb
