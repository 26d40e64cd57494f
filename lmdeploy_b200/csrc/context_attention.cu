// Prefill (context) attention over the KV cache, fp16, head size 128: causal softmax(q k^T / sqrt(d)) v for
// every new token of every sequence, keys and values read IN PLACE from the per-sequence cache
// ([kv heads, max_seq_len, 128], fp16 or int8), output packed [token, heads * 128].
//
// Replaces what LlamaContextAttentionLayer<T>::fusedMultiHeadAttention drives
// (src/turbomind/models/llama/LlamaContextAttentionLayer.cc:257-313: FlashAttentionOp over q_buf_2_,
// the cache pointers with the layer offset, cu_seqlens and context_lengths, GQA group_size) and, for an
// int8 cache, the unfused route's invokeTransposeKVCache + batched GEMMs + invokeMaskedSoftmax
// (:316-420) without the dequantised copy of the cache.
//
// One CTA = 64 queries of one (sequence, head): 4 warps x 16 query rows, key/value tiles of 64 rows
// double-buffered in shared memory (cp.async for fp16; int8 rows are fetched to registers one tile ahead
// and dequantised on their way to shared memory), mma.m16n8k16 with fp32 accumulators, online softmax
// in registers, probabilities rounded to fp16 for the second product.  Tiles above the causal
// diagonal are never visited; the longest query tiles are scheduled first.
#include "common.cuh"
#include "context_attention.h"
#include "tm_b200.h"

#include <cstdlib>
#include <mutex>

namespace tmb {
namespace {

constexpr int kD       = 128;
constexpr int kBM      = 64;  // queries per CTA
constexpr int kBN      = 64;  // keys per tile
constexpr int kThreads = 128;
constexpr int kTileBytes = kBN * kD * 2;                         // 16 KB
constexpr int kSmemBytes = kBM * kD * 2 + 4 * kTileBytes;        // q + 2 x (k, v) = 80 KB


// byte offset of the 16-byte chunk `chunk` (0..15) of row `row` in a [rows][128] fp16 tile
__device__ __forceinline__ uint32_t tile_off(int row, int chunk)
{
    return (uint32_t)(row * 256 + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
// 16 bytes global -> shared; bytes == 0 writes zeros and reads nothing
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit_group()
{
    asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void cp_async_wait_all()
{
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}
// 2^x by the special-function unit (one instruction; relative error 2^-22, far below the fp16 rounding of p)
__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b)
{
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// 4 int8 -> 4 halves, half(q * scale + zp) with one fp32 fused multiply-add (llama_kernels.cu:309-316).  The
// integer -> float step avoids the conversion unit (a quarter-rate pipe shared with ex2): byte q + 128 is dropped into
// the mantissa of 2^23, and 2^23 + 128 subtracted again — exact, so the result is the same float as (float)q.
__device__ __forceinline__ uint2 dequant4(uint32_t w, float scale, float zp)
{
    const uint32_t u = w ^ 0x80808080u;
    const float    f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.f;
    const float    f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.f;
    const float    f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.f;
    const float    f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.f;
    uint2 r;
    r.x = pack_half2(__fmaf_rn(f0, scale, zp), __fmaf_rn(f1, scale, zp));
    r.y = pack_half2(__fmaf_rn(f2, scale, zp), __fmaf_rn(f3, scale, zp));
    return r;
}

template<bool INT8>
__global__ void __launch_bounds__(kThreads) context_attention_kernel(CtxParams p)
{
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t q_s  = smem_u32(smem);
    const uint32_t kv_s = q_s + kBM * kD * 2;  // [buf][k | v]
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int bi = blockIdx.z, h = blockIdx.y;
    const int qt    = gridDim.x - 1 - blockIdx.x;  // the longest (latest) query tiles first
    const int tok0  = p.cu_seqlens[bi];
    const int q_len = p.cu_seqlens[bi + 1] - tok0;
    const int ctx   = p.context_length[bi];
    const int hist  = ctx - q_len;
    const int q0    = qt * kBM;
    if (q0 >= q_len) return;
    // keys any query of this tile may see; never past the rows a cache head holds
    const int kv_end  = min(min(ctx, p.max_seq_len), hist + min(q0 + kBM, q_len));
    const int n_tiles = (kv_end + kBN - 1) / kBN;
    const int kvh     = h / p.n_rep;

    const size_t         head_off = p.offset + (size_t)kvh * p.max_seq_len * kD;  // elements
    const unsigned char* k_base   = static_cast<const unsigned char*>(p.k_cache[bi]) + head_off * (INT8 ? 1 : 2);
    const unsigned char* v_base   = static_cast<const unsigned char*>(p.v_cache[bi]) + head_off * (INT8 ? 1 : 2);

    // ---- tile movers
    auto load_tile_f16 = [&](int t, int buf) {
        const int key0 = t * kBN;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const int  c = tid + r * kThreads, row = c >> 4, chunk = c & 15;
            const bool ok  = key0 + row < kv_end;
            const size_t src = ((size_t)(ok ? key0 + row : 0) * kD + chunk * 8) * 2;
            const uint32_t dst = kv_s + buf * 2 * kTileBytes + tile_off(row, chunk);
            cp_async16(dst, k_base + src, ok ? 16 : 0);
            cp_async16(dst + kTileBytes, v_base + src, ok ? 16 : 0);
        }
    };
    uint4 stage_k[4], stage_v[4];  // int8 only: the next tile on its way from global to shared memory
    auto fetch_tile_s8 = [&](int t) {
        const int key0 = t * kBN;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int  c = tid + r * kThreads, row = c >> 3, chunk = c & 7;
            const bool ok = key0 + row < kv_end;
            stage_k[r] = stage_v[r] = make_uint4(0, 0, 0, 0);
            if (ok) {
                const size_t src = (size_t)(key0 + row) * kD + chunk * 16;
                stage_k[r]       = *reinterpret_cast<const uint4*>(k_base + src);
                stage_v[r]       = *reinterpret_cast<const uint4*>(v_base + src);
            }
        }
    };
    auto store_tile_s8 = [&](int t, int buf) {
        const int key0 = t * kBN;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int  c = tid + r * kThreads, row = c >> 3, chunk = c & 7;
            const bool ok = key0 + row < kv_end;  // rows past the end stay exact zeros (not the zero point)
            unsigned char* dst = smem + kBM * kD * 2 + buf * 2 * kTileBytes;
            uint4 k0 = make_uint4(0, 0, 0, 0), k1 = k0, v0 = k0, v1 = k0;
            if (ok) {
                const uint2 a = dequant4(stage_k[r].x, p.k_scale, p.k_zp), b = dequant4(stage_k[r].y, p.k_scale, p.k_zp);
                const uint2 c2 = dequant4(stage_k[r].z, p.k_scale, p.k_zp), d = dequant4(stage_k[r].w, p.k_scale, p.k_zp);
                k0 = make_uint4(a.x, a.y, b.x, b.y), k1 = make_uint4(c2.x, c2.y, d.x, d.y);
                const uint2 e = dequant4(stage_v[r].x, p.v_scale, p.v_zp), f = dequant4(stage_v[r].y, p.v_scale, p.v_zp);
                const uint2 g2 = dequant4(stage_v[r].z, p.v_scale, p.v_zp), hh = dequant4(stage_v[r].w, p.v_scale, p.v_zp);
                v0 = make_uint4(e.x, e.y, f.x, f.y), v1 = make_uint4(g2.x, g2.y, hh.x, hh.y);
            }
            *reinterpret_cast<uint4*>(dst + tile_off(row, 2 * chunk))                  = k0;
            *reinterpret_cast<uint4*>(dst + tile_off(row, 2 * chunk + 1))              = k1;
            *reinterpret_cast<uint4*>(dst + kTileBytes + tile_off(row, 2 * chunk))     = v0;
            *reinterpret_cast<uint4*>(dst + kTileBytes + tile_off(row, 2 * chunk + 1)) = v1;
        }
    };

    // ---- prologue: the query tile and key/value tile 0
    {
        const __half* qsrc = p.q + ((size_t)bi * p.H + h) * p.max_q_len * kD;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const int  c = tid + r * kThreads, row = c >> 4, chunk = c & 15;
            const bool ok = q0 + row < q_len;
            cp_async16(q_s + tile_off(row, chunk), qsrc + (size_t)(ok ? q0 + row : 0) * kD + chunk * 8, ok ? 16 : 0);
        }
    }
    if (INT8) {
        fetch_tile_s8(0);
        store_tile_s8(0, 0);
    }
    else {
        load_tile_f16(0, 0);
    }
    cp_async_commit_group();
    cp_async_wait_all();
    __syncthreads();

    uint32_t qf[8][4];  // this warp's 16 query rows as A fragments of the 8 k-steps
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
        const int m = lane >> 3;
        ldsm_x4(qf[kk], q_s + tile_off(warp * 16 + (m & 1) * 8 + (lane & 7), 2 * kk + (m >> 1)));
    }

    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float row_max[2] = {-1e30f, -1e30f}, row_sum[2] = {0.f, 0.f};
    const int g = lane >> 2, tq = lane & 3;
    const int qpos0 = hist + q0 + warp * 16 + g;  // position of this thread's first row; the second is + 8

    for (int t = 0; t < n_tiles; ++t) {
        const int buf = t & 1;
        if (t + 1 < n_tiles) {
            if (INT8) {
                fetch_tile_s8(t + 1);
            }
            else {
                load_tile_f16(t + 1, buf ^ 1);
                cp_async_commit_group();
            }
        }
        const uint32_t k_s = kv_s + buf * 2 * kTileBytes, v_s = k_s + kTileBytes;

        // ---- s = q k^T : 16 x 64 per warp
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        {
            // one ldmatrix.x4 = the B fragments of two key groups for one k-step, fetched one step ahead of the two
            // (independent) MMAs that use them
            const int m      = lane >> 3;
            auto      k_addr = [&](int i) { return k_s + tile_off((2 * (i & 3) + (m >> 1)) * 8 + (lane & 7), 2 * (i >> 2) + (m & 1)); };
            uint32_t  b[2][4];
            ldsm_x4(b[0], k_addr(0));
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                if (i + 1 < 32) ldsm_x4(b[(i + 1) & 1], k_addr(i + 1));
                const int kk = i >> 2, jp = i & 3;
                mma_m16n8k16(s[2 * jp], qf[kk], b[i & 1][0], b[i & 1][1]);
                mma_m16n8k16(s[2 * jp + 1], qf[kk], b[i & 1][2], b[i & 1][3]);
            }
        }
        // ---- causal mask (only tiles that reach the diagonal of this warp's rows)
        const int key0 = t * kBN;
        if (key0 + kBN - 1 > hist + q0 + warp * 16) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int kj = key0 + j * 8 + 2 * tq;
                if (kj > qpos0) s[j][0] = -1e30f;
                if (kj + 1 > qpos0) s[j][1] = -1e30f;
                if (kj > qpos0 + 8) s[j][2] = -1e30f;
                if (kj + 1 > qpos0 + 8) s[j][3] = -1e30f;
            }
        }
        // ---- online softmax; rows g and g + 8 live in the 4 lanes of a quad
        float mx[2] = {row_max[0], row_max[1]};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
            mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        }
        const float corr[2] = {fast_exp2((row_max[0] - mx[0]) * p.scale_log2), fast_exp2((row_max[1] - mx[1]) * p.scale_log2)};
        const float off[2]  = {-mx[0] * p.scale_log2, -mx[1] * p.scale_log2};  // p = 2^(s * scale + off): one fma per score
        row_max[0] = mx[0], row_max[1] = mx[1];
        float part[2] = {0.f, 0.f};
        uint32_t pa[4][4];  // probabilities as A fragments of the 4 key blocks of 16
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float p0 = fast_exp2(fmaf(s[j][0], p.scale_log2, off[0])), p1 = fast_exp2(fmaf(s[j][1], p.scale_log2, off[0]));
            const float p2 = fast_exp2(fmaf(s[j][2], p.scale_log2, off[1])), p3 = fast_exp2(fmaf(s[j][3], p.scale_log2, off[1]));
            part[0] += p0 + p1;
            part[1] += p2 + p3;
            pa[j >> 1][(j & 1) * 2]     = pack_half2(p0, p1);
            pa[j >> 1][(j & 1) * 2 + 1] = pack_half2(p2, p3);
        }
        row_sum[0] = row_sum[0] * corr[0] + part[0];
        row_sum[1] = row_sum[1] * corr[1] + part[1];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            o[i][0] *= corr[0], o[i][1] *= corr[0];
            o[i][2] *= corr[1], o[i][3] *= corr[1];
        }
        // ---- o += p v
        {
            const int m      = lane >> 3;
            auto      v_addr = [&](int i) { return v_s + tile_off((i >> 3) * 16 + (m & 1) * 8 + (lane & 7), 2 * (i & 7) + (m >> 1)); };
            uint32_t  b[2][4];
            ldsm_x4_trans(b[0], v_addr(0));
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                if (i + 1 < 32) ldsm_x4_trans(b[(i + 1) & 1], v_addr(i + 1));
                const int kb = i >> 3, dn2 = i & 7;
                mma_m16n8k16(o[2 * dn2], pa[kb], b[i & 1][0], b[i & 1][1]);
                mma_m16n8k16(o[2 * dn2 + 1], pa[kb], b[i & 1][2], b[i & 1][3]);
            }
        }
        if (t + 1 < n_tiles) {
            if (INT8) {
                store_tile_s8(t + 1, buf ^ 1);
            }
            else {
                cp_async_wait_all();
            }
        }
        __syncthreads();
    }

    // ---- normalise and store: out[token, h * 128 + d]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float sum = row_sum[r];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const int   qi  = q0 + warp * 16 + g + r * 8;
        const float inv = 1.f / sum;
        if (qi < q_len) {
            __half* dst = p.out + ((size_t)(tok0 + qi) * p.H + h) * kD + 2 * tq;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_half2(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
            }
        }
    }
}

}  // namespace
}  // namespace tmb

using namespace tmb;

namespace {
unsigned* own_status[64] = {};  // per device: the status word of callers that bring none
}

extern "C" int tm_context_attention_last_status(unsigned* word)
{
    if (!word) return TM_ERR_INVALID_ARG;
    *word   = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TM_ERR_CUDA;
    if (!own_status[dev]) return TM_OK;
    if (cudaDeviceSynchronize() != cudaSuccess) return TM_ERR_CUDA;
    if (cudaMemcpy(word, own_status[dev], sizeof(unsigned), cudaMemcpyDeviceToHost) != cudaSuccess) return TM_ERR_CUDA;
    if (*word) cudaMemset(own_status[dev], 0, sizeof(unsigned));
    return TM_OK;
}

extern "C" int tm_context_attention(const tm_context_attention_params* a, void* stream)
{
    if (!a || !a->attn_out || !a->query || !a->key_cache || !a->val_cache || !a->cu_seqlens || !a->context_lengths) {
        return TM_ERR_INVALID_ARG;
    }
    if (a->batch_size < 0 || a->head_num <= 0 || a->kv_head_num <= 0 || a->head_num % a->kv_head_num || a->max_q_len < 0
        || a->max_seq_len <= 0) {
        return TM_ERR_INVALID_ARG;
    }
    if (a->size_per_head != kD) return TM_ERR_UNSUPPORTED;
    if ((((uintptr_t)a->attn_out | (uintptr_t)a->query) & 15u) || a->cache_layer_offset % 16) return TM_ERR_INVALID_ARG;
    if (a->batch_size == 0 || a->max_q_len == 0) return TM_OK;
    if (a->batch_size > 65535 || a->head_num > 65535) return TM_ERR_UNSUPPORTED;
    const bool int8 = (a->quant_policy & 0x04) != 0;  // QuantPolicy::kCacheKVInt8, llama_utils.h:12-20
    CtxParams  p{};
    p.out = (__half*)a->attn_out, p.q = (const __half*)a->query;
    p.k_cache = a->key_cache, p.v_cache = a->val_cache, p.offset = a->cache_layer_offset;
    p.cu_seqlens = a->cu_seqlens, p.context_length = a->context_lengths;
    p.max_q_len = a->max_q_len, p.max_seq_len = a->max_seq_len, p.H = a->head_num, p.n_rep = a->head_num / a->kv_head_num;
    p.scale_log2 = 1.4426950408889634f / sqrtf((float)kD);
    p.k_scale = a->kv_scale[0], p.k_zp = a->kv_scale[1], p.v_scale = a->kv_scale[2], p.v_zp = a->kv_scale[3];
    // bounded waits of the tcgen05 kernel report into the caller's status word, or into one kept by the library
    // (tm_context_attention_last_status) when the caller has none
    p.status = a->status_word;
    if (!p.status) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TM_ERR_CUDA;
        static std::mutex mu;
        std::lock_guard<std::mutex> lock(mu);
        if (!own_status[dev]) {
            if (cudaMalloc((void**)&own_status[dev], sizeof(unsigned)) != cudaSuccess) return TM_ERR_CUDA;
            cudaMemset(own_status[dev], 0, sizeof(unsigned));
        }
        p.status = own_status[dev];
    }
    p.max_wait_cycles = kMaxWaitCycles;
    // TM_B200_CTX_ATTN_LEGACY=1: the mma.sync kernel below instead of the tcgen05 one (comparison)
    static const bool legacy = [] {
        const char* e = std::getenv("TM_B200_CTX_ATTN_LEGACY");
        return e && e[0] == '1';
    }();
    if (!legacy) {
        return context_attention_tc_launch(p, int8, a->batch_size, (cudaStream_t)stream) == cudaSuccess ? TM_OK : TM_ERR_CUDA;
    }
    auto kernel = int8 ? context_attention_kernel<true> : context_attention_kernel<false>;
    // per call, like every attribute in this library that depends on the current device; cheap next to the kernel
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) return TM_ERR_CUDA;
    const dim3 grid((a->max_q_len + kBM - 1) / kBM, a->head_num, a->batch_size);
    return launch_kernel(kernel, grid, dim3(kThreads), kSmemBytes, (cudaStream_t)stream, false, p) == cudaSuccess ? TM_OK : TM_ERR_CUDA;
}
