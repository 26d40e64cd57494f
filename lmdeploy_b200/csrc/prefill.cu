// Prefill-side writers around the KV cache (lmdeploy v0.0.9, fp16):
//
//   add_fused_qkv_bias_transpose   replaces invokeAddFusedQKVBiasTranspose
//                                  (src/turbomind/kernels/unfused_attention_kernels.cu:852-1027)
//   extend_kv_cache                replaces invokeExtendKVCache
//                                  (src/turbomind/models/llama/llama_kernels.cu:245-464)
//   transpose_kv_cache             replaces invokeTransposeKVCache
//                                  (src/turbomind/models/llama/llama_kernels.cu:497-660)
//
// All three are pure HBM traffic, so each moves 16 bytes per thread and does the K and the V half of
// its job in ONE launch (the reference launches K and V separately, and one 64-thread CTA per
// (token, head) for the first).  The rotary angles of a token are the same for all of its heads:
// one CTA owns a token, computes its 64 (cos, sin) pairs once and applies them to all heads.
// The transpose reads a cached row once and writes it to every query head of its group.
#include "common.cuh"
#include "mmha.h"

namespace tmb {
namespace {

constexpr int kD            = 128;  // size_per_head: the only one the reference instantiates
constexpr int kVecPerHead   = kD / 8;
constexpr int kHeadsPerCta  = 16;
constexpr int kQkvThreads   = kHeadsPerCta * kVecPerHead;  // 256
constexpr int kCacheThreads = 256;

struct QkvParams {
    __half*       q_buf;
    __half*       k_buf;
    __half*       v_buf;
    const __half* qkv;
    const __half* bias;
    const int*    padding_offset;
    const int*    history_length;
    const int*    input_length;
    int           batch, seq_len;
    int           H, Hkv;
    int           rot_dim;
    float         rope_base;
    int           max_pos;
    int           use_dynamic_ntk;
    int           use_logn;
};

constexpr int kHeadBatch = 4;  // 16-byte loads a thread keeps in flight: 4 x 16 heads per pass

// grid (token_num); thread = (head within a group of 16, 16-byte vector of the head); the CTA walks all
// H + 2 Hkv heads of its token in passes of 64, so the token's angles are computed once
__global__ void __launch_bounds__(kQkvThreads) qkv_bias_rope_transpose_kernel(QkvParams p)
{
    __shared__ float2 coef[kD / 2];  // (cos, sin) of pair i = elements 2i, 2i + 1
    pdl_wait();
    pdl_launch_dependents();
    const int token = blockIdx.x;
    const int total = p.H + 2 * p.Hkv;
    const int hsub  = threadIdx.x / kVecPerHead;
    const int vec   = threadIdx.x % kVecPerHead;
    const __half* row = p.qkv + (size_t)token * total * kD + vec * 8;
    uint4 x[kHeadBatch], b[kHeadBatch];
    auto  load_pass = [&](int h0) {
#pragma unroll
        for (int j = 0; j < kHeadBatch; ++j) {
            const int head = h0 + j * kHeadsPerCta + hsub;
            x[j] = b[j] = make_uint4(0, 0, 0, 0);
            if (head < total) {
                x[j] = *reinterpret_cast<const uint4*>(row + (size_t)head * kD);
                if (p.bias) b[j] = *reinterpret_cast<const uint4*>(p.bias + (size_t)head * kD + vec * 8);
            }
        }
    };
    load_pass(0);  // requested first: the angle arithmetic below runs while the rows are in flight
    const int tgt  = token + (p.padding_offset ? p.padding_offset[token] : 0);  // :877-878
    const int bi   = tgt / p.seq_len;
    const int si   = tgt % p.seq_len;
    if (tgt < 0 || bi >= p.batch) return;  // a padding offset that points outside [batch, seq_len]: nothing is written
    const int hist = p.history_length[bi];
    const int step = hist + si;  // :929
    if (threadIdx.x < kD / 2) {
        float2 c = make_float2(1.f, 0.f);
        if (2 * (int)threadIdx.x < p.rot_dim) {
            float base = p.rope_base;
            if (p.use_dynamic_ntk) {
                // decoder_masked_multihead_attention_utils.h:862-871 with the context length (:928,931-934)
                const float len = (float)(hist + p.input_length[bi]);
                if (!(len < (float)p.max_pos)) {
                    const float alpha = fmaxf(exp2f(ceilf(log2f(len / (float)p.max_pos) + 1.f)) - 1.f, 1.f);
                    base *= powf(alpha, (float)p.rot_dim / ((float)p.rot_dim - 2.f));
                }
            }
            const float ang = (float)step / powf(base, (float)(2 * threadIdx.x) / (float)p.rot_dim);  // utils.h:885-889
            c = make_float2(cosf(ang), sinf(ang));  // two separate calls, as utils.h:888 makes them: the pair call rounds differently
        }
        coef[threadIdx.x] = c;
    }
    __syncthreads();
    // :940-950: scaling of the length at this step, rounded to fp16, multiplied in fp16
    const float   len1 = (float)(step + 1);
    const __half2 logn = __half2half2(__float2half(len1 <= (float)p.max_pos ? 1.f : log2f(len1) / log2f((float)p.max_pos)));
    for (int h0 = 0; h0 < total; h0 += kHeadBatch * kHeadsPerCta) {
        if (h0) load_pass(h0);
#pragma unroll
        for (int j = 0; j < kHeadBatch; ++j) {
            const int head = h0 + j * kHeadsPerCta + hsub;
            if (head >= total) continue;
            __half2* xh = reinterpret_cast<__half2*>(&x[j]);
            if (p.bias) {
                const __half2* bh = reinterpret_cast<const __half2*>(&b[j]);
#pragma unroll
                for (int e = 0; e < 4; ++e) xh[e] = __hadd2(xh[e], bh[e]);  // fp16 add, :903-904
            }
            const bool is_q = head < p.H;
            if (head < p.H + p.Hkv) {  // q and k rotate, v does not
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int pr = vec * 4 + e;
                    if (2 * pr < p.rot_dim) {
                        const float2 c = coef[pr];
                        const float2 v = __half22float2(xh[e]);
                        // utils.h:891-904; the contraction the reference build ends up with: second product rounded, first fused
                        xh[e] = __floats2half2_rn(__fmaf_rn(c.x, v.x, -__fmul_rn(c.y, v.y)), __fmaf_rn(c.x, v.y, __fmul_rn(c.y, v.x)));
                    }
                }
            }
            if (is_q && p.use_logn) {
#pragma unroll
                for (int e = 0; e < 4; ++e) xh[e] = __hmul2(logn, xh[e]);
            }
            // [B, heads, seq_len, D]
            if (is_q) {
                *reinterpret_cast<uint4*>(p.q_buf + (((size_t)bi * p.H + head) * p.seq_len + si) * kD + vec * 8) = x[j];
            }
            else {
                const bool is_k = head < p.H + p.Hkv;
                const int  kvh  = head - p.H - (is_k ? 0 : p.Hkv);
                __half*    dst  = is_k ? p.k_buf : p.v_buf;
                *reinterpret_cast<uint4*>(dst + (((size_t)bi * p.Hkv + kvh) * p.seq_len + si) * kD + vec * 8) = x[j];
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// cache writers / readers.  One thread = 8 consecutive elements of one cache row.

// llama_kernels.cu:318-341: (x - zp) / scale, round to nearest even, saturate to int8
__device__ __forceinline__ uint32_t quant4(__half2 a, __half2 b, float scale, float zp)
{
    const float2 fa = __half22float2(a), fb = __half22float2(b);
    int          q[4];
    q[0] = __float2int_rn(__fdiv_rn(fa.x - zp, scale));
    q[1] = __float2int_rn(__fdiv_rn(fa.y - zp, scale));
    q[2] = __float2int_rn(__fdiv_rn(fb.x - zp, scale));
    q[3] = __float2int_rn(__fdiv_rn(fb.y - zp, scale));
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) w |= (uint32_t)(uint8_t)(int8_t)max(-128, min(127, q[i])) << (8 * i);
    return w;
}

// llama_kernels.cu:309-316: q * scale + zp in fp32 (one fused multiply-add), rounded to fp16
__device__ __forceinline__ uint2 dequant4(uint32_t w, float scale, float zp)
{
    __half h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __float2half(__fmaf_rn((float)(int8_t)(w >> (8 * i)), scale, zp));
    uint2 r;
    r.x = (uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16);
    r.y = (uint32_t)__half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16);
    return r;
}

struct CacheParams {
    void* const*  k_cache;  // [B] base pointers (fp16 or int8 elements)
    void* const*  v_cache;
    size_t        offset;  // elements
    __half*       k_lin;   // [B, heads, max_len, D] contiguous side
    __half*       v_lin;
    const int*    length;   // rows to move per sequence
    const int*    history;  // first cache row per sequence (extend only)
    int           max_len;  // rows per head of the contiguous side
    int           max_seq_len;
    int           Hkv;
    int           n_rep;  // query heads per cached head (transpose only)
    float         k_scale, k_zp, v_scale, v_zp;
};

// grid (ceil(max_q_len * 16 / 256), B, 2 * Hkv): [B, Hkv, s, D] -> cache rows [history, history + s)
template<bool INT8>
__global__ void __launch_bounds__(kCacheThreads) extend_kv_cache_kernel(CacheParams p)
{
    pdl_wait();
    pdl_launch_dependents();
    const int  bi   = blockIdx.y;
    const bool is_v = (int)blockIdx.z >= p.Hkv;
    const int  hi   = blockIdx.z - (is_v ? p.Hkv : 0);
    const int  idx  = blockIdx.x * kCacheThreads + threadIdx.x;
    const int  vec  = idx % kVecPerHead;
    const int  row  = idx / kVecPerHead;
    // a length beyond what the contiguous side holds per head is a caller error: never read the neighbouring head
    if (row >= p.length[bi] || row >= p.max_len) return;
    if (row + p.history[bi] >= p.max_seq_len) return;  // never past the rows a cache head holds
    const __half* src  = (is_v ? p.v_lin : p.k_lin) + (((size_t)bi * p.Hkv + hi) * p.max_len + row) * kD + vec * 8;
    const uint4   x    = *reinterpret_cast<const uint4*>(src);
    const size_t  dsti = p.offset + ((size_t)hi * p.max_seq_len + row + p.history[bi]) * kD + vec * 8;
    void*         base = (is_v ? p.v_cache : p.k_cache)[bi];
    if (INT8) {
        const __half2* xh    = reinterpret_cast<const __half2*>(&x);
        const float    scale = is_v ? p.v_scale : p.k_scale, zp = is_v ? p.v_zp : p.k_zp;
        uint2          w;
        w.x = quant4(xh[0], xh[1], scale, zp);
        w.y = quant4(xh[2], xh[3], scale, zp);
        *reinterpret_cast<uint2*>(static_cast<int8_t*>(base) + dsti) = w;
    }
    else {
        *reinterpret_cast<uint4*>(static_cast<__half*>(base) + dsti) = x;
    }
}

// grid (ceil(max_kv_len * 16 / 256), B, 2 * Hkv): cache rows [0, length) -> [B, Hkv * n_rep, max_kv_len, D]
template<bool INT8>
__global__ void __launch_bounds__(kCacheThreads) transpose_kv_cache_kernel(CacheParams p)
{
    pdl_wait();
    pdl_launch_dependents();
    const int  bi   = blockIdx.y;
    const bool is_v = (int)blockIdx.z >= p.Hkv;
    const int  hi   = blockIdx.z - (is_v ? p.Hkv : 0);
    const int  idx  = blockIdx.x * kCacheThreads + threadIdx.x;
    const int  vec  = idx % kVecPerHead;
    const int  row  = idx / kVecPerHead;
    // rows beyond what either side holds per head (a caller error) are skipped, not taken from the next head
    if (row >= p.length[bi] || row >= p.max_len || row >= p.max_seq_len) return;
    const size_t srci = p.offset + ((size_t)hi * p.max_seq_len + row) * kD + vec * 8;
    const void*  base = (is_v ? p.v_cache : p.k_cache)[bi];
    uint4        x;
    if (INT8) {
        const uint2 w     = *reinterpret_cast<const uint2*>(static_cast<const int8_t*>(base) + srci);
        const float scale = is_v ? p.v_scale : p.k_scale, zp = is_v ? p.v_zp : p.k_zp;
        const uint2 lo = dequant4(w.x, scale, zp), hi2 = dequant4(w.y, scale, zp);
        x = make_uint4(lo.x, lo.y, hi2.x, hi2.y);
    }
    else {
        x = *reinterpret_cast<const uint4*>(static_cast<const __half*>(base) + srci);
    }
    __half* dst = is_v ? p.v_lin : p.k_lin;
    for (int r = 0; r < p.n_rep; ++r) {  // llama_kernels.cu:526: query head h reads cached head h / n_rep
        const size_t h = (size_t)hi * p.n_rep + r;
        *reinterpret_cast<uint4*>(dst + (((size_t)bi * p.Hkv * p.n_rep + h) * p.max_len + row) * kD + vec * 8) = x;
    }
}

}  // namespace
}  // namespace tmb

#include "tm_b200.h"

using namespace tmb;

namespace {
bool aligned16(std::initializer_list<const void*> ptrs)
{
    uintptr_t all = 0;
    for (const void* p : ptrs) all |= (uintptr_t)p;
    return (all & 15u) == 0;
}
int status_of(cudaError_t e)
{
    return e == cudaSuccess ? TM_OK : TM_ERR_CUDA;
}
}  // namespace

extern "C" int tm_add_fused_qkv_bias_transpose(void* q_buf, void* k_buf, void* v_buf, const void* QKV, const void* qkv_bias,
                                               const int* padding_offset, const int* history_length, const int* input_length,
                                               int batch_size, int seq_len, int token_num, int head_num, int kv_head_num,
                                               int size_per_head, int rotary_embedding_dim, float rotary_embedding_base,
                                               int max_position_embeddings, int use_dynamic_ntk, int use_logn_attn, void* stream)
{
    if (!q_buf || !k_buf || !v_buf || !QKV || !history_length || !input_length) return TM_ERR_INVALID_ARG;
    if (batch_size < 0 || seq_len <= 0 || token_num < 0 || head_num <= 0 || kv_head_num <= 0) return TM_ERR_INVALID_ARG;
    if (rotary_embedding_dim <= 0) return TM_ERR_INVALID_ARG;  // FT_CHECK(rotary_embedding_dim), :1020
    if (size_per_head != kD || rotary_embedding_dim > kD || rotary_embedding_dim % 2) return TM_ERR_UNSUPPORTED;
    if (!aligned16({q_buf, k_buf, v_buf, QKV, qkv_bias})) return TM_ERR_INVALID_ARG;
    if (token_num == 0 || batch_size == 0) return TM_OK;
    QkvParams p{(__half*)q_buf, (__half*)k_buf, (__half*)v_buf, (const __half*)QKV, (const __half*)qkv_bias, padding_offset,
                history_length, input_length, batch_size, seq_len, head_num, kv_head_num, rotary_embedding_dim, rotary_embedding_base,
                max_position_embeddings, use_dynamic_ntk, use_logn_attn};
    const dim3 grid(token_num);
    return status_of(launch_kernel(qkv_bias_rope_transpose_kernel, grid, dim3(kQkvThreads), 0, (cudaStream_t)stream, false, p));
}

extern "C" int tm_extend_kv_cache(void** k_dst, void** v_dst, size_t dst_offset, const void* k_src, const void* v_src,
                                  int local_batch_size, const int* query_length, int max_q_len, const int* history_length,
                                  int max_seq_len, int size_per_head, int local_head_num, void* stream, int quant,
                                  const float* kv_scale)
{
    if (!k_dst || !v_dst || !k_src || !v_src || !query_length || !history_length) return TM_ERR_INVALID_ARG;
    if (local_batch_size < 0 || max_q_len < 0 || max_seq_len <= 0 || local_head_num <= 0) return TM_ERR_INVALID_ARG;
    const bool int8 = (quant & 0x04) != 0;  // QuantPolicy::kCacheKVInt8, llama_utils.h:12-20
    if (int8 && !kv_scale) return TM_ERR_INVALID_ARG;
    if (size_per_head != kD) return TM_ERR_UNSUPPORTED;
    if (!aligned16({k_src, v_src}) || dst_offset % 16) return TM_ERR_INVALID_ARG;
    if (local_batch_size == 0 || max_q_len == 0) return TM_OK;
    if (local_batch_size > 65535 || 2 * local_head_num > 65535) return TM_ERR_UNSUPPORTED;
    CacheParams p{};
    p.k_cache = k_dst, p.v_cache = v_dst, p.offset = dst_offset;
    p.k_lin = (__half*)k_src, p.v_lin = (__half*)v_src;
    p.length = query_length, p.history = history_length;
    p.max_len = max_q_len, p.max_seq_len = max_seq_len, p.Hkv = local_head_num, p.n_rep = 1;
    if (int8) p.k_scale = kv_scale[0], p.k_zp = kv_scale[1], p.v_scale = kv_scale[2], p.v_zp = kv_scale[3];
    const dim3 grid((max_q_len * kVecPerHead + kCacheThreads - 1) / kCacheThreads, local_batch_size, 2 * local_head_num);
    return status_of(int8 ? launch_kernel(extend_kv_cache_kernel<true>, grid, dim3(kCacheThreads), 0, (cudaStream_t)stream, false, p) :
                            launch_kernel(extend_kv_cache_kernel<false>, grid, dim3(kCacheThreads), 0, (cudaStream_t)stream, false, p));
}

extern "C" int tm_transpose_kv_cache(void* key_cache_trans, void* val_cache_trans, const void** key_cache, const void** val_cache,
                                     size_t src_offset, int batch_size, const int* key_length, int max_kv_len, int max_seq_len,
                                     int size_per_head, int head_num, int head_n_rep, void* stream, int quant,
                                     const float* kv_scale)
{
    if (!key_cache_trans || !val_cache_trans || !key_cache || !val_cache || !key_length) return TM_ERR_INVALID_ARG;
    if (batch_size < 0 || max_kv_len < 0 || max_seq_len <= 0 || head_num <= 0 || head_n_rep <= 0 || head_num % head_n_rep) {
        return TM_ERR_INVALID_ARG;
    }
    const bool int8 = (quant & 0x04) != 0;
    if (int8 && !kv_scale) return TM_ERR_INVALID_ARG;
    if (size_per_head != kD) return TM_ERR_UNSUPPORTED;
    if (!aligned16({key_cache_trans, val_cache_trans}) || src_offset % 16) return TM_ERR_INVALID_ARG;
    if (batch_size == 0 || max_kv_len == 0) return TM_OK;
    const int hkv = head_num / head_n_rep;
    if (batch_size > 65535 || 2 * hkv > 65535) return TM_ERR_UNSUPPORTED;
    CacheParams p{};
    p.k_cache = (void* const*)key_cache, p.v_cache = (void* const*)val_cache, p.offset = src_offset;
    p.k_lin = (__half*)key_cache_trans, p.v_lin = (__half*)val_cache_trans;
    p.length = key_length, p.history = nullptr;
    p.max_len = max_kv_len, p.max_seq_len = max_seq_len, p.Hkv = hkv, p.n_rep = head_n_rep;
    if (int8) p.k_scale = kv_scale[0], p.k_zp = kv_scale[1], p.v_scale = kv_scale[2], p.v_zp = kv_scale[3];
    const dim3 grid((max_kv_len * kVecPerHead + kCacheThreads - 1) / kCacheThreads, batch_size, 2 * hkv);
    return status_of(int8 ? launch_kernel(transpose_kv_cache_kernel<true>, grid, dim3(kCacheThreads), 0, (cudaStream_t)stream, false, p) :
                            launch_kernel(transpose_kv_cache_kernel<false>, grid, dim3(kCacheThreads), 0, (cudaStream_t)stream, false, p));
}
