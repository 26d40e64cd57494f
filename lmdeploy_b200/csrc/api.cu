// C ABI: handle management and the GEMM entry point.
#include <mutex>
#include "handle.h"
#include "tm_b200.h"

#include <cstdlib>
#include <cstring>
#include <new>
#include <string>

using namespace tmb;

namespace tmb {
thread_local int g_pdl = 0;
thread_local const GemmNormFusion* g_gemm_fusion = nullptr;

bool gemm_can_fuse_norm(const tm_handle* h, int m, int n, int k)
{
    if (!h || n < h->gemm_tc_min_n || n > 128 || k % 128 || m % 32) return false;
    const GemmTcPlan pl = gemm_tc_plan(m, n, k, h->sm_count);
    return gemm_tc_all_tiles_split(pl, k) && pl.workspace_floats * sizeof(float) <= h->scratch_bytes && pl.counter_ints <= h->counter_ints;
}
}

namespace {

int env_int(const char* name, int dflt)
{
    const char* v = std::getenv(name);
    return v && *v ? std::atoi(v) : dflt;
}

}  // namespace

extern "C" const char* tm_status_string(int status)
{
    switch (status) {
        case TM_OK: return "ok";
        case TM_ERR_INVALID_ARG: return "invalid argument";
        case TM_ERR_UNSUPPORTED: return "unsupported shape or option";
        case TM_ERR_WORKSPACE: return "workspace too small";
        case TM_ERR_CUDA: return "CUDA runtime error";
        case TM_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
        case TM_ERR_NCCL: return "NCCL error";
        case TM_ERR_NOT_BUILT: return "feature not built";
        case TM_ERR_IO: return "weight file missing or of the wrong size";
        default: return "unknown status";
    }
}

extern "C" int tm_create(tm_handle** out, int device)
{
    if (!out) return TM_ERR_INVALID_ARG;
    *out = nullptr;
    int prev = 0;
    if (cudaGetDevice(&prev) != cudaSuccess) return TM_ERR_CUDA;
    if (cudaSetDevice(device) != cudaSuccess) return TM_ERR_CUDA;
    tm_handle* h = new (std::nothrow) tm_handle();
    if (!h) return TM_ERR_CUDA;
    h->device = device;
    cudaDeviceProp prop{};
    cudaError_t    e = cudaGetDeviceProperties(&prop, device);
    if (e == cudaSuccess) {
        h->sm_count = prop.multiProcessorCount;
        h->max_smem = (int)prop.sharedMemPerBlockOptin;
        h->l2_bytes = prop.l2CacheSize;
        // scratch: split-K partial tiles + self-resetting tickets, status word
        // TM_B200_GEMM_SCRATCH_MB: more scratch lets one launch of the many-token GEMM cover more tokens (prefill)
        const int scratch_mb = env_int("TM_B200_GEMM_SCRATCH_MB", 256);
        h->scratch_bytes = (size_t)(scratch_mb < 64 ? 64 : (scratch_mb > 16384 ? 16384 : scratch_mb)) << 20;
        h->counter_ints  = 1u << 16;
        e                = cudaMalloc(&h->scratch, h->scratch_bytes);
    }
    if (e == cudaSuccess) e = cudaMalloc(&h->counters, h->counter_ints * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(h->counters, 0, h->counter_ints * sizeof(int));
    h->attn_scratch_bytes = 128u << 20;
    h->attn_counter_ints  = 1u << 18;
    if (e == cudaSuccess) e = cudaMalloc(&h->attn_scratch, h->attn_scratch_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&h->attn_counters, h->attn_counter_ints * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(h->attn_counters, 0, h->attn_counter_ints * sizeof(int));
    if (e == cudaSuccess) e = mmha_prepare();
    if (e == cudaSuccess) e = cudaMalloc(&h->status, 256);
    if (e == cudaSuccess) e = cudaMemset(h->status, 0, 256);
    if (e == cudaSuccess) e = gemm_small_prepare(h->max_smem);
    if (e == cudaSuccess) e = gemm_tc_prepare(h->max_smem);
    if (e == cudaSuccess) e = lm_head_prepare(h->max_smem);
    if (e == cudaSuccess) e = sampling_prepare(h->max_smem);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    h->pdl           = env_int("TM_B200_PDL", 1);
    h->p2p_allreduce = env_int("TM_B200_P2P_ALLREDUCE", 1);
    h->lm_head_cublas = env_int("TM_B200_LM_HEAD_CUBLAS", 0);
    h->fold_norm      = env_int("TM_B200_FOLD_NORM", 1);
    h->gemv_cols      = env_int("TM_B200_GEMV_COLS", 1);
    h->gemm_tc_min_n = env_int("TM_B200_GEMM_TC_MIN", 17);
    h->mmha_chunk  = env_int("TM_B200_MMHA_CHUNK", 0);
    h->mmha_warps  = env_int("TM_B200_MMHA_WARPS", 0);
    cudaSetDevice(prev);
    if (e != cudaSuccess) {
        h->last_cuda_error = (int)e;
        tm_destroy(h);
        return TM_ERR_CUDA;
    }
    *out = h;
    return TM_OK;
}

// One shared handle per device for callers that have nowhere to keep one (the header shims under include/compat, whose
// classes and free functions must keep the reference's signatures).  Created on first use, kept until the process exits.
extern "C" tm_handle* tm_handle_of_current_device(void)
{
    static std::mutex mu;
    static tm_handle* table[64] = {};
    int               dev       = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!table[dev] && tm_create(&table[dev], dev) != TM_OK) table[dev] = nullptr;
    return table[dev];
}

extern "C" int tm_destroy(tm_handle* h)
{
    if (!h) return TM_OK;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(h->device);
    if (h->scratch) cudaFree(h->scratch);
    if (h->counters) cudaFree(h->counters);
    if (h->attn_scratch) cudaFree(h->attn_scratch);
    if (h->attn_counters) cudaFree(h->attn_counters);
    if (h->status) cudaFree(h->status);
    cudaSetDevice(prev);
    delete h;
    return TM_OK;
}

extern "C" int tm_last_cuda_error(const tm_handle* h)
{
    return h ? h->last_cuda_error : 0;
}

extern "C" int tm_set_option(tm_handle* h, const char* name, int value)
{
    if (!h || !name) return TM_ERR_INVALID_ARG;
    const std::string n(name);
    if (n == "gemm_tc_min_n" && value >= 1) {
        h->gemm_tc_min_n = value;
    }
    else if (n == "mmha_chunk" && value >= 0) {
        h->mmha_chunk = value;
    }
    else if (n == "mmha_warps" && (value == 0 || value == 1 || value == 2 || value == 4)) {
        h->mmha_warps = value;
    }
    else if (n == "pdl" && (value == 0 || value == 1)) {
        h->pdl = value;
    }
    else if (n == "p2p_allreduce" && (value == 0 || value == 1)) {
        // 0: the tensor-parallel decode step reduces with NCCL even where the peer-memory path is set up
        h->p2p_allreduce = value;
    }
    else if (n == "fold_norm" && (value == 0 || value == 1)) {
        h->fold_norm = value;
    }
    else if (n == "gemv_cols" && value >= 0 && value <= 2) {
        h->gemv_cols = value;
    }
    else if (n == "lm_head_cublas" && (value == 0 || value == 1)) {
        h->lm_head_cublas = value;
    }
    else if (n == "pdl_direct" && (value == 0 || value == 1)) {
        // GEMM and attention calls made DIRECTLY through this handle also launch with programmatic stream
        // serialization: the kernel may start (and request the packed weights / cache rows of earlier steps) while the
        // kernel before it in the stream still runs.  Only for callers whose preceding kernels never write those.
        h->pdl_direct = value;
    }
    else if (n == "gemm_wait_cycles" && value >= 0) {
        // bound, in SM clock cycles, of the tcgen05 GEMM's wait for the partners of a split column tile
        // (0 = the default of about a quarter of a second); tests set a tiny value to see the time-out path
        h->gemm_wait_cycles = value;
    }
    else {
        return TM_ERR_INVALID_ARG;
    }
    return TM_OK;
}

extern "C" unsigned long long tm_launch_count(const tm_handle* h)
{
    return h ? h->launches : 0ull;
}

extern "C" int tm_check_device_status(tm_handle* h, void* stream, unsigned* word)
{
    if (!h || !word) return TM_ERR_INVALID_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    unsigned     w  = 0;
    cudaError_t  e  = cudaMemcpyAsync(&w, h->status, sizeof(w), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e == cudaSuccess && w != 0) e = cudaMemsetAsync(h->status, 0, sizeof(unsigned), st);
    if (e != cudaSuccess) {
        h->last_cuda_error = (int)e;
        return TM_ERR_CUDA;
    }
    *word = w;
    return w ? TM_ERR_DEVICE_TIMEOUT : TM_OK;
}

extern "C" size_t tm_gemm_s4_f16_workspace_bytes(int m, int n, int k)
{
    if (m <= 0 || n <= 0 || k <= 0 || k % 128 || m % 32) return 0;
    // device independent: the slot count grows with the grid, so plan for a grid no part exceeds
    GemmSmallPlan pl = gemm_small_plan(m, n, k, 256, 227 * 1024);
    size_t        b  = pl.workspace_floats * sizeof(float) + pl.counter_ints * sizeof(int) + 256;
    if (n > 16) {
        GemmTcPlan   tc = gemm_tc_plan(m, n, k, 256);
        const size_t t  = tc.workspace_floats * sizeof(float) + tc.counter_ints * sizeof(int) + 256;
        if (t > b) b = t;
    }
    return b;
}

extern "C" int tm_gemm_s4_f16(tm_handle*  h,
                              void*       C,
                              const void* A,
                              const void* B,
                              const void* Q,
                              int         m,
                              int         n,
                              int         k,
                              int         group_size,
                              int         type,
                              void*       workspace,
                              size_t      workspace_bytes,
                              void*       stream)
{
    if (!h || !C || !A || !B || !Q) return TM_ERR_INVALID_ARG;
    if (((uintptr_t)C | (uintptr_t)A | (uintptr_t)B | (uintptr_t)Q | (uintptr_t)workspace) & 15u) return TM_ERR_INVALID_ARG;
    if (m <= 0 || n <= 0 || k <= 0) return TM_ERR_INVALID_ARG;
    if (group_size != 128 || k % 128 || m % 32) return TM_ERR_UNSUPPORTED;
    if (type != TM_GEMM_PLAIN && type != TM_GEMM_FUSED_SILU_FFN) return TM_ERR_UNSUPPORTED;
    if (type == TM_GEMM_FUSED_SILU_FFN && m % 64) return TM_ERR_UNSUPPORTED;

    if (n >= h->gemm_tc_min_n) {
        // tensor-core tiles; token ranges that would overflow the scratch go in several launches
        const size_t n_out_tc = type == TM_GEMM_FUSED_SILU_FFN ? (size_t)m / 2 : (size_t)m;
        int          per      = n;
        for (;;) {
            GemmTcPlan   pl   = gemm_tc_plan(m, per, k, h->sm_count);
            const size_t c_b  = ((pl.counter_ints * sizeof(int) + 255) / 256) * 256;
            const bool   fits = workspace ? workspace_bytes >= pl.workspace_floats * sizeof(float) + c_b :
                                            (pl.workspace_floats * sizeof(float) <= h->scratch_bytes
                                             && pl.counter_ints <= h->counter_ints);
            if (fits) break;
            if (per <= 128) return TM_ERR_WORKSPACE;
            per = ((per / 2 + 127) / 128) * 128;
        }
        for (int t0 = 0; t0 < n; t0 += per) {
            const int    nt = n - t0 < per ? n - t0 : per;
            GemmTcPlan   pl = gemm_tc_plan(m, nt, k, h->sm_count);
            GemmTcParams p{};
            p.C          = (__half*)C + (size_t)t0 * n_out_tc;
            p.A          = (const unsigned char*)A;
            p.X          = (const unsigned char*)B + (size_t)t0 * k * 2;
            p.Q          = (const unsigned char*)Q;
            p.workspace  = workspace ? (float*)((char*)workspace + ((pl.counter_ints * sizeof(int) + 255) / 256) * 256) :
                                       (float*)h->scratch;
            p.counters   = workspace ? (int*)workspace : h->counters;
            p.status     = h->status;
            p.N          = m;
            p.T          = nt;
            p.K          = k;
            p.fused_silu = type == TM_GEMM_FUSED_SILU_FFN;
            p.max_wait_cycles = h->gemm_wait_cycles;
            if (g_gemm_fusion) {
                if (per != n || workspace || !gemm_tc_all_tiles_split(pl, k)) return TM_ERR_UNSUPPORTED;  // the driver checked
                p.norm = *g_gemm_fusion;
            }
            cudaError_t e = gemm_tc_launch(pl, p, (cudaStream_t)stream, g_pdl != 0 || h->pdl_direct != 0);
            h->launches += 1;
            if (e != cudaSuccess) {
                h->last_cuda_error = (int)e;
                return TM_ERR_CUDA;
            }
        }
        return TM_OK;
    }

    if (g_gemm_fusion) return TM_ERR_UNSUPPORTED;  // only the tensor-core kernel folds the norm in
    // One launch covers up to `n_launch` tokens; more tokens than the scratch can hold partial
    // tiles for are processed in several launches over consecutive token ranges.
    const size_t n_out = type == TM_GEMM_FUSED_SILU_FFN ? (size_t)m / 2 : (size_t)m;
    int          n_launch = n;
    for (;;) {
        GemmSmallPlan pl   = gemm_small_plan(m, n_launch, k, h->sm_count, h->max_smem, h->gemv_cols);
        const size_t  c_b  = ((pl.counter_ints * sizeof(int) + 255) / 256) * 256;
        const size_t  need = pl.workspace_floats * sizeof(float) + c_b;
        const bool    fits = workspace ? workspace_bytes >= need :
                                         (pl.workspace_floats * sizeof(float) <= h->scratch_bytes
                                          && pl.counter_ints <= h->counter_ints);
        if (fits) break;
        if (n_launch <= 32) return TM_ERR_WORKSPACE;
        n_launch = ((n_launch / 2 + 31) / 32) * 32;
    }

    for (int t0 = 0; t0 < n; t0 += n_launch) {
        const int     nt = n - t0 < n_launch ? n - t0 : n_launch;
        GemmSmallPlan pl = gemm_small_plan(m, nt, k, h->sm_count, h->max_smem, h->gemv_cols);
        float*        ws_f;
        int*          ws_c;
        if (workspace) {
            // tickets first (they start at zero and reset themselves), 256-byte aligned partials after
            ws_c = (int*)workspace;
            ws_f = (float*)((char*)workspace + ((pl.counter_ints * sizeof(int) + 255) / 256) * 256);
        }
        else {
            ws_f = (float*)h->scratch;
            ws_c = h->counters;
        }
        GemmSmallParams p{};
        p.C          = (__half*)C + (size_t)t0 * n_out;
        p.A          = (const unsigned char*)A;
        p.X          = (const unsigned char*)B + (size_t)t0 * k * 2;
        p.Q          = (const unsigned char*)Q;
        p.workspace  = ws_f;
        p.counters   = ws_c;
        p.status     = h->status;
        p.N          = m;
        p.T          = nt;
        p.K          = k;
        p.fused_silu = type == TM_GEMM_FUSED_SILU_FFN;

        cudaError_t e = gemm_small_launch(pl, p, (cudaStream_t)stream, g_pdl != 0 || h->pdl_direct != 0);
        h->launches += 1;
        if (e != cudaSuccess) {
            h->last_cuda_error = (int)e;
            return TM_ERR_CUDA;
        }
    }
    return TM_OK;
}

int tm_mmha_decode_impl(tm_handle* h, const tm_mmha_params* a, void* stream, int pos_from_length, const int* order,
                        const tmb::MmhaSeqDesc* desc = nullptr, const float2* rope_table = nullptr);

extern "C" int tm_lm_head_f16(tm_handle* h, float* logits, int ld, const void* x, const void* w, int tokens, int vocab, int hidden,
                              void* stream)
{
    if (!h) return TM_ERR_INVALID_ARG;
    if (ld < vocab) return TM_ERR_INVALID_ARG;
    return lm_head_launch(logits, ld, (const __half*)x, (const __half*)w, tokens, vocab, hidden, h->status, h->gemm_wait_cycles,
                          h->max_smem, (cudaStream_t)stream, g_pdl != 0 || h->pdl_direct != 0, &h->launches);
}

extern "C" int tm_mmha_decode(tm_handle* h, const tm_mmha_params* a, void* stream)
{
    return tm_mmha_decode_impl(h, a, stream, 0, nullptr);
}

// pos_from_length: the RoPE position of sequence b is length_per_sample[b] (what the engine's
// timestep - padding evaluates to), so that nothing in the launch depends on the step number.
int tm_mmha_decode_impl(tm_handle* h, const tm_mmha_params* a, void* stream, int pos_from_length, const int* order,
                        const tmb::MmhaSeqDesc* desc, const float2* rope_table)
{
    if (!h || !a) return TM_ERR_INVALID_ARG;
    if (!a->out || !a->q || !a->k || !a->v || !a->length_per_sample || !a->k_cache_per_sample || !a->v_cache_per_sample) {
        return TM_ERR_INVALID_ARG;
    }
    if (a->batch_size <= 0 || a->num_heads <= 0 || a->num_kv_heads <= 0 || a->memory_max_len <= 0 || a->timestep < 0) {
        return TM_ERR_INVALID_ARG;
    }
    if (a->hidden_size_per_head != 128) return TM_ERR_UNSUPPORTED;  // decoder_masked_multihead_attention.cu:28-34
    if (a->num_heads % a->num_kv_heads) return TM_ERR_UNSUPPORTED;
    if (a->rotary_embedding_dim < 0 || a->rotary_embedding_dim > 128 || a->rotary_embedding_dim % 2) return TM_ERR_UNSUPPORTED;
    const bool int8 = (a->int8_mode & 4) != 0;
    if (int8 && !(a->attention_k_scale > 0.f && a->attention_v_scale > 0.f)) return TM_ERR_INVALID_ARG;
    // q, k, v must be the three column blocks of one fused buffer (the only form LLaMA uses)
    const __half* q = (const __half*)a->q;
    if ((const __half*)a->k != q + (size_t)a->num_heads * 128
        || (const __half*)a->v != q + (size_t)(a->num_heads + a->num_kv_heads) * 128) {
        return TM_ERR_UNSUPPORTED;
    }
    if (a->stride < (a->num_heads + 2 * a->num_kv_heads) * 128 || a->stride % 8) return TM_ERR_INVALID_ARG;
    if (((uintptr_t)a->out | (uintptr_t)a->q) & 15u) return TM_ERR_INVALID_ARG;
    const __half* bias = nullptr;
    if (a->q_bias || a->k_bias || a->v_bias) {
        if (!a->q_bias || (const __half*)a->k_bias != (const __half*)a->q_bias + (size_t)a->num_heads * 128
            || (const __half*)a->v_bias != (const __half*)a->q_bias + (size_t)(a->num_heads + a->num_kv_heads) * 128) {
            return TM_ERR_UNSUPPORTED;
        }
        bias = (const __half*)a->q_bias;
    }

    const int max_len = a->timestep < a->memory_max_len ? a->timestep : a->memory_max_len;
    MmhaPlan  pl      = mmha_plan(a->batch_size, a->num_heads, a->num_kv_heads, max_len, h->sm_count, h->mmha_chunk, h->mmha_warps);
    while (pl.ws_floats * sizeof(float) > h->attn_scratch_bytes && pl.chunk < (1 << 20)) {
        pl = mmha_plan(a->batch_size, a->num_heads, a->num_kv_heads, max_len, h->sm_count, pl.chunk * 2, h->mmha_warps);
    }
    if (pl.ws_floats * sizeof(float) > h->attn_scratch_bytes || pl.counter_ints > h->attn_counter_ints) {
        return TM_ERR_WORKSPACE;
    }

    MmhaParams p{};
    p.out             = (__half*)a->out;
    p.qkv             = q;
    p.bias            = bias;
    p.k_cache         = a->k_cache_per_sample;
    p.v_cache         = a->v_cache_per_sample;
    p.cache_offset    = a->kv_cache_per_sample_offset;
    p.lengths         = a->length_per_sample;
    p.finished        = a->finished;
    p.padding         = a->total_padding_tokens;
    p.order           = order;
    p.desc            = desc;
    // the table holds plain rotary coefficients of the cached length: usable when that is the position asked for
    // (and it is laid out in the launch order of `desc`)
    p.rope_table      = (desc && pos_from_length && !a->use_dynamic_ntk && a->rotary_embedding_dim == 128) ? rope_table : nullptr;
    p.B               = a->batch_size;
    p.H               = a->num_heads;
    p.Hkv             = a->num_kv_heads;
    p.stride          = a->stride;
    p.S_max           = a->memory_max_len;
    p.timestep        = a->timestep;
    p.rot_dim         = a->rotary_embedding_dim;
    p.max_pos         = a->max_position_embeddings;
    p.use_dynamic_ntk = a->use_dynamic_ntk;
    p.use_logn        = a->use_logn_attn;
    p.pos_from_length = pos_from_length;
    p.rope_base       = a->rotary_embedding_base > 0.f ? a->rotary_embedding_base : 10000.f;
    p.inv_sqrt_dh     = a->inv_sqrt_dh;
    p.k_scale         = a->attention_k_scale;
    p.k_zp            = a->attention_k_zp;
    p.v_scale         = a->attention_v_scale;
    p.v_zp            = a->attention_v_zp;
    p.ws              = (float*)h->attn_scratch;
    p.counters        = h->attn_counters;
    p.status          = h->status;

    cudaError_t e = mmha_launch(pl, p, int8, (cudaStream_t)stream, g_pdl != 0 || h->pdl_direct != 0);
    h->launches += 1;
    if (e != cudaSuccess) {
        h->last_cuda_error = (int)e;
        return TM_ERR_CUDA;
    }
    return TM_OK;
}

extern "C" int tm_rmsnorm(void* out, const void* in, const void* scale, float eps, int m, int n, void* stream)
{
    if (!out || !in || !scale || m < 0 || n <= 0) return TM_ERR_INVALID_ARG;
    if (n % 8 || n > 16384) return TM_ERR_UNSUPPORTED;
    if (((uintptr_t)out | (uintptr_t)in | (uintptr_t)scale) & 15u) return TM_ERR_INVALID_ARG;
    if (m == 0) return TM_OK;
    return rmsnorm_launch((__half*)out, (const __half*)in, (const __half*)scale, eps, m, n, (cudaStream_t)stream, g_pdl != 0)
                   == cudaSuccess ?
               TM_OK :
               TM_ERR_CUDA;
}

extern "C" int tm_add_residual_rmsnorm(
    void* residual, void* in_out, const void* bias, const void* scale, float eps, int m, int n, void* stream)
{
    if (!residual || !in_out || !scale || m < 0 || n <= 0) return TM_ERR_INVALID_ARG;
    if (n % 8 || n > 16384) return TM_ERR_UNSUPPORTED;
    if (((uintptr_t)residual | (uintptr_t)in_out | (uintptr_t)scale | (uintptr_t)bias) & 15u) return TM_ERR_INVALID_ARG;
    if (m == 0) return TM_OK;
    return add_residual_rmsnorm_launch((__half*)residual, (__half*)in_out, (const __half*)bias, (const __half*)scale, eps,
                                       m, n, (cudaStream_t)stream, g_pdl != 0)
                   == cudaSuccess ?
               TM_OK :
               TM_ERR_CUDA;
}
