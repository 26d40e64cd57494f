// C ABI: handle management and the GEMM entry point.
#include "handle.h"
#include "tm_b200.h"

#include <cstdlib>
#include <cstring>
#include <new>

using namespace tmb;

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
        h->scratch_bytes = 64u << 20;
        h->counter_ints  = 1u << 16;
        e                = cudaMalloc(&h->scratch, h->scratch_bytes);
    }
    if (e == cudaSuccess) e = cudaMalloc(&h->counters, h->counter_ints * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(h->counters, 0, h->counter_ints * sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&h->status, 256);
    if (e == cudaSuccess) e = cudaMemset(h->status, 0, 256);
    if (e == cudaSuccess) e = gemm_small_prepare(h->max_smem);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    h->gemv_stages = env_int("TM_B200_GEMV_STAGES", 0);
    h->gemv_groups = env_int("TM_B200_GEMV_GROUPS", 0);
    cudaSetDevice(prev);
    if (e != cudaSuccess) {
        h->last_cuda_error = (int)e;
        tm_destroy(h);
        return TM_ERR_CUDA;
    }
    *out = h;
    return TM_OK;
}

extern "C" int tm_destroy(tm_handle* h)
{
    if (!h) return TM_OK;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(h->device);
    if (h->scratch) cudaFree(h->scratch);
    if (h->counters) cudaFree(h->counters);
    if (h->status) cudaFree(h->status);
    cudaSetDevice(prev);
    delete h;
    return TM_OK;
}

extern "C" int tm_last_cuda_error(const tm_handle* h)
{
    return h ? h->last_cuda_error : 0;
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
    GemmSmallPlan pl = gemm_small_plan(m, n, k, 256, 227 * 1024, 0, 0);
    return pl.workspace_floats * sizeof(float) + pl.counter_ints * sizeof(int) + 256;
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

    GemmSmallPlan pl = gemm_small_plan(m, n, k, h->sm_count, h->max_smem, h->gemv_stages, h->gemv_groups);

    float* ws_f = nullptr;
    int*   ws_c = nullptr;
    if (workspace) {
        const size_t need = pl.workspace_floats * sizeof(float) + pl.counter_ints * sizeof(int) + 256;
        if (workspace_bytes < need) return TM_ERR_WORKSPACE;
        // counters first (they must start at zero and reset themselves), 256-byte aligned partials after
        ws_c = (int*)workspace;
        ws_f = (float*)((char*)workspace + ((pl.counter_ints * sizeof(int) + 255) / 256) * 256);
    }
    else {
        if (pl.workspace_floats * sizeof(float) > h->scratch_bytes || pl.counter_ints > h->counter_ints) {
            return TM_ERR_WORKSPACE;
        }
        ws_f = (float*)h->scratch;
        ws_c = h->counters;
    }

    GemmSmallParams p{};
    p.C          = (__half*)C;
    p.A          = (const unsigned char*)A;
    p.X          = (const unsigned char*)B;
    p.Q          = (const unsigned char*)Q;
    p.workspace  = ws_f;
    p.counters   = ws_c;
    p.status     = h->status;
    p.N          = m;
    p.T          = n;
    p.K          = k;
    p.fused_silu = type == TM_GEMM_FUSED_SILU_FFN;

    cudaError_t e = gemm_small_launch(pl, p, (cudaStream_t)stream);
    h->launches += 1;
    if (e != cudaSuccess) {
        h->last_cuda_error = (int)e;
        return TM_ERR_CUDA;
    }
    return TM_OK;
}
