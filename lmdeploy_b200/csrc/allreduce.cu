// Tensor-parallel sum over peer memory, fused with the residual add and the RMSNorm that follow it in the decoder
// loop: what the reference does with ftNcclAllReduceSum (src/turbomind/utils/nccl_utils.cc:57-69, call sites
// LlamaDecoderSelfAttentionLayer.cc:292-297, LlamaFfnLayer.cc:106-110) followed by
// invokeFusedAddBiasResidualRMSNorm (llama_decoder_kernels.cu:104-160), in one kernel and without NCCL.
//
// Every rank keeps two slots in a buffer that its peers have mapped (CUDA IPC; one process per GPU).  The row-split
// GEMM (o_proj, w2) writes its partial sums straight into a slot; the kernel here then, per token row,
//   1. tells every peer that this rank's slot is complete (a counter in the peer's memory, release at system scope),
//   2. waits, with a bound, until every peer has said the same (counters in this rank's own memory),
//   3. reads the row from every rank's slot with ordinary 128-bit loads over NVLink, in rank order (the sum is the
//      same on every rank and from run to run), rounds it to fp16 like the all-reduce it replaces,
//   4. adds the residual, stores it, normalises and stores the input of the next GEMM.
// With more than two ranks the rows are dealt to the ranks instead (allreduce_rows_kernel): the owner of a row does
// steps 1-4 for it, parks the normalised row in a third mapped buffer and raises a per-row counter in every peer's
// memory; the other ranks wait for that counter and fetch the finished row.  Every rank then reads (w - 1) / w of the
// tensor twice instead of (w - 1) times, and the residual is only ever touched by the owner of a row.
// Nothing is multicast and no rank writes another rank's data: peers only ever write each other's counters.
// The two slots alternate (o_proj -> 0, w2 -> 1).  A rank overwrites a slot two calls after its peers read it: by then
// it has itself passed the wait of the call in between, for which every peer had to finish the earlier one first.
// A wait that runs out sets a status bit and lets the kernel finish (on garbage): nothing here can hang.
#include "comm.h"
#include "common.cuh"
#include "tm_b200.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace tmb {
namespace {

constexpr int kArThreadsMax = 1024;

struct ArParams {
    const unsigned char* slot[kMaxP2pRanks];   // this call's slot of every rank (own rank: local address)
    unsigned*            peer_flags[kMaxP2pRanks];  // counter array of every rank; this rank writes entry [rank]
    unsigned*            my_flags;             // this rank's counter array: entry [j] is written by rank j
    unsigned*            state;                // [0] calls completed, [1] CTAs finished in the current call
    __half*              residual;             // [m, n] updated in place
    __half*              out;                  // [m, n] normalised rows
    const __half*        scale;                // [n]
    unsigned*            status;
    long long            max_wait_cycles;
    float                eps;
    int                  n, world, rank;
    // row-owner variant
    unsigned char*       h_slot[kMaxP2pRanks];     // finished rows of every rank (own rank: local address)
    unsigned*            row_flags[kMaxP2pRanks];  // per-row counters of every rank; the owner of a row writes them all
    unsigned*            my_row_flags;
    int                  rows_per_rank;
    int                  bulk;                     // 1: the peers' rows are staged in shared memory by bulk copies
};

// Shared memory of the bulk path: an mbarrier, then one row per other rank.
constexpr int kArStageOff = 128;

// One bulk copy (global -> shared, completion counted on an mbarrier): the copy engine keeps far more of a peer's memory
// in flight over NVLink than the 16-byte loads of a CTA's threads can.  No multicast; source and destination 16-byte aligned.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ uint4 ld_peer(const unsigned char* p)
{
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kArThreadsMax) allreduce_add_rmsnorm_kernel(ArParams p)
{
    extern __shared__ __align__(128) unsigned char ar_smem[];
    __shared__ float    red[kArThreadsMax / 32];
    __shared__ unsigned s_epoch;
    const int tid = threadIdx.x;
    uint64_t* stage_bar = reinterpret_cast<uint64_t*>(ar_smem);
    if (p.bulk && tid == 0) {
        mbar_init(stage_bar, 1);
        fence_mbar_init();
    }
    pdl_wait();  // the slot is written by the GEMM before this kernel
    pdl_launch_dependents();
    if (tid == 0) s_epoch = *(volatile unsigned*)&p.state[0] + 1u;
    __syncthreads();
    const unsigned epoch = s_epoch;
    if (blockIdx.x == 0 && tid < p.world && tid != p.rank) {
        // this rank's slot is complete (the GEMM's grid has finished): publish that to peer `tid`
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.peer_flags[tid] + p.rank), "r"(epoch) : "memory");
    }
    if (tid < p.world && tid != p.rank) {
        const long long t0 = clock64();
        unsigned        seen;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.my_flags + tid) : "memory");
            if ((int)(seen - epoch) >= 0) break;
            if (clock64() - t0 > p.max_wait_cycles) {
                atomicOr(p.status, kStatusCommWait);
                break;
            }
            __nanosleep(40);
        }
    }
    __syncthreads();

    const size_t row  = (size_t)blockIdx.x * p.n;
    const int    nvec = p.n / 8;
    float        ss   = 0.f;
    if (p.bulk) {
        // the other ranks' pieces of this row come to shared memory with one bulk copy each
        const uint32_t row_bytes = (uint32_t)p.n * 2;
        if (tid == 0) {
            asm volatile("fence.proxy.async;" ::: "memory");  // the counters were read through the generic proxy
            mbar_arrive_expect_tx(stage_bar, row_bytes * (uint32_t)(p.world - 1));
            for (int j = 0; j < p.world; ++j) {
                if (j == p.rank) continue;
                const int idx = j < p.rank ? j : j - 1;
                bulk_g2s(smem_u32(ar_smem + kArStageOff) + (uint32_t)idx * row_bytes, p.slot[j] + row * 2, row_bytes, stage_bar);
            }
        }
        if (!mbar_wait(stage_bar, 0, p.max_wait_cycles)) atomicOr(p.status, kStatusCommWait);
    }
    // sum of one 16-byte piece of the row over the ranks (their loads in flight together) + residual -> fp16 piece
    auto reduce_piece = [&](int v) {
        uint4 part[kMaxP2pRanks];
#pragma unroll
        for (int j = 0; j < kMaxP2pRanks; ++j) {
            if (j < p.world) {
                if (p.bulk && j != p.rank) {
                    part[j] = *reinterpret_cast<const uint4*>(ar_smem + kArStageOff + (size_t)(j < p.rank ? j : j - 1) * p.n * 2 + (size_t)v * 16);
                }
                else {
                    part[j] = ld_peer(p.slot[j] + (row + (size_t)v * 8) * 2);
                }
            }
        }
        uint4 r = reinterpret_cast<const uint4*>(p.residual + row)[v];
        float sum[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) sum[e] = 0.f;
#pragma unroll
        for (int j = 0; j < kMaxP2pRanks; ++j) {
            if (j < p.world) {
                const __half2* h = reinterpret_cast<const __half2*>(&part[j]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(h[e]);
                    sum[2 * e] += f.x, sum[2 * e + 1] += f.y;
                }
            }
        }
        __half2* rh = reinterpret_cast<__half2*>(&r);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            // the all-reduce result is an fp16 tensor; then r = a + b in fp32, stored as fp16 (llama_decoder_kernels.cu:52-57)
            const float2 x = __half22float2(__floats2half2_rn(sum[2 * e], sum[2 * e + 1]));
            const float2 a = __half22float2(rh[e]);
            const float2 t = make_float2(a.x + x.x, a.y + x.y);
            ss += t.x * t.x + t.y * t.y;
            rh[e] = __float22half2_rn(t);
        }
        reinterpret_cast<uint4*>(p.residual + row)[v] = r;
        return r;
    };
    auto scaled = [&](uint4 o, int v, float inv) {
        const uint4    s  = reinterpret_cast<const uint4*>(p.scale)[v];
        const __half2* sh = reinterpret_cast<const __half2*>(&s);
        __half2*       oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 a = __half22float2(oh[e]), w = __half22float2(sh[e]);
            oh[e]          = __float22half2_rn(make_float2(a.x * w.x * inv, a.y * w.y * inv));  // llama_decoder_kernels.cu:58-61
        }
        return o;
    };
    auto block_total = [&]() {
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
        if ((tid & 31) == 0) red[tid >> 5] = ss;
        __syncthreads();
        float t = 0.f;
        for (int w = 0; w < (int)(blockDim.x + 31) / 32; ++w) t += red[w];
        return t;
    };
    if (nvec <= (int)blockDim.x) {
        // one piece per thread (rows up to 8192 features): the piece stays in registers across the reduction
        uint4 mine = make_uint4(0, 0, 0, 0);
        if (tid < nvec) mine = reduce_piece(tid);
        const float inv = rsqrtf(block_total() / (float)p.n + p.eps);
        if (tid < nvec) reinterpret_cast<uint4*>(p.out + row)[tid] = scaled(mine, tid, inv);
    }
    else {
        // wider rows: the pieces are parked in `out` and scaled in a second sweep
        for (int v = tid; v < nvec; v += blockDim.x) reinterpret_cast<uint4*>(p.out + row)[v] = reduce_piece(v);
        const float inv = rsqrtf(block_total() / (float)p.n + p.eps);
        for (int v = tid; v < nvec; v += blockDim.x) {
            reinterpret_cast<uint4*>(p.out + row)[v] = scaled(reinterpret_cast<const uint4*>(p.out + row)[v], v, inv);
        }
    }
    // the last CTA of the call closes it: the next call waits for the next count
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&p.state[1], 1u) == gridDim.x - 1) {
            p.state[1] = 0u;
            __threadfence();
            *(volatile unsigned*)&p.state[0] = epoch;
        }
    }
}


// Row-owner variant (more than two ranks).  One CTA per token row on every rank.  Row t belongs to rank t / rows_per_rank.
__global__ void __launch_bounds__(kArThreadsMax) allreduce_rows_kernel(ArParams p)
{
    extern __shared__ __align__(128) unsigned char ar_smem[];
    __shared__ float    red[kArThreadsMax / 32];
    __shared__ unsigned s_epoch;
    const int tid = threadIdx.x;
    uint64_t* stage_bar = reinterpret_cast<uint64_t*>(ar_smem);
    if (p.bulk && tid == 0) {
        mbar_init(stage_bar, 1);
        fence_mbar_init();
    }
    pdl_wait();  // the slot is written by the GEMM before this kernel
    pdl_launch_dependents();
    if (tid == 0) s_epoch = *(volatile unsigned*)&p.state[0] + 1u;
    __syncthreads();
    const unsigned epoch = s_epoch;
    if (blockIdx.x == 0 && tid < p.world && tid != p.rank) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.peer_flags[tid] + p.rank), "r"(epoch) : "memory");
    }
    const int    t     = blockIdx.x;
    const int    owner = min(t / p.rows_per_rank, p.world - 1);
    const size_t row   = (size_t)t * p.n;
    const int    nvec  = p.n / 8;
    auto bounded_wait = [&](const unsigned* flag) {
        const long long t0 = clock64();
        unsigned        seen;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
            if ((int)(seen - epoch) >= 0) break;
            if (clock64() - t0 > p.max_wait_cycles) {
                atomicOr(p.status, kStatusCommWait);
                break;
            }
            __nanosleep(40);
        }
    };
    if (owner == p.rank) {
        // ---- this rank finishes the row: partial sums of every rank -> residual -> normalised row
        if (tid < p.world && tid != p.rank) bounded_wait(p.my_flags + tid);
        __syncthreads();
        float ss = 0.f;
        if (p.bulk) {
            const uint32_t row_bytes = (uint32_t)p.n * 2;
            if (tid == 0) {
                asm volatile("fence.proxy.async;" ::: "memory");
                mbar_arrive_expect_tx(stage_bar, row_bytes * (uint32_t)(p.world - 1));
                for (int j = 0; j < p.world; ++j) {
                    if (j == p.rank) continue;
                    const int idx = j < p.rank ? j : j - 1;
                    bulk_g2s(smem_u32(ar_smem + kArStageOff) + (uint32_t)idx * row_bytes, p.slot[j] + row * 2, row_bytes, stage_bar);
                }
            }
            if (!mbar_wait(stage_bar, 0, p.max_wait_cycles)) atomicOr(p.status, kStatusCommWait);
        }
        auto reduce_piece = [&](int v) {
            uint4 part[kMaxP2pRanks];
#pragma unroll
            for (int j = 0; j < kMaxP2pRanks; ++j) {
                if (j < p.world) {
                    if (p.bulk && j != p.rank) {
                        part[j] = *reinterpret_cast<const uint4*>(ar_smem + kArStageOff + (size_t)(j < p.rank ? j : j - 1) * p.n * 2 + (size_t)v * 16);
                    }
                    else {
                        part[j] = ld_peer(p.slot[j] + (row + (size_t)v * 8) * 2);
                    }
                }
            }
            uint4 r = reinterpret_cast<const uint4*>(p.residual + row)[v];
            float sum[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) sum[e] = 0.f;
#pragma unroll
            for (int j = 0; j < kMaxP2pRanks; ++j) {
                if (j < p.world) {
                    const __half2* h = reinterpret_cast<const __half2*>(&part[j]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = __half22float2(h[e]);
                        sum[2 * e] += f.x, sum[2 * e + 1] += f.y;
                    }
                }
            }
            __half2* rh = reinterpret_cast<__half2*>(&r);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 x = __half22float2(__floats2half2_rn(sum[2 * e], sum[2 * e + 1]));
                const float2 a = __half22float2(rh[e]);
                const float2 u = make_float2(a.x + x.x, a.y + x.y);
                ss += u.x * u.x + u.y * u.y;
                rh[e] = __float22half2_rn(u);
            }
            reinterpret_cast<uint4*>(p.residual + row)[v] = r;
            return r;
        };
        auto scaled = [&](uint4 o, int v, float inv) {
            const uint4    sc = reinterpret_cast<const uint4*>(p.scale)[v];
            const __half2* sh = reinterpret_cast<const __half2*>(&sc);
            __half2*       oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 a = __half22float2(oh[e]), w = __half22float2(sh[e]);
                oh[e]          = __float22half2_rn(make_float2(a.x * w.x * inv, a.y * w.y * inv));
            }
            return o;
        };
        auto block_total = [&]() {
#pragma unroll
            for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
            if ((tid & 31) == 0) red[tid >> 5] = ss;
            __syncthreads();
            float tot = 0.f;
            for (int w = 0; w < (int)(blockDim.x + 31) / 32; ++w) tot += red[w];
            return tot;
        };
        uint4* mine_h = reinterpret_cast<uint4*>(p.h_slot[p.rank] + row * 2);
        if (nvec <= (int)blockDim.x) {
            uint4 piece = make_uint4(0, 0, 0, 0);
            if (tid < nvec) piece = reduce_piece(tid);
            const float inv = rsqrtf(block_total() / (float)p.n + p.eps);
            if (tid < nvec) {
                const uint4 o = scaled(piece, tid, inv);
                reinterpret_cast<uint4*>(p.out + row)[tid] = o;
                mine_h[tid]                                = o;
            }
        }
        else {
            for (int v = tid; v < nvec; v += blockDim.x) reinterpret_cast<uint4*>(p.out + row)[v] = reduce_piece(v);
            const float inv = rsqrtf(block_total() / (float)p.n + p.eps);
            for (int v = tid; v < nvec; v += blockDim.x) {
                const uint4 o = scaled(reinterpret_cast<const uint4*>(p.out + row)[v], v, inv);
                reinterpret_cast<uint4*>(p.out + row)[v] = o;
                mine_h[v]                                = o;
            }
        }
        // the finished row is in this rank's mapped buffer: tell every peer (the barrier orders every thread's stores
        // before the fence of the threads that raise the counters)
        __syncthreads();
        if (tid < p.world && tid != p.rank) {
            __threadfence_system();
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.row_flags[tid] + t), "r"(epoch) : "memory");
        }
    }
    else {
        // ---- another rank finishes the row: wait for its counter, fetch the row
        if (tid == 0) bounded_wait(p.my_row_flags + t);
        __syncthreads();
        const unsigned char* src = p.h_slot[owner] + row * 2;
        if (p.bulk) {
            const uint32_t row_bytes = (uint32_t)p.n * 2;
            if (tid == 0) {
                asm volatile("fence.proxy.async;" ::: "memory");
                mbar_arrive_expect_tx(stage_bar, row_bytes);
                bulk_g2s(smem_u32(ar_smem + kArStageOff), src, row_bytes, stage_bar);
            }
            if (!mbar_wait(stage_bar, 0, p.max_wait_cycles)) atomicOr(p.status, kStatusCommWait);
            for (int v = tid; v < nvec; v += blockDim.x) {
                reinterpret_cast<uint4*>(p.out + row)[v] = *reinterpret_cast<const uint4*>(ar_smem + kArStageOff + (size_t)v * 16);
            }
        }
        else {
            for (int v = tid; v < nvec; v += blockDim.x) reinterpret_cast<uint4*>(p.out + row)[v] = ld_peer(src + (size_t)v * 16);
        }
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&p.state[1], 1u) == gridDim.x - 1) {
            p.state[1] = 0u;
            __threadfence();
            *(volatile unsigned*)&p.state[0] = epoch;
        }
    }
}

}  // namespace

// layout of a rank's exported region: [0, 1 KB) counters written by the peers | [1 KB, 2 KB) own call state |
// [2 KB, 8 KB) per-row counters written by the row owners | partial-sum slots 0, 1 | finished rows
constexpr size_t kP2pRowFlags = 2048;
constexpr int    kP2pMaxRows  = 1536;
constexpr size_t kP2pHeader   = 8192;

cudaError_t allreduce_add_rmsnorm_launch(tm_comm* c, int slot, __half* residual, __half* out, const __half* scale, float eps, int m,
                                         int n, unsigned* status, cudaStream_t st, bool pdl)
{
    ArParams p{};
    for (int j = 0; j < c->world; ++j) {
        unsigned char* base = (unsigned char*)(j == c->rank ? c->p2p_local : c->p2p_peer[j]);
        p.slot[j]           = base + kP2pHeader + (size_t)slot * c->p2p_slot_bytes;
        p.peer_flags[j]     = (unsigned*)base;
    }
    p.my_flags        = (unsigned*)c->p2p_local;
    p.state           = (unsigned*)((unsigned char*)c->p2p_local + 1024);
    p.residual        = residual;
    p.out             = out;
    p.scale           = scale;
    p.status          = status;
    p.max_wait_cycles = c->p2p_wait_cycles > 0 ? c->p2p_wait_cycles : kMaxWaitCycles;
    p.eps             = eps;
    p.n               = n;
    p.world           = c->world;
    p.rank            = c->rank;
    for (int j = 0; j < c->world; ++j) {
        unsigned char* base = (unsigned char*)(j == c->rank ? c->p2p_local : c->p2p_peer[j]);
        p.h_slot[j]         = base + kP2pHeader + 2 * c->p2p_slot_bytes;
        p.row_flags[j]      = (unsigned*)(base + kP2pRowFlags);
    }
    p.my_row_flags  = (unsigned*)((unsigned char*)c->p2p_local + kP2pRowFlags);
    p.rows_per_rank = (m + c->world - 1) / c->world;
    int threads = n / 8;
    if (threads > kArThreadsMax) threads = kArThreadsMax;
    threads = (threads + 31) / 32 * 32;
    // rows dealt to owners read less over the links but hand every row over once more: measured slower at 4 ranks
    // (14.7 against 13.6 ms per 70B decode step) and faster at 8 (13.0 against 14.0 ms)
    const bool rows = (c->p2p_mode == 2 || (c->p2p_mode == 0 && c->world > 4)) && m <= kP2pMaxRows;
    // the peers' rows through the copy engine when they fit shared memory (one row of n halves per other rank)
    const size_t stage = kArStageOff + (size_t)(c->world - 1) * n * 2;
    // measured on 70B decode steps: no gain at two ranks (17.9 vs 18.0 ms), 13.1 -> 12.7 ms at eight
    const bool want    = c->p2p_bulk < 0 ? c->world > 2 : c->p2p_bulk != 0;
    p.bulk             = want && stage <= 200u * 1024u ? 1 : 0;
    const size_t smem  = p.bulk ? stage : 0;
    auto kernel        = rows ? allreduce_rows_kernel : allreduce_add_rmsnorm_kernel;
    if (smem > 48u * 1024u && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        return cudaErrorInvalidValue;
    }
    return launch_kernel(kernel, dim3(m), dim3(threads), smem, st, pdl, p);
}

}  // namespace tmb

using namespace tmb;

extern "C" int tm_comm_p2p_export(tm_comm* c, size_t slot_bytes, void* handle64)
{
    if (!c || !handle64 || slot_bytes == 0) return TM_ERR_INVALID_ARG;
    if (c->world > kMaxP2pRanks) return TM_ERR_UNSUPPORTED;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (c->p2p_local) return TM_ERR_INVALID_ARG;  // once per communicator
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(c->device);
    slot_bytes         = (slot_bytes + 255) / 256 * 256;
    const size_t bytes = kP2pHeader + 3 * slot_bytes;
    cudaError_t  e     = cudaMalloc(&c->p2p_local, bytes);
    if (e == cudaSuccess) e = cudaMemset(c->p2p_local, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, c->p2p_local);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaSetDevice(prev);
    if (e != cudaSuccess) return TM_ERR_CUDA;
    c->p2p_slot_bytes = slot_bytes;
    if (const char* e = std::getenv("TM_B200_P2P_MODE")) c->p2p_mode = std::max(0, std::min(2, std::atoi(e)));
    if (const char* e = std::getenv("TM_B200_P2P_BULK")) c->p2p_bulk = std::atoi(e) != 0;
    std::memcpy(handle64, &h, 64);
    return TM_OK;
}

extern "C" int tm_comm_p2p_import(tm_comm* c, const void* handles)
{
    if (!c || !handles || !c->p2p_local) return TM_ERR_INVALID_ARG;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(c->device);
    int rc = TM_OK;
    for (int j = 0; j < c->world && rc == TM_OK; ++j) {
        if (j == c->rank) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, (const unsigned char*)handles + (size_t)j * 64, 64);
        if (cudaIpcOpenMemHandle(&c->p2p_peer[j], h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) rc = TM_ERR_CUDA;
    }
    cudaSetDevice(prev);
    if (rc == TM_OK) c->p2p_ready = 1;
    return rc;
}

extern "C" int tm_comm_set_option(tm_comm* c, const char* name, long long value)
{
    if (!c || !name) return TM_ERR_INVALID_ARG;
    if (std::strcmp(name, "p2p_bulk") == 0 && value >= -1 && value <= 1) {
        c->p2p_bulk = (int)value;  // 1: peers' rows staged in shared memory by bulk copies; 0: 16-byte loads; -1: by world size
        return TM_OK;
    }
    if (std::strcmp(name, "p2p_mode") == 0 && value >= 0 && value <= 2) {
        c->p2p_mode = (int)value;  // 0 automatic, 1 every rank reads every slot, 2 rows dealt to owners
        return TM_OK;
    }
    if (std::strcmp(name, "p2p_wait_cycles") == 0 && value >= 0) {
        c->p2p_wait_cycles = value;  // bound of the wait for the peers' slots, SM clock cycles; 0 = default
        return TM_OK;
    }
    return TM_ERR_INVALID_ARG;
}

extern "C" void* tm_comm_p2p_slot(tm_comm* c, int slot)
{
    if (!c || !c->p2p_ready || slot < 0 || slot > 1) return nullptr;
    return (unsigned char*)c->p2p_local + kP2pHeader + (size_t)slot * c->p2p_slot_bytes;
}

extern "C" size_t tm_comm_p2p_slot_bytes(const tm_comm* c)
{
    return c && c->p2p_ready ? c->p2p_slot_bytes : 0;
}

extern "C" int tm_allreduce_add_residual_rmsnorm(tm_comm* c, int slot, void* residual, void* out, const void* scale, float eps, int m,
                                                 int n, unsigned* status_word, void* stream)
{
    if (!c || !residual || !out || !scale || !status_word || m < 0 || n <= 0 || slot < 0 || slot > 1) return TM_ERR_INVALID_ARG;
    if (!c->p2p_ready) return TM_ERR_NOT_BUILT;
    if (n % 8 || n > 16384) return TM_ERR_UNSUPPORTED;
    if ((size_t)m * n * 2 > c->p2p_slot_bytes) return TM_ERR_WORKSPACE;
    if (m == 0) return TM_OK;
    return allreduce_add_rmsnorm_launch(c, slot, (__half*)residual, (__half*)out, (const __half*)scale, eps, m, n, status_word,
                                        (cudaStream_t)stream, false)
                   == cudaSuccess ?
               TM_OK :
               TM_ERR_CUDA;
}
