// W4A16 GEMM for small token counts (the HBM-bound regime): a persistent, stream-K balanced
// kernel.  A few producer lanes stream the packed int4 weight (one contiguous 8 KB run per copy:
// 32 input rows x 512 output columns) and the {zero, scale} rows through a ring of
// shared-memory stages with bulk copies (TMA, mbarrier completion).  Sixteen consumer warps, one
// per 32-column tile, unpack nibbles with lop3, subtract the zero point exactly in fp16, feed the
// integers to mma.m16n8k16 (the runtime int4 layout IS that instruction's A fragment; the
// activations come straight from L1/L2 as B fragments) and apply the group scale to the fp32
// group sums.  K is split across CTAs (every CTA gets the same number of 32x512 weight units);
// partial tiles meet in a scratch buffer and the last CTA to arrive for a column tile reduces
// them in a fixed order, so the result is deterministic and no CTA ever waits for another.
//
// Replaces the small-n end of GemmS4F16::Run (src/turbomind/kernels/gemm_s_f16/
// gemm_s4_f16.cu:208-234) / gemm_s4_f16_nn (gemm_template.h:338-444), whose smallest token
// tile is 8 and which has no split-K across CTAs.
#include "common.cuh"
#include "gemm_s4_f16.h"
#include "tm_b200.h"

#include <mutex>

namespace tmb {

namespace {

constexpr int kColsPerTile   = 32;   // one packed 32x32 tile = 512 B
constexpr int kTileBytes     = 512;
constexpr int kTilesPerUnit  = 16;   // column tiles per unit: one contiguous 8 KB run of the packed weight
constexpr int kUnitCols      = kColsPerTile * kTilesPerUnit;  // 512
constexpr int kWBytes        = kTilesPerUnit * kTileBytes;    // 8192
constexpr int kQBytes        = kUnitCols * 4;                 // 2048
constexpr int kStageBytes    = kWBytes + kQBytes;
constexpr int kConsumers     = kTilesPerUnit;                 // one consumer warp per column tile
constexpr int kConsThreads   = kConsumers * 32;
constexpr int kProducerLanes = 4;                             // lanes of warp 0 that issue bulk copies

// dynamic shared memory: [stages][kStageBytes] | full[stages] | empty[stages] | flag

// B fragments (activations) of one 32-row slab for NT token tiles, straight from global memory.
template<int NT>
__device__ __forceinline__ void
load_x_frags(uint32_t (&bf)[NT][4], const unsigned char* X, int K, int T, int t0, int k32, int r, int c)
{
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int t = t0 + j * 8 + r;
        if (t < T) {
            const uint32_t* xr = reinterpret_cast<const uint32_t*>(X + ((size_t)t * K + (size_t)k32 * 32) * 2) + c;
            bf[j][0]           = __ldg(xr);
            bf[j][1]           = __ldg(xr + 4);
            bf[j][2]           = __ldg(xr + 8);
            bf[j][3]           = __ldg(xr + 12);
        }
        else {
            bf[j][0] = bf[j][1] = bf[j][2] = bf[j][3] = 0u;
        }
    }
}

template<int NT>
__global__ void __launch_bounds__(32 + kConsThreads, 1) gemm_s4_f16_small_kernel(GemmSmallParams p)
{
    constexpr int TP = NT * 8;
    extern __shared__ __align__(128) unsigned char smem_raw[];

    const int stages = p.stages;

    unsigned char* stage_base = smem_raw;
    uint64_t*      full_bar   = reinterpret_cast<uint64_t*>(smem_raw + (size_t)stages * kStageBytes);
    uint64_t*      empty_bar  = full_bar + stages;
    int*           s_flag     = reinterpret_cast<int*>(empty_bar + stages);

    const int tid  = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    // token chunk handled by this CTA row
    const int t0     = blockIdx.y * TP;
    const int t_rows = min(TP, p.T - t0);

    const int G32       = p.K / 32;  // units (32-row slabs) per column tile
    const int upc       = p.units_per_cta;
    const int u_begin   = blockIdx.x * upc;
    const int u_end     = min(u_begin + upc, p.total_units);
    const int n_units   = u_end - u_begin;
    const int n_tiles32 = p.N / kColsPerTile;

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kConsumers);
        }
        fence_mbar_init();
    }
    __syncthreads();

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        // lane l issues the copies of units l, l + kProducerLanes, ...: several copies are being
        // issued at any time, each a single contiguous run of up to 8 KB.
        if (lane < kProducerLanes) {
            const uint64_t pol_w  = policy_evict_first();
            bool           dead   = false;
            int            issued = -1;
            for (int it = lane; it < n_units && !dead; it += kProducerLanes) {
                const int s = it % stages;
                if (it >= stages) {
                    if (!mbar_wait(&empty_bar[s], ((it / stages) - 1) & 1)) {
                        atomicOr(p.status, kStatusGemvEmptyWait);
                        dead = true;
                        break;
                    }
                }
                const int  u      = u_begin + it;
                const int  jt     = u / G32;
                const int  k32    = u - jt * G32;
                const int  tile0  = jt * kTilesPerUnit;
                const int  ntw    = min(kTilesPerUnit, n_tiles32 - tile0);
                const bool need_q = (it == 0) || ((k32 & 3) == 0);

                unsigned char* sb = stage_base + (size_t)s * kStageBytes;
                const uint32_t tx = (uint32_t)(ntw * kTileBytes + (need_q ? ntw * kColsPerTile * 4 : 0));
                mbar_arrive_expect_tx(&full_bar[s], tx);
                bulk_g2s_hint(sb,
                              p.A + ((size_t)k32 * n_tiles32 + tile0) * kTileBytes,
                              (uint32_t)(ntw * kTileBytes),
                              &full_bar[s],
                              pol_w);
                if (need_q) {
                    bulk_g2s_hint(sb + kWBytes,
                                  p.Q + ((size_t)(k32 >> 2) * p.N + (size_t)tile0 * kColsPerTile) * 4,
                                  (uint32_t)(ntw * kColsPerTile * 4),
                                  &full_bar[s],
                                  pol_w);
                }
                issued = it;
            }
            if (dead) {
                // consumers may have stopped too: make sure none of this lane's copies is still
                // in flight towards this CTA's shared memory before the CTA can retire.
                for (int j = issued; j >= 0 && j > issued - stages; j -= kProducerLanes) {
                    (void)mbar_wait(&full_bar[j % stages], (j / stages) & 1);
                }
            }
        }
    }
    else {
        // ------------------------------------------------------------------ consumers
        const int wt   = warp - 1;   // column tile inside the unit
        const int r    = lane >> 2;  // fragment row
        const int c    = lane & 3;   // fragment column pair
        const int ctid = tid - 32;
        bool      dead = false;

        float tot[2][NT][4];
        float acc[2][NT][4];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    tot[a][j][i] = 0.f;
                    acc[a][j][i] = 0.f;
                }

        uint32_t z1024[2] = {0u, 0u}, nz64[2] = {0u, 0u};
        float    sc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};

        // with few token tiles the next unit's activations are requested one unit ahead
        constexpr bool kPrefetchX = NT <= 2;
        uint32_t       bf[NT][4];
        if (kPrefetchX && n_units > 0) {
            load_x_frags<NT>(bf, p.X, p.K, p.T, t0, u_begin % G32, r, c);
        }

        for (int it = 0; it < n_units; ++it) {
            const int  u       = u_begin + it;
            const int  jt      = u / G32;
            const int  k32     = u - jt * G32;
            const int  tile0   = jt * kTilesPerUnit;
            const int  ntw     = min(kTilesPerUnit, n_tiles32 - tile0);
            const bool need_q  = (it == 0) || ((k32 & 3) == 0);
            const bool last    = (it == n_units - 1);
            const bool seg_end = last || (k32 == G32 - 1);
            const bool grp_end = seg_end || ((k32 & 3) == 3);
            const int  s       = it % stages;

            // activations of the next unit: requested before this unit's math
            uint32_t bn[kPrefetchX ? NT : 1][4];
            if constexpr (kPrefetchX) {
                if (!last) {
                    load_x_frags<NT>(bn, p.X, p.K, p.T, t0, (u + 1) % G32, r, c);
                }
            }
            else {
                load_x_frags<NT>(bf, p.X, p.K, p.T, t0, k32, r, c);
            }

            if (!dead) {
                // the verdict is made warp-uniform: the shuffles below need every lane
                const bool ok = mbar_wait(&full_bar[s], (it / stages) & 1);
                if (!__all_sync(0xffffffffu, ok)) {
                    if (lane == 0) atomicOr(p.status, kStatusGemvFullWait);
                    dead = true;
                }
            }
            if (!dead && wt < ntw) {
                const unsigned char* sb = stage_base + (size_t)s * kStageBytes;
                if (need_q) {
                    // {64+z, s} of the four rows this lane owns: n16 in {0,1} x {r, r+8}
                    const __half2* qs = reinterpret_cast<const __half2*>(sb + kWBytes) + wt * kColsPerTile;
#pragma unroll
                    for (int a = 0; a < 2; ++a) {
                        const __half2 q_lo = qs[a * 16 + r];
                        const __half2 q_hi = qs[a * 16 + r + 8];
                        const __half2 zl2  = __half2half2(__hadd(__low2half(q_lo), __float2half_rn(960.f)));
                        const __half2 zh2  = __half2half2(__hneg(__low2half(q_hi)));
                        z1024[a]           = reinterpret_cast<const uint32_t&>(zl2);
                        nz64[a]            = reinterpret_cast<const uint32_t&>(zh2);
                        sc[a][0]           = __high2float(q_lo);
                        sc[a][1]           = __high2float(q_hi);
                    }
                }
                const uint4    w     = reinterpret_cast<const uint4*>(sb)[wt * 32 + lane];
                const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) {
                    const int k16 = wi >> 1;
                    const int a   = wi & 1;
                    uint32_t  af[4];
                    unpack_s4_minus_zero(wv[wi], z1024[a], nz64[a], af);
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        mma_m16n8k16(acc[a][j], af, bf[j][2 * k16], bf[j][2 * k16 + 1]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0 && !dead) {
                mbar_arrive(&empty_bar[s]);
            }
            if (grp_end) {
#pragma unroll
                for (int a = 0; a < 2; ++a)
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        tot[a][j][0] = fmaf(sc[a][0], acc[a][j][0], tot[a][j][0]);
                        tot[a][j][1] = fmaf(sc[a][0], acc[a][j][1], tot[a][j][1]);
                        tot[a][j][2] = fmaf(sc[a][1], acc[a][j][2], tot[a][j][2]);
                        tot[a][j][3] = fmaf(sc[a][1], acc[a][j][3], tot[a][j][3]);
                        acc[a][j][0] = acc[a][j][1] = acc[a][j][2] = acc[a][j][3] = 0.f;
                    }
            }
            if constexpr (kPrefetchX) {
                if (!last) {
#pragma unroll
                    for (int j = 0; j < NT; ++j)
#pragma unroll
                        for (int i = 0; i < 4; ++i) bf[j][i] = bn[j][i];
                }
            }
            if (!seg_end) {
                continue;
            }

            // ---- segment end: publish this CTA's part of column tile jt ----------------------
            const int c_first = (jt * G32) / upc;
            const int c_last  = ((jt + 1) * G32 - 1) / upc;
            const int n_split = c_last - c_first + 1;
            const int n_cols  = ntw * kColsPerTile;
            const int col0    = tile0 * kColsPerTile;

            if (n_split == 1) {
                // this CTA saw the whole K range: straight from registers to C
                if (!dead && wt < ntw) {
#pragma unroll
                    for (int a = 0; a < 2; ++a)
#pragma unroll
                        for (int j = 0; j < NT; ++j)
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int   n = col0 + wt * kColsPerTile + a * 16 + r + (i >> 1) * 8;
                                const int   t = t0 + j * 8 + 2 * c + (i & 1);
                                const float v = tot[a][j][i];
                                if (p.fused_silu) {
                                    // kernels/gemm_s_f16/gemm_s4_f16.cu:31-43 on the fp16-rounded pair;
                                    // the partner column n^1 lives in lane^4
                                    const float mine  = __half2float(__float2half_rn(v));
                                    const float other = __shfl_xor_sync(0xffffffffu, mine, 4);
                                    if ((r & 1) == 0 && t < p.T) {
                                        const float silu = mine / (1.f + __expf(-mine));
                                        p.C[(size_t)t * (p.N / 2) + n / 2] = __float2half_rn(silu * other);
                                    }
                                }
                                else if (t < p.T) {
                                    p.C[(size_t)t * p.N + n] = __float2half_rn(v);
                                }
                            }
                }
            }
            else {
                // (cta + column tile) is unique per segment: along the unit order either the CTA
                // or the column tile advances, never both backwards.
                float* slot = p.workspace
                              + ((size_t)blockIdx.y * p.slots_per_chunk + blockIdx.x + jt) * (size_t)(TP * kUnitCols);
#pragma unroll
                for (int a = 0; a < 2; ++a)
#pragma unroll
                    for (int j = 0; j < NT; ++j)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int n = wt * kColsPerTile + a * 16 + r + (i >> 1) * 8;
                            const int t = j * 8 + 2 * c + (i & 1);
                            __stcg(slot + t * kUnitCols + n, tot[a][j][i]);
                        }
                __threadfence();
                named_bar_sync(1, kConsThreads);
                if (ctid == 0) {
                    int*      counter = p.counters + (size_t)blockIdx.y * p.n_col_tiles + jt;
                    const int ticket  = atomicAdd(counter, 1);
                    const int is_last = (ticket == n_split - 1);
                    if (is_last) {
                        *counter = 0;  // self-reset for the next launch
                    }
                    s_flag[0] = is_last;
                }
                named_bar_sync(1, kConsThreads);
                const bool finalize = s_flag[0] != 0;
                if (finalize && !dead) {
                    __threadfence();
                    // fixed-order reduction of every CTA's partial, two adjacent columns per thread
                    const int pairs = n_cols / 2;
                    for (int i = ctid; i < t_rows * pairs; i += kConsThreads) {
                        const int t  = i / pairs;
                        const int n  = (i - t * pairs) * 2;
                        float     v0 = 0.f, v1 = 0.f;
                        for (int cc = c_first; cc <= c_last; ++cc) {
                            const float* sl = p.workspace
                                              + ((size_t)blockIdx.y * p.slots_per_chunk + cc + jt)
                                                    * (size_t)(TP * kUnitCols);
                            const float2 v = __ldcg(reinterpret_cast<const float2*>(sl + t * kUnitCols + n));
                            v0 += v.x;
                            v1 += v.y;
                        }
                        const __half2 h = __floats2half2_rn(v0, v1);
                        if (p.fused_silu) {
                            const float2 u    = __half22float2(h);
                            const float  silu = u.x / (1.f + __expf(-u.x));
                            p.C[(size_t)(t0 + t) * (p.N / 2) + (col0 + n) / 2] = __float2half_rn(silu * u.y);
                        }
                        else {
                            *reinterpret_cast<__half2*>(p.C + (size_t)(t0 + t) * p.N + col0 + n) = h;
                        }
                    }
                }
                named_bar_sync(1, kConsThreads);  // s_flag is reused by the next segment
            }
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) tot[a][j][i] = 0.f;
        }
    }
}

}  // namespace

size_t gemm_small_smem_bytes(int stages)
{
    return (size_t)stages * kStageBytes + (size_t)stages * 16 + 16;
}

GemmSmallPlan gemm_small_plan(int N, int T, int K, int sm_count, int max_smem, int want_stages)
{
    GemmSmallPlan pl{};
    pl.nt = T <= 8 ? 1 : (T <= 16 ? 2 : 4);
    const int tp   = pl.nt * 8;
    pl.t_chunks    = (T + tp - 1) / tp;
    pl.n_col_tiles = (N / kColsPerTile + kTilesPerUnit - 1) / kTilesPerUnit;
    const int G32  = K / 32;
    pl.total_units = pl.n_col_tiles * G32;
    int ctas       = sm_count < pl.total_units ? sm_count : pl.total_units;
    pl.units_per_cta   = (pl.total_units + ctas - 1) / ctas;
    pl.ctas            = (pl.total_units + pl.units_per_cta - 1) / pl.units_per_cta;
    pl.slots_per_chunk = pl.ctas + pl.n_col_tiles;
    int stages         = want_stages > 0 ? want_stages : 20;
    if (stages > pl.units_per_cta) stages = pl.units_per_cta < 2 ? 2 : pl.units_per_cta;
    while (stages > 2 && gemm_small_smem_bytes(stages) > (size_t)max_smem) --stages;
    pl.stages           = stages;
    pl.smem_bytes       = gemm_small_smem_bytes(stages);
    pl.workspace_floats = (size_t)pl.t_chunks * pl.slots_per_chunk * tp * kUnitCols;
    pl.counter_ints     = (size_t)pl.t_chunks * pl.n_col_tiles;
    return pl;
}

cudaError_t gemm_small_prepare(int max_smem)
{
    cudaError_t e;
    e = cudaFuncSetAttribute(gemm_s4_f16_small_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(gemm_s4_f16_small_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(gemm_s4_f16_small_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
}

cudaError_t gemm_small_launch(const GemmSmallPlan& pl, GemmSmallParams p, cudaStream_t st)
{
    p.units_per_cta   = pl.units_per_cta;
    p.total_units     = pl.total_units;
    p.slots_per_chunk = pl.slots_per_chunk;
    p.n_col_tiles     = pl.n_col_tiles;
    p.stages          = pl.stages;
    dim3 grid(pl.ctas, pl.t_chunks);
    dim3 block(32 + kConsThreads);
    switch (pl.nt) {
        case 1: gemm_s4_f16_small_kernel<1><<<grid, block, pl.smem_bytes, st>>>(p); break;
        case 2: gemm_s4_f16_small_kernel<2><<<grid, block, pl.smem_bytes, st>>>(p); break;
        default: gemm_s4_f16_small_kernel<4><<<grid, block, pl.smem_bytes, st>>>(p); break;
    }
    return cudaGetLastError();
}

}  // namespace tmb

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the small-token GEMM (tm_gemm_s4_f16_noalloc in tm_b200.h).
//
// Some hosts of this library cannot call the CUDA allocator at all: an inference-server plugin
// whose device memory is owned and budgeted by the server, a process that has already handed
// every free byte to its KV-cache pool, or a latency-critical loop that must not hit
// cudaMalloc's implicit device synchronisation.  tm_create() allocates the split-K scratch of
// this kernel with cudaMalloc; the entry point below needs no handle and calls no allocator:
// the scratch lives in the library image itself, in the fixed-size device array declared here,
// which every GPU that loads the library holds until the process exits.
//
// Layout of the array: [0, 4 KB) arrival tickets (int) with the status word of the bounded waits
// at byte 4092; [4 KB, end) split-K partial tiles (fp32).
namespace tmb {
namespace {

constexpr size_t kStaticScratchBytes  = 8u << 20;  // 8 MB per GPU, the stated maximum
constexpr size_t kStaticControlBytes  = 4096;
constexpr int    kStaticMaxDevices    = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct StaticScratchDevice {
    void* ptr      = nullptr;  // DEVICE address of g_static_scratch on this GPU
    int   sm_count = 0;
    int   max_smem = 0;
    bool  ready    = false;
};
StaticScratchDevice g_static_dev[kStaticMaxDevices];  // guarded by g_static_mutex
std::mutex          g_static_mutex;

}  // namespace
}  // namespace tmb

extern "C" int tm_gemm_s4_f16_noalloc(
    void* C, const void* A, const void* B, const void* Q, int m, int n, int k, int group_size, int type, void* stream)
{
    using namespace tmb;
    if (!C || !A || !B || !Q) return TM_ERR_INVALID_ARG;
    if (((uintptr_t)C | (uintptr_t)A | (uintptr_t)B | (uintptr_t)Q) & 15u) return TM_ERR_INVALID_ARG;
    if (m <= 0 || n <= 0 || k <= 0) return TM_ERR_INVALID_ARG;
    if (group_size != 128 || k % 128 || m % 32) return TM_ERR_UNSUPPORTED;
    if (type != TM_GEMM_PLAIN && type != TM_GEMM_FUSED_SILU_FFN) return TM_ERR_UNSUPPORTED;
    if (type == TM_GEMM_FUSED_SILU_FFN && m % 64) return TM_ERR_UNSUPPORTED;
    if (n > 16) return TM_ERR_WORKSPACE;  // beyond the built-in scratch: only the small-token kernel is offered here

    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return TM_ERR_CUDA;
    if (dev < 0 || dev >= kStaticMaxDevices) return TM_ERR_UNSUPPORTED;

    StaticScratchDevice d;
    {
        // First call on this device: resolve the device address of the array (its name is only a
        // host-side stand-in for the symbol), read two device attributes and raise the kernel's
        // shared-memory limit.  None of these allocates.  Do this first call outside stream capture.
        std::lock_guard<std::mutex> lock(g_static_mutex);
        StaticScratchDevice&        s = g_static_dev[dev];
        if (!s.ready) {
            void* p = nullptr;
            if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return TM_ERR_CUDA;
            int sms = 0, smem = 0;
            if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return TM_ERR_CUDA;
            if (cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return TM_ERR_CUDA;
            if (gemm_small_prepare(smem) != cudaSuccess) return TM_ERR_CUDA;
            s.ptr      = p;
            s.sm_count = sms;
            s.max_smem = smem;
            s.ready    = true;
        }
        d = s;
    }

    const GemmSmallPlan pl = gemm_small_plan(m, n, k, d.sm_count, d.max_smem, 0);
    if (pl.counter_ints * sizeof(int) > kStaticControlBytes - 8
        || pl.workspace_floats * sizeof(float) > kStaticScratchBytes - kStaticControlBytes) {
        return TM_ERR_WORKSPACE;  // problem too large for the 8 MB built into the library
    }
    // The array keeps whatever the previous call left.  Tickets and the status word must start at
    // zero (a call that was cut short may have left them otherwise); the partial tiles need no
    // clearing, every slot is written before it is read.
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemsetAsync(d.ptr, 0, kStaticControlBytes, st) != cudaSuccess) return TM_ERR_CUDA;

    GemmSmallParams p{};
    p.C          = (__half*)C;
    p.A          = (const unsigned char*)A;
    p.X          = (const unsigned char*)B;
    p.Q          = (const unsigned char*)Q;
    p.workspace  = (float*)((char*)d.ptr + kStaticControlBytes);
    p.counters   = (int*)d.ptr;
    p.status     = (unsigned*)((char*)d.ptr + kStaticControlBytes - 4);
    p.N          = m;
    p.T          = n;
    p.K          = k;
    p.fused_silu = type == TM_GEMM_FUSED_SILU_FFN;
    return gemm_small_launch(pl, p, st) == cudaSuccess ? TM_OK : TM_ERR_CUDA;
}
