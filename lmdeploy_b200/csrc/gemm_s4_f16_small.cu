// W4A16 GEMM for small token counts (the HBM-bound regime): a persistent, stream-K balanced
// kernel.  One producer thread streams the packed int4 weight, the {zero, scale} rows and the
// activation slices through a ring of shared-memory stages with bulk copies (TMA, mbarrier
// completion); consumer warps unpack nibbles with lop3, subtract the zero point exactly in
// fp16, feed the integers to mma.m16n8k16 (the runtime int4 layout IS that instruction's A
// fragment) and apply the group scale to the fp32 group sums.  K is split across CTAs
// (every CTA gets the same number of 128x128 weight units); partial tiles meet in a scratch
// buffer and the last CTA to arrive for a column tile reduces them in a fixed order, so the
// result is deterministic and no CTA ever waits for another.
//
// Replaces the small-n end of GemmS4F16::Run (src/turbomind/kernels/gemm_s_f16/
// gemm_s4_f16.cu:208-234) / gemm_s4_f16_nn (gemm_template.h:338-444), whose smallest token
// tile is 8 and which has no split-K across CTAs.
#include "common.cuh"
#include "gemm_s4_f16.h"

namespace tmb {

namespace {

constexpr int kColsPerTile   = 32;   // one packed 32x32 tile = 512 B
constexpr int kTilesPerUnit  = 4;    // column tiles per CTA unit
constexpr int kUnitCols      = kColsPerTile * kTilesPerUnit;  // 128
constexpr int kGroup         = 128;  // quantisation group = K extent of a unit
constexpr int kK32PerUnit    = kGroup / 32;
constexpr int kTileBytes     = 512;
constexpr int kWBytes        = kK32PerUnit * kTilesPerUnit * kTileBytes;  // 8192
constexpr int kQBytes        = kUnitCols * 4;                             // 512
constexpr int kXRowBytes     = kGroup * 2 + 16;                           // 272: conflict-free B fragments
constexpr int kWarpsPerGroup = kTilesPerUnit;
constexpr int kGroupThreads  = kWarpsPerGroup * 32;

__host__ __device__ constexpr int stage_bytes(int tp)
{
    return kWBytes + kQBytes + tp * kXRowBytes;  // multiple of 16 for tp % 8 == 0
}

// dynamic shared memory: [stages][stage_bytes] | red[groups][TP][kUnitCols] f32 | full[stages] |
// empty[stages] | flag

template<int NT>
__global__ void __launch_bounds__(32 + 4 * kGroupThreads, 1) gemm_s4_f16_small_kernel(GemmSmallParams p)
{
    constexpr int TP = NT * 8;
    extern __shared__ __align__(128) unsigned char smem_raw[];

    const int stages   = p.stages;
    const int n_groups = p.consumer_groups;
    const int sbytes   = stage_bytes(TP);

    unsigned char* stage_base = smem_raw;
    float*         red        = reinterpret_cast<float*>(smem_raw + (size_t)stages * sbytes);
    uint64_t*      full_bar   = reinterpret_cast<uint64_t*>(red + (size_t)n_groups * TP * kUnitCols);
    uint64_t*      empty_bar  = full_bar + stages;
    int*           s_flag     = reinterpret_cast<int*>(empty_bar + stages);  // [0] ticket result

    const int tid  = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    // token chunk handled by this CTA row
    const int t0     = blockIdx.y * TP;
    const int t_rows = min(TP, p.T - t0);

    const int G        = p.K / kGroup;           // units per column tile
    const int upc      = p.units_per_cta;
    const int u_begin  = blockIdx.x * upc;
    const int u_end    = min(u_begin + upc, p.total_units);
    const int n_units  = u_end - u_begin;
    const int n_tiles32 = p.N / kColsPerTile;

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kWarpsPerGroup);
        }
        fence_mbar_init();
    }
    // zero the activation rows that no copy will ever write (token padding of the MMA tile)
    for (int s = 0; s < stages; ++s) {
        uint32_t* xs = reinterpret_cast<uint32_t*>(stage_base + (size_t)s * sbytes + kWBytes + kQBytes);
        for (int i = tid; i < TP * kXRowBytes / 4; i += blockDim.x) {
            xs[i] = 0u;
        }
    }
    fence_proxy_async_smem();
    __syncthreads();

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            const uint64_t pol_w = policy_evict_first();
            const uint64_t pol_x = policy_evict_last();
            bool           dead  = false;
            int            it    = 0;
            for (; it < n_units && !dead; ++it) {
                const int s = it % stages;
                if (it >= stages) {
                    if (!mbar_wait(&empty_bar[s], ((it / stages) - 1) & 1)) {
                        atomicOr(p.status, kStatusGemvEmptyWait);
                        dead = true;
                        break;
                    }
                }
                const int u     = u_begin + it;
                const int jt    = u / G;
                const int g     = u - jt * G;
                const int tile0 = jt * kTilesPerUnit;
                const int ntw   = min(kTilesPerUnit, n_tiles32 - tile0);

                unsigned char* sb = stage_base + (size_t)s * sbytes;
                const uint32_t tx = (uint32_t)(kK32PerUnit * ntw * kTileBytes + ntw * kColsPerTile * 4 + t_rows * kGroup * 2);
                mbar_arrive_expect_tx(&full_bar[s], tx);
#pragma unroll
                for (int r = 0; r < kK32PerUnit; ++r) {
                    const size_t k32 = (size_t)g * kK32PerUnit + r;
                    bulk_g2s_hint(sb + r * kTilesPerUnit * kTileBytes,
                                  p.A + (k32 * n_tiles32 + tile0) * kTileBytes,
                                  (uint32_t)(ntw * kTileBytes),
                                  &full_bar[s],
                                  pol_w);
                }
                bulk_g2s_hint(sb + kWBytes,
                              p.Q + ((size_t)g * p.N + (size_t)tile0 * kColsPerTile) * 4,
                              (uint32_t)(ntw * kColsPerTile * 4),
                              &full_bar[s],
                              pol_w);
                for (int t = 0; t < t_rows; ++t) {
                    bulk_g2s_hint(sb + kWBytes + kQBytes + t * kXRowBytes,
                                  p.X + ((size_t)(t0 + t) * p.K + (size_t)g * kGroup) * 2,
                                  kGroup * 2,
                                  &full_bar[s],
                                  pol_x);
                }
            }
            if (dead) {
                // consumers may have stopped too: make sure none of our copies is still in
                // flight towards this CTA's shared memory before the CTA can retire.
                const int issued = it;
                for (int j = max(0, issued - stages); j < issued; ++j) {
                    (void)mbar_wait(&full_bar[j % stages], (j / stages) & 1);
                }
            }
        }
    }
    else {
        // ------------------------------------------------------------------ consumers
        const int cw    = warp - 1;
        const int grp   = cw / kWarpsPerGroup;   // consumer group
        const int wt    = cw % kWarpsPerGroup;   // column tile inside the unit
        const int r     = lane >> 2;             // fragment row
        const int c     = lane & 3;              // fragment column pair
        const int n_cons = n_groups * kGroupThreads;
        const int ctid  = tid - 32;
        bool      dead  = false;

        float tot[2][NT][4];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) tot[a][j][i] = 0.f;

        float* my_red = red + (size_t)grp * TP * kUnitCols;

        int it = 0;  // unit index inside this CTA
        while (it < n_units) {
            // one segment = the run of this CTA's units that share a column tile
            const int u_first = u_begin + it;
            const int jt      = u_first / G;
            const int seg_end = min(n_units, (jt + 1) * G - u_begin);  // exclusive, CTA-local
            const int tile0   = jt * kTilesPerUnit;
            const int ntw     = min(kTilesPerUnit, n_tiles32 - tile0);

            // first unit of the segment that belongs to this consumer group
            int my = it + ((grp - it) % n_groups + n_groups) % n_groups;
            for (; my < seg_end; my += n_groups) {
                const int s = my % stages;
                if (!dead && !mbar_wait(&full_bar[s], (my / stages) & 1)) {
                    atomicOr(p.status, kStatusGemvFullWait);
                    dead = true;
                }
                if (!dead && wt < ntw) {
                    const unsigned char* sb = stage_base + (size_t)s * sbytes;
                    const uint4*         ws = reinterpret_cast<const uint4*>(sb) + wt * 32 + lane;
                    const __half2*       qs = reinterpret_cast<const __half2*>(sb + kWBytes) + wt * kColsPerTile;
                    const uint32_t*      xs = reinterpret_cast<const uint32_t*>(sb + kWBytes + kQBytes);

                    // {64+z, s} of the four rows this lane owns: n16 in {0,1} x {r, r+8}
                    uint32_t z1024[2], nz64[2];
                    float    sc[2][2];
#pragma unroll
                    for (int a = 0; a < 2; ++a) {
                        const __half2 q_lo = qs[a * 16 + r];
                        const __half2 q_hi = qs[a * 16 + r + 8];
                        const __half  zl   = __hadd(__low2half(q_lo), __float2half_rn(960.f));
                        const __half  zh   = __hneg(__low2half(q_hi));
                        const __half2 zl2  = __half2half2(zl);
                        const __half2 zh2  = __half2half2(zh);
                        z1024[a]           = reinterpret_cast<const uint32_t&>(zl2);
                        nz64[a]            = reinterpret_cast<const uint32_t&>(zh2);
                        sc[a][0]           = __high2float(q_lo);
                        sc[a][1]           = __high2float(q_hi);
                    }

                    float acc[2][NT][4];
#pragma unroll
                    for (int a = 0; a < 2; ++a)
#pragma unroll
                        for (int j = 0; j < NT; ++j)
#pragma unroll
                            for (int i = 0; i < 4; ++i) acc[a][j][i] = 0.f;

#pragma unroll
                    for (int ks = 0; ks < kK32PerUnit; ++ks) {
                        const uint4 w = ws[ks * kTilesPerUnit * 32];
                        uint32_t    bf[NT][4];
#pragma unroll
                        for (int j = 0; j < NT; ++j) {
                            const uint32_t* xr = xs + (j * 8 + r) * (kXRowBytes / 4) + ks * 16 + c;
                            bf[j][0]           = xr[0];
                            bf[j][1]           = xr[4];
                            bf[j][2]           = xr[8];
                            bf[j][3]           = xr[12];
                        }
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
                    if (lane == 0) {
                        mbar_arrive(&empty_bar[s]);
                    }
#pragma unroll
                    for (int a = 0; a < 2; ++a)
#pragma unroll
                        for (int j = 0; j < NT; ++j) {
                            tot[a][j][0] = fmaf(sc[a][0], acc[a][j][0], tot[a][j][0]);
                            tot[a][j][1] = fmaf(sc[a][0], acc[a][j][1], tot[a][j][1]);
                            tot[a][j][2] = fmaf(sc[a][1], acc[a][j][2], tot[a][j][2]);
                            tot[a][j][3] = fmaf(sc[a][1], acc[a][j][3], tot[a][j][3]);
                        }
                }
                else {
                    __syncwarp();
                    if (lane == 0 && !dead) {
                        mbar_arrive(&empty_bar[s]);
                    }
                }
            }

            // ---- segment end: fold the consumer groups, then publish --------------------
            // red[grp][t][n]  (t = token inside the chunk, n = column inside the unit)
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const int n  = wt * kColsPerTile + a * 16 + r;
                    const int tt = j * 8 + 2 * c;
                    my_red[(tt + 0) * kUnitCols + n]     = tot[a][j][0];
                    my_red[(tt + 1) * kUnitCols + n]     = tot[a][j][1];
                    my_red[(tt + 0) * kUnitCols + n + 8] = tot[a][j][2];
                    my_red[(tt + 1) * kUnitCols + n + 8] = tot[a][j][3];
                    tot[a][j][0] = tot[a][j][1] = tot[a][j][2] = tot[a][j][3] = 0.f;
                }
            named_bar_sync(1, n_cons);

            // which CTAs share this column tile?
            const int c_first = (jt * G) / upc;
            const int c_last  = ((jt + 1) * G - 1) / upc;
            const int n_split = c_last - c_first + 1;
            const int n_cols  = ntw * kColsPerTile;
            const int col0    = tile0 * kColsPerTile;

            bool   finalize = true;
            float* ws_tile  = nullptr;
            if (n_split > 1) {
                // (cta + column tile) is unique per segment: along the unit order either the
                // CTA or the column tile advances, never both backwards.
                float* slot = p.workspace
                              + ((size_t)blockIdx.y * p.slots_per_chunk + blockIdx.x + jt) * (size_t)(TP * kUnitCols);
                for (int i = ctid; i < t_rows * kUnitCols; i += n_cons) {
                    float v = 0.f;
                    for (int gI = 0; gI < n_groups; ++gI) v += red[(size_t)gI * TP * kUnitCols + i];
                    __stcg(slot + i, v);
                }
                __threadfence();
                named_bar_sync(1, n_cons);
                if (ctid == 0) {
                    int*      counter = p.counters + (size_t)blockIdx.y * p.n_col_tiles + jt;
                    const int ticket  = atomicAdd(counter, 1);
                    const int last    = (ticket == n_split - 1);
                    if (last) {
                        *counter = 0;  // self-reset for the next launch
                    }
                    s_flag[0] = last;
                }
                named_bar_sync(1, n_cons);
                finalize = s_flag[0] != 0;
                if (finalize) {
                    __threadfence();
                }
                ws_tile = p.workspace;
            }

            if (finalize && !dead) {
                // epilogue over [t_rows][n_cols], two adjacent columns per thread
                const int pairs = n_cols / 2;
                for (int i = ctid; i < t_rows * pairs; i += n_cons) {
                    const int t  = i / pairs;
                    const int n  = (i - t * pairs) * 2;
                    float     v0 = 0.f, v1 = 0.f;
                    if (n_split > 1) {
                        for (int cc = c_first; cc <= c_last; ++cc) {
                            const float* slot = ws_tile
                                                + ((size_t)blockIdx.y * p.slots_per_chunk + cc + jt)
                                                      * (size_t)(TP * kUnitCols);
                            const float2 v = __ldcg(reinterpret_cast<const float2*>(slot + t * kUnitCols + n));
                            v0 += v.x;
                            v1 += v.y;
                        }
                    }
                    else {
                        for (int gI = 0; gI < n_groups; ++gI) {
                            const float2 v =
                                *reinterpret_cast<const float2*>(red + (size_t)gI * TP * kUnitCols + t * kUnitCols + n);
                            v0 += v.x;
                            v1 += v.y;
                        }
                    }
                    const __half2 h = __floats2half2_rn(v0, v1);
                    if (p.fused_silu) {
                        // kernels/gemm_s_f16/gemm_s4_f16.cu:31-43: on the fp16-rounded pair
                        const float2 u    = __half22float2(h);
                        const float  silu = u.x / (1.f + __expf(-u.x));
                        p.C[(size_t)(t0 + t) * (p.N / 2) + (col0 + n) / 2] = __float2half_rn(silu * u.y);
                    }
                    else {
                        *reinterpret_cast<__half2*>(p.C + (size_t)(t0 + t) * p.N + col0 + n) = h;
                    }
                }
            }
            named_bar_sync(1, n_cons);  // red[] is reused by the next segment
            it = seg_end;
        }
    }
}

}  // namespace

size_t gemm_small_smem_bytes(int nt, int stages, int groups)
{
    const int tp = nt * 8;
    return (size_t)stages * stage_bytes(tp) + (size_t)groups * tp * kUnitCols * 4 + (size_t)stages * 16 + 16;
}

GemmSmallPlan gemm_small_plan(int N, int T, int K, int sm_count, int max_smem, int want_stages, int want_groups)
{
    GemmSmallPlan pl{};
    pl.nt = T <= 8 ? 1 : (T <= 16 ? 2 : 4);
    const int tp   = pl.nt * 8;
    pl.t_chunks    = (T + tp - 1) / tp;
    pl.n_col_tiles = (N / kColsPerTile + kTilesPerUnit - 1) / kTilesPerUnit;
    const int G    = K / kGroup;
    pl.total_units = pl.n_col_tiles * G;
    int ctas       = sm_count < pl.total_units ? sm_count : pl.total_units;
    pl.units_per_cta = (pl.total_units + ctas - 1) / ctas;
    pl.ctas          = (pl.total_units + pl.units_per_cta - 1) / pl.units_per_cta;
    pl.slots_per_chunk = pl.ctas + pl.n_col_tiles;
    pl.groups        = want_groups > 0 ? want_groups : (pl.nt >= 4 ? 2 : 3);
    if (pl.groups > 4) pl.groups = 4;
    int stages = want_stages > 0 ? want_stages : 16;
    if (stages > pl.units_per_cta) stages = pl.units_per_cta < 2 ? 2 : pl.units_per_cta;
    while (stages > 2 && gemm_small_smem_bytes(pl.nt, stages, pl.groups) > (size_t)max_smem) --stages;
    pl.stages     = stages;
    pl.smem_bytes = gemm_small_smem_bytes(pl.nt, stages, pl.groups);
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
    p.consumer_groups = pl.groups;
    dim3 grid(pl.ctas, pl.t_chunks);
    dim3 block(32 + pl.groups * kGroupThreads);
    switch (pl.nt) {
        case 1: gemm_s4_f16_small_kernel<1><<<grid, block, pl.smem_bytes, st>>>(p); break;
        case 2: gemm_s4_f16_small_kernel<2><<<grid, block, pl.smem_bytes, st>>>(p); break;
        default: gemm_s4_f16_small_kernel<4><<<grid, block, pl.smem_bytes, st>>>(p); break;
    }
    return cudaGetLastError();
}

}  // namespace tmb
