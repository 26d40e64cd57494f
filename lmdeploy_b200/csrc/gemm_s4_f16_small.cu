// W4A16 GEMM for small token counts (the HBM-bound regime): persistent, stream-K balanced, two CTAs
// per SM for up to 8 tokens.  Work unit = 64 input rows x 512 output columns of the packed weight:
// two slabs of 16 tiles (512 B each), every slab one contiguous 8 KB run.  Each of the 8 warps owns
// two adjacent 32-column tiles of every slab and streams them through its own cp.async ring
// (16 bytes per lane, a whole 512-byte tile per instruction); the activations of the unit (64 B per
// token and slab) go to a slab shared by the CTA, stored with a chunk swizzle so that ldmatrix
// delivers them as B fragments without bank conflicts.  One __syncthreads per unit publishes the
// activations and frees the slot that is refilled next.
// A tile is exactly four mma.m16n8k16 A fragments of packed nibbles; a warp turns a packed word into
// tensor-core operands with five integer instructions (one shift, four lop3) and nothing else: the
// fp16 values fed to the MMA are 1024 + q (rows r) and 1024 + 16 q (rows r + 8), and zero point,
// offsets and scale are applied once per 128-row group to the fp32 group sums, using the group sum
// of the activations that an extra MMA against an all-ones fragment delivers in the same register
// layout:
//     y += s (P - (1024 + z) SX)            rows r
//     y += s/16 (P' - (1024 + 16 z) SX)     rows r + 8
// K is split across CTAs (every CTA gets the same number of units); partial column tiles meet in a
// scratch buffer and the last CTA to arrive for a column tile reduces them in a fixed order, so the
// result is deterministic and no CTA ever waits for another.
//
// Replaces the small-n end of GemmS4F16::Run (src/turbomind/kernels/gemm_s_f16/
// gemm_s4_f16.cu:208-234) / gemm_s4_f16_nn (gemm_template.h:338-444), whose smallest token
// tile is 8 and which has no split-K across CTAs.  The weight seen by the MMA differs from the
// reference's fp16_rn((q - z) s) only by that one rounding (the products are exact in fp32 here).
#include "common.cuh"
#include "gemm_s4_f16.h"
#include "tm_b200.h"

#include <mutex>

#ifdef TM_B200_GEMM_TRACE
// Developer build only (never defined by lmdeploy_b200/build.py): per-CTA time stamps of one launch.
__device__ unsigned long long g_small_trace[640][4];  // start, first data, loop end, end (globaltimer ns)
__device__ int                g_small_launch;
extern "C" __attribute__((visibility("default"))) int tm_dev_gemv_trace(unsigned long long* out, int want_launch)
{
    cudaMemcpyFromSymbol(out, g_small_trace, sizeof(unsigned long long) * 640 * 4);
    int z = -want_launch;   // the launch that reaches 0 is recorded
    cudaMemcpyToSymbol(g_small_launch, &z, sizeof(z));
    return 0;
}
__device__ __forceinline__ unsigned long long small_globaltimer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define SMALL_TRACE(slot)                                                                                              \
    do {                                                                                                                   \
        if (trace_on && threadIdx.x == 0 && blockIdx.x < 640) g_small_trace[blockIdx.x][slot] = small_globaltimer();       \
    } while (0)
#else
#define SMALL_TRACE(slot) do { } while (0)
#endif

namespace tmb {

namespace {

constexpr int kColsPerTile  = 32;   // one packed 32x32 tile = 512 B
constexpr int kTileBytes    = 512;
constexpr int kTilesPerUnit = 16;   // column tiles per unit
constexpr int kUnitCols     = kColsPerTile * kTilesPerUnit;  // 512
constexpr int kUnitRows     = 64;   // input rows per unit: two 32-row slabs
constexpr int kWarps        = 8;
constexpr int kTilesPerWarp = kTilesPerUnit / kWarps;        // 2
constexpr int kThreads      = kWarps * 32;
constexpr int kSlabBytes    = kTilesPerWarp * kTileBytes;    // a warp's part of one slab: 1 KB
constexpr int kWarpStage    = 2 * kSlabBytes + 256;          // two slabs + {zero, scale} of the 64 columns

// stages of the cp.async rings per token-tile count
__host__ __device__ constexpr int stages_for(int nt) { return nt == 1 ? 5 : 6; }
// co-resident CTAs per SM
__host__ __device__ constexpr int ctas_per_sm_for(int nt) { return nt == 1 ? 2 : 1; }

// dynamic shared memory: [warps][stages][kWarpStage] | [stages][2 slabs][TP x 64 B] | flag

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit()
{
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template<int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// One packed word -> A fragment {1024 + q | rows r, 1024 + 16 q | rows r + 8, same for k + 8}
__device__ __forceinline__ void unpack_s4_biased(uint32_t w, uint32_t (&out)[4])
{
    constexpr uint32_t kLut   = (0xf0 & 0xcc) | 0xaa;  // (a & b) | c
    constexpr uint32_t kBot   = 0x000f000f;
    constexpr uint32_t kTop   = 0x00f000f0;
    constexpr uint32_t kMagic = 0x64006400;  // half2{1024, 1024}
    const uint32_t     hi     = w >> 8;
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(out[0]) : "r"(w), "n"(kBot), "n"(kMagic), "n"(kLut));
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(out[1]) : "r"(w), "n"(kTop), "n"(kMagic), "n"(kLut));
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(out[2]) : "r"(hi), "n"(kBot), "n"(kMagic), "n"(kLut));
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(out[3]) : "r"(hi), "n"(kTop), "n"(kMagic), "n"(kLut));
}

// B fragments (activations) of one 32-row slab for one 8-token tile.  A slab holds [tokens][4 chunks
// of 16 B]; chunk i of token t sits at position i ^ ((t >> 1) & 3), which makes both the cp.async
// writes and these ldmatrix reads free of bank conflicts.  `addr` = tile base + this lane's row.
__device__ __forceinline__ void load_x_frag(uint32_t (&bf)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(bf[0]), "=r"(bf[1]), "=r"(bf[2]), "=r"(bf[3])
                 : "r"(addr));
}

template<int NT>
__global__ void __launch_bounds__(kThreads, ctas_per_sm_for(NT)) gemm_s4_f16_small_kernel(GemmSmallParams p)
{
    constexpr int TP     = NT * 8;
    constexpr int ST     = stages_for(NT);
    constexpr int kXSlab = TP * 64;      // activations of one 32-row slab
    constexpr int kXUnit = 2 * kXSlab;   // ... of one unit
    extern __shared__ __align__(128) unsigned char smem_raw[];

    constexpr int  kXRingOff = kWarps * ST * kWarpStage;
    const uint32_t smem_s    = smem_u32(smem_raw);
    int*           s_flag    = reinterpret_cast<int*>(smem_raw + kXRingOff + ST * kXUnit);

    const int tid  = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int r    = lane >> 2;  // fragment row
    const int c    = lane & 3;   // fragment column pair
#ifdef TM_B200_GEMM_TRACE
    const bool trace_on = *(volatile int*)&g_small_launch == 0 && blockIdx.y == 0;
    SMALL_TRACE(0);
#endif

    // token chunk handled by this CTA row
    const int t0     = blockIdx.y * TP;
    const int t_rows = min(TP, p.T - t0);

    const int G         = p.K / kUnitRows;  // units per column tile
    const int upc       = p.units_per_cta;
    const int u_begin   = blockIdx.x * upc;
    const int n_units   = min(u_begin + upc, p.total_units) - u_begin;
    const int n_tiles32 = p.N / kColsPerTile;

    // rows of the activation slabs that no token fills stay zero for the whole kernel
    if (t_rows < TP) {
        for (int i = tid; i < ST * 2 * TP * 4; i += kThreads) {
            if (((i >> 2) % TP) >= t_rows) {
                *reinterpret_cast<uint4*>(smem_raw + kXRingOff + i * 16) = make_uint4(0, 0, 0, 0);
            }
        }
    }

    // ---- copies: each warp feeds its private weight ring, the first threads also the shared slabs ----
    const uint32_t ring_s = smem_s + warp * (ST * kWarpStage);
    // activation chunk of this thread: token x_row, 16-byte piece x_sub of the unit's 128 B per token
    const int      x_row    = tid >> 3;
    const int      x_sub    = tid & 7;
    const bool     x_loader = x_row < t_rows;  // implies tid < TP * 8
    const unsigned char* const x_base =
        p.X + ((size_t)(t0 + (x_loader ? x_row : 0)) * p.K) * 2 + x_sub * 16;
    const uint32_t x_dst = smem_s + kXRingOff + (x_sub >> 2) * kXSlab + x_row * 64
                           + (((x_sub & 3) ^ ((x_row >> 1) & 3)) << 4);
    const size_t slab_stride = (size_t)n_tiles32 * kTileBytes;  // bytes between 32-row slabs of the weight

    // state of the copy front (runs ST - 1 units ahead of the math)
    int                  i_jt = u_begin / G, i_k = u_begin - i_jt * G;
    int                  i_tile  = 0;
    const unsigned char* i_w     = nullptr;  // this lane's 16 B of the warp's first tile, slab 2 i_k
    const unsigned char* i_q     = nullptr;  // this lane's 16 B of the {zero, scale} row of the group of i_k
    int                  i_step  = 0;        // bytes to the warp's second tile (0 where N ends after the first)
    bool                 i_qok   = false;
    auto                 i_seek  = [&]() {
        // a warp whose tiles lie beyond N re-reads the last pair; what it computes is never stored
        i_tile = min(i_jt * kTilesPerUnit + warp * kTilesPerWarp, (n_tiles32 - 1) & ~1);
        i_step = i_tile + 1 < n_tiles32 ? kTileBytes : 0;
        i_w    = p.A + ((size_t)(2 * i_k) * n_tiles32 + i_tile) * kTileBytes + lane * 16;
        i_q    = p.Q + ((size_t)(i_k >> 1) * p.N + (size_t)i_tile * kColsPerTile) * 4 + (lane & 15) * 16;
        i_qok  = lane < 16 && i_tile * kColsPerTile + lane * 4 < p.N;
    };
    i_seek();
    // `with_x`: also the unit's activations (not before pdl_wait(): they come from the kernel before this one)
    auto issue_unit = [&](int stage, bool with_x) {
        const uint32_t dst = ring_s + stage * kWarpStage + lane * 16;
        // the warp's two tiles are adjacent in memory: 1 KB contiguous per slab
        cp_async16(dst, i_w);
        cp_async16(dst + kTileBytes, i_w + i_step);
        cp_async16(dst + kSlabBytes, i_w + slab_stride);
        cp_async16(dst + kSlabBytes + kTileBytes, i_w + slab_stride + i_step);
        if ((i_k & 1) == 0) {
            // {64 + z, s} of the warp's 64 columns for this group: 256 B
            if (i_qok) cp_async16(dst + 2 * kSlabBytes, i_q);
            i_q += (size_t)p.N * 4;
        }
        if (with_x && x_loader) cp_async16(x_dst + stage * kXUnit, x_base + (size_t)i_k * (kUnitRows * 2));
        i_w += 2 * slab_stride;
        if (++i_k == G) {
            i_k = 0;
            ++i_jt;
            i_seek();
        }
    };
    // The weights of the first ST - 1 units are requested before the kernel ahead of this one in the
    // stream is known to be complete (nothing writes them).  Their activations follow after the wait as
    // plain loads and shared-memory stores, which the first barrier of the loop publishes: the first unit
    // then waits for its own 16 KB of weights only, not for the whole window of requests behind it.
    const int x_k0 = i_k;
#pragma unroll
    for (int sidx = 0; sidx < ST - 1; ++sidx) {
        if (sidx < n_units) issue_unit(sidx, false);
        cp_async_commit();
    }
    pdl_wait();
    pdl_launch_dependents();
    if (x_loader) {
        int   xk = x_k0;
        uint4 xv[ST - 1];
#pragma unroll
        for (int sidx = 0; sidx < ST - 1; ++sidx) {
            xv[sidx] = make_uint4(0, 0, 0, 0);
            if (sidx < n_units) xv[sidx] = __ldcg(reinterpret_cast<const uint4*>(x_base + (size_t)xk * (kUnitRows * 2)));
            if (++xk == G) xk = 0;
        }
#pragma unroll
        for (int sidx = 0; sidx < ST - 1; ++sidx) {
            if (sidx < n_units) *reinterpret_cast<uint4*>(smem_raw + (x_dst - smem_s) + sidx * kXUnit) = xv[sidx];
        }
    }

    // per (tile, 16-row half): Z = offset + zero (rows r / r + 8) and the scale (s, s / 16)
    float zl[kTilesPerWarp][2], zh[kTilesPerWarp][2], sl[kTilesPerWarp][2], sh[kTilesPerWarp][2];
#pragma unroll
    for (int w = 0; w < kTilesPerWarp; ++w)
#pragma unroll
        for (int a = 0; a < 2; ++a) zl[w][a] = zh[w][a] = sl[w][a] = sh[w][a] = 0.f;

    float tot[kTilesPerWarp][2][NT][4];
    float acc[kTilesPerWarp][2][NT][4];
    float sx[NT][4];
#pragma unroll
    for (int w = 0; w < kTilesPerWarp; ++w)
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) tot[w][a][j][i] = acc[w][a][j][i] = 0.f;
#pragma unroll
    for (int j = 0; j < NT; ++j) sx[j][0] = sx[j][1] = sx[j][2] = sx[j][3] = 0.f;

    const uint32_t ones[4] = {0x3c003c00u, 0x3c003c00u, 0x3c003c00u, 0x3c003c00u};
    const int      my_t0   = warp * kTilesPerWarp;  // first tile of this warp inside the unit
    // this lane's row address inside an activation tile (ldmatrix: row = lane % 8, matrix = lane / 8)
    const uint32_t x_lane = smem_s + kXRingOff + (lane & 7) * 64 + (((lane >> 3) ^ ((lane >> 1) & 3)) << 4);

    // Every CTA owns whole 128-row groups (an even number of units), so the two units of a group are
    // unrolled: the first fetches {zero, scale}, the second ends the group.
    int jt = u_begin / G, kk = u_begin - jt * G;
    int s = 0, s_fill = ST - 1;  // slot read now / slot refilled now (the one read one unit ago)
    int to_issue = n_units - (ST - 1);  // units the copy front still has to start
    for (int it = 0; it < n_units; it += 2) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            cp_async_wait<ST - 2>();
            if (it == 0 && u == 0) SMALL_TRACE(1);
            // every thread's copies for this unit have landed, and every warp is done with the unit before
            __syncthreads();
            if (to_issue > 0) issue_unit(s_fill, true);
            --to_issue;
            cp_async_commit();

            const unsigned char* sb = smem_raw + (warp * ST + s) * kWarpStage + lane * 16;
            if (u == 0) {
                const __half2* qs = reinterpret_cast<const __half2*>(sb - lane * 16 + 2 * kSlabBytes);
#pragma unroll
                for (int w = 0; w < kTilesPerWarp; ++w) {
#pragma unroll
                    for (int a = 0; a < 2; ++a) {
                        const float2 q_lo = __half22float2(qs[w * 32 + a * 16 + r]);      // {64 + z, s} of row r
                        const float2 q_hi = __half22float2(qs[w * 32 + a * 16 + r + 8]);  // row r + 8
                        zl[w][a] = 960.f + q_lo.x;           // 1024 + z
                        zh[w][a] = 16.f * q_hi.x;            // 1024 + 16 z
                        sl[w][a] = q_lo.y;
                        sh[w][a] = q_hi.y * 0.0625f;
                    }
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const bool fresh = (u == 0 && h == 0);  // first slab of the group: accumulators start at zero
                uint32_t   bf[NT][4];
#pragma unroll
                for (int j = 0; j < NT; ++j) load_x_frag(bf[j], x_lane + s * kXUnit + h * kXSlab + j * 512);
                // group sums of the activations, in the accumulator layout (every row alike)
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    if (fresh) {
                        mma_m16n8k16_init(sx[j], ones, bf[j][0], bf[j][1]);
                    }
                    else {
                        mma_m16n8k16(sx[j], ones, bf[j][0], bf[j][1]);
                    }
                    mma_m16n8k16(sx[j], ones, bf[j][2], bf[j][3]);
                }
                // all eight fragments of the slab first (independent chains the scheduler can
                // interleave), then the MMAs, k halves outermost so that back-to-back MMAs hit
                // different accumulators
                uint32_t af[kTilesPerWarp][4][4];
#pragma unroll
                for (int w = 0; w < kTilesPerWarp; ++w) {
                    const uint4    wq    = *reinterpret_cast<const uint4*>(sb + h * kSlabBytes + w * kTileBytes);
                    const uint32_t wv[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
                    for (int wi = 0; wi < 4; ++wi) unpack_s4_biased(wv[wi], af[w][wi]);
                }
#pragma unroll
                for (int k16 = 0; k16 < 2; ++k16) {
#pragma unroll
                    for (int w = 0; w < kTilesPerWarp; ++w) {
#pragma unroll
                        for (int a = 0; a < 2; ++a) {
#pragma unroll
                            for (int j = 0; j < NT; ++j) {
                                if (fresh && k16 == 0) {
                                    mma_m16n8k16_init(acc[w][a][j], af[w][2 * k16 + a], bf[j][0], bf[j][1]);
                                }
                                else {
                                    mma_m16n8k16(acc[w][a][j], af[w][2 * k16 + a], bf[j][2 * k16], bf[j][2 * k16 + 1]);
                                }
                            }
                        }
                    }
                }
            }
            s      = (s == ST - 1) ? 0 : s + 1;
            s_fill = (s_fill == ST - 1) ? 0 : s_fill + 1;
        }

        // ---- end of the group: remove offsets and zero point, apply the scale ----------------------
#pragma unroll
        for (int w = 0; w < kTilesPerWarp; ++w)
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    tot[w][a][j][0] = fmaf(sl[w][a], fmaf(-zl[w][a], sx[j][0], acc[w][a][j][0]), tot[w][a][j][0]);
                    tot[w][a][j][1] = fmaf(sl[w][a], fmaf(-zl[w][a], sx[j][1], acc[w][a][j][1]), tot[w][a][j][1]);
                    tot[w][a][j][2] = fmaf(sh[w][a], fmaf(-zh[w][a], sx[j][0], acc[w][a][j][2]), tot[w][a][j][2]);
                    tot[w][a][j][3] = fmaf(sh[w][a], fmaf(-zh[w][a], sx[j][1], acc[w][a][j][3]), tot[w][a][j][3]);
                }
        if (it + 2 >= n_units) SMALL_TRACE(2);
        const int  this_jt = jt;
        const int  tile0   = jt * kTilesPerUnit;
        const int  ntw     = min(kTilesPerUnit, n_tiles32 - tile0) - my_t0;  // tiles of this warp that exist
        const bool seg_end = (it + 2 >= n_units) || (kk + 2 == G);
        kk += 2;
        if (kk == G) {
            kk = 0;
            ++jt;
        }
        if (!seg_end) {
            continue;
        }

        // ---- segment end: publish this CTA's part of column tile this_jt --------------------------
        const int c_first = (this_jt * G) / upc;
        const int c_last  = ((this_jt + 1) * G - 1) / upc;
        const int n_split = c_last - c_first + 1;
        const int n_cols  = min(kTilesPerUnit, n_tiles32 - tile0) * kColsPerTile;
        const int col0    = tile0 * kColsPerTile;

        if (n_split == 1) {
            // this CTA saw the whole K range: straight from registers to C
#pragma unroll
            for (int w = 0; w < kTilesPerWarp; ++w) {
                if (w < ntw) {
#pragma unroll
                    for (int a = 0; a < 2; ++a)
#pragma unroll
                        for (int j = 0; j < NT; ++j)
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int   n = col0 + (my_t0 + w) * kColsPerTile + a * 16 + r + (i >> 1) * 8;
                                const int   t = t0 + j * 8 + 2 * c + (i & 1);
                                const float v = tot[w][a][j][i];
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
        }
        else {
            // (cta + column tile) is unique per segment: along the unit order either the CTA or the
            // column tile advances, never both backwards.
            float* slot = p.workspace
                          + ((size_t)blockIdx.y * p.slots_per_chunk + blockIdx.x + this_jt) * (size_t)(TP * kUnitCols);
#pragma unroll
            for (int w = 0; w < kTilesPerWarp; ++w)
#pragma unroll
                for (int a = 0; a < 2; ++a)
#pragma unroll
                    for (int j = 0; j < NT; ++j)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int n = (my_t0 + w) * kColsPerTile + a * 16 + r + (i >> 1) * 8;
                            const int t = j * 8 + 2 * c + (i & 1);
                            if (t < t_rows) __stcg(slot + t * kUnitCols + n, tot[w][a][j][i]);
                        }
            // the barrier orders every thread's stores before the fence of the one thread that takes the ticket
            __syncthreads();
            if (tid == 0) {
                __threadfence();
                int*      counter = p.counters + (size_t)blockIdx.y * p.n_col_tiles + this_jt;
                const int ticket  = atomicAdd(counter, 1);
                const int is_last = (ticket == n_split - 1);
                if (is_last) {
                    *counter = 0;  // self-reset for the next launch
                }
                s_flag[0] = is_last;
            }
            __syncthreads();
            if (s_flag[0] != 0) {
                __threadfence();
                // fixed-order reduction of every CTA's partial: four adjacent columns per thread, the
                // loads of up to eight slots in flight together
                constexpr int kBatch = 8;
                const int     quads  = n_cols / 4;
                const float*  slot0  = p.workspace + (size_t)blockIdx.y * p.slots_per_chunk * (size_t)(TP * kUnitCols);
                for (int i = tid; i < t_rows * quads; i += kThreads) {
                    const int    t    = i / quads;
                    const int    n    = (i - t * quads) * 4;
                    const float* base = slot0 + t * kUnitCols + n;
                    float4       v    = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int cc = c_first; cc <= c_last; cc += kBatch) {
                        float4 part[kBatch];
#pragma unroll
                        for (int e = 0; e < kBatch; ++e) {
                            part[e] = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (cc + e <= c_last) {
                                part[e] = __ldcg(reinterpret_cast<const float4*>(base + (size_t)(cc + e + this_jt) * (TP * kUnitCols)));
                            }
                        }
#pragma unroll
                        for (int e = 0; e < kBatch; ++e) {
                            v.x += part[e].x;  // absent slots add +0
                            v.y += part[e].y;
                            v.z += part[e].z;
                            v.w += part[e].w;
                        }
                    }
                    const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
                    if (p.fused_silu) {
                        const float2 u0 = __half22float2(h0), u1 = __half22float2(h1);
                        const float  s0 = u0.x / (1.f + __expf(-u0.x)), s1 = u1.x / (1.f + __expf(-u1.x));
                        *reinterpret_cast<__half2*>(p.C + (size_t)(t0 + t) * (p.N / 2) + (col0 + n) / 2) =
                            __floats2half2_rn(s0 * u0.y, s1 * u1.y);
                    }
                    else {
                        __half2* dst = reinterpret_cast<__half2*>(p.C + (size_t)(t0 + t) * p.N + col0 + n);
                        dst[0]       = h0;
                        dst[1]       = h1;
                    }
                }
            }
            __syncthreads();  // s_flag is reused by the next segment
        }
#pragma unroll
        for (int w = 0; w < kTilesPerWarp; ++w)
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) tot[w][a][j][i] = 0.f;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
#ifdef TM_B200_GEMM_TRACE
    SMALL_TRACE(3);
    __syncthreads();
    if (tid == 0 && blockIdx.x == 0 && blockIdx.y == 0) atomicAdd(&g_small_launch, 1);
#endif
}

// ---- column-owner variant for up to 8 tokens --------------------------------------------------------------------
// Where the weight has at least as many column strips as the device has SMs (the qkv and gate/up projections),
// nothing needs to be split between CTAs: a CTA owns one strip of TILES packed tiles (32 or 64 columns: 512 B or 1 KB
// contiguous per 32-row slab) over the whole K range, its eight warps take the 128-row quantisation groups round
// robin (warp w: groups w, w + 8, ...), each through a private cp.async ring of whole groups (2 KB of weight per tile
// + its {zero, scale}), and the eight partial sums meet once in shared memory, in a fixed order.  No scratch, no
// tickets, no fence, no CTA that reduces for others.  The ring is as deep as the plan says: with 32-column strips and
// K = 4096 every byte the CTA will read is requested before the first one is used.  The activations (a few KB, the
// same for every CTA) come as B fragments straight from L1 / L2.  The arithmetic per group is that of the kernel
// above.
// kOne: a single token.  The group sums of the activations then come from plain adds (every lane takes four of the
// group's 128 values, a butterfly over the warp sums them) instead of two more MMAs per slab.
__device__ __forceinline__ void cp_async_wait_pending(int n)
{
    switch (n) {
        case 0: cp_async_wait<0>(); break;
        case 1: cp_async_wait<1>(); break;
        case 2: cp_async_wait<2>(); break;
        case 3: cp_async_wait<3>(); break;
        case 4: cp_async_wait<4>(); break;
        case 5: cp_async_wait<5>(); break;
        case 6: cp_async_wait<6>(); break;
        default: cp_async_wait<7>(); break;  // more may be pending than asked for: waiting for fewer is always right
    }
}

__host__ __device__ constexpr int co_stage_bytes(int tiles) { return tiles * (4 * kTileBytes + 128); }  // four slabs + {zero, scale} per tile

template<int TILES, bool kOne>
__global__ void __launch_bounds__(kThreads, TILES == 1 ? 3 : 2) gemm_s4_f16_cols_kernel(GemmSmallParams p)
{
    constexpr int kStage = co_stage_bytes(TILES);
    constexpr int kSlab  = TILES * kTileBytes;  // one 32-row slab of the strip
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t smem_s = smem_u32(smem_raw);
    const int      tid    = threadIdx.x;
    const int      warp   = tid >> 5;
    const int      lane   = tid & 31;
    const int      r      = lane >> 2;
    const int      c      = lane & 3;
    const int      ST     = p.stages;  // ring slots per warp

    const int    n_tiles32   = p.N / kColsPerTile;
    const int    G           = p.K / 128;
    const int    tile0       = blockIdx.x * TILES;
    const int    step        = (TILES == 2 && tile0 + 1 < n_tiles32) ? kTileBytes : 0;  // a strip at the edge of N: one tile, read twice
    const size_t slab_stride = (size_t)n_tiles32 * kTileBytes;
    const int    n_groups    = warp < G ? (G - 1 - warp) / kWarps + 1 : 0;

    const uint32_t       ring_s = smem_s + warp * (ST * kStage);
    const unsigned char* i_w    = p.A + ((size_t)(4 * warp) * n_tiles32 + tile0) * kTileBytes + lane * 16;
    const unsigned char* i_q    = p.Q + ((size_t)warp * p.N + (size_t)tile0 * kColsPerTile) * 4 + lane * 16;
    const bool           i_qok  = lane < 8 * TILES && tile0 * kColsPerTile + lane * 4 < p.N;
    auto issue_group = [&](int slot) {
        const uint32_t dst = ring_s + slot * kStage;
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            cp_async16(dst + h * kSlab + lane * 16, i_w + h * slab_stride);
            if (TILES == 2) cp_async16(dst + h * kSlab + kTileBytes + lane * 16, i_w + h * slab_stride + step);
        }
        if (i_qok) cp_async16(dst + 4 * kSlab + lane * 16, i_q);
        cp_async_commit();
        i_w += (size_t)(4 * kWarps) * slab_stride;  // this warp's next group: eight groups further down
        i_q += (size_t)kWarps * p.N * 4;
    };
    // the packed weight is written by no kernel: its first copies start ahead of the wait for the kernel before
    int issued = 0;
    for (; issued < ST && issued < n_groups; ++issued) issue_group(issued);
    pdl_wait();
    pdl_launch_dependents();

    // B fragments: token = fragment row (tokens beyond T repeat the last one: their columns are never stored)
    const uint32_t* x_row = reinterpret_cast<const uint32_t*>(p.X + (size_t)min(r, p.T - 1) * p.K * 2) + c;

    float tot[TILES][2][4];
#pragma unroll
    for (int w = 0; w < TILES; ++w)
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int i = 0; i < 4; ++i) tot[w][a][i] = 0.f;
    const uint32_t ones[4] = {0x3c003c00u, 0x3c003c00u, 0x3c003c00u, 0x3c003c00u};

    int slot = 0;  // ring slot of group `it`
    for (int it = 0; it < n_groups; ++it) {
        const int g = warp + it * kWarps;
        // the group's activations: k = 128 g + 32 h + 8 i + 2 c, + 1
        uint32_t bf[4][4];
#pragma unroll
        for (int h = 0; h < 4; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i) bf[h][i] = __ldg(x_row + g * 64 + h * 16 + i * 4);
        uint2 xs = make_uint2(0u, 0u);
        if (kOne) xs = __ldg(reinterpret_cast<const uint2*>(p.X) + g * 32 + lane);  // this lane's four values of the group
        // copies complete in the order they were committed: group `it` has landed once at most issued - it - 1 are pending
        cp_async_wait_pending(issued - it - 1);
        __syncwarp();  // every lane's copies of this group have landed, and every lane is done with the group before
        if (it >= 1 && issued < n_groups) {
            issue_group(slot == 0 ? ST - 1 : slot - 1);  // the slot of the group before: free now
            ++issued;
        }

        const unsigned char* sb = smem_raw + warp * (ST * kStage) + slot * kStage;
        const __half2*       qs = reinterpret_cast<const __half2*>(sb + 4 * kSlab);
        float zl[TILES][2], zh[TILES][2], sl[TILES][2], sh[TILES][2];
#pragma unroll
        for (int w = 0; w < TILES; ++w) {
#pragma unroll
            for (int a = 0; a < 2; ++a) {
                const float2 q_lo = __half22float2(qs[w * 32 + a * 16 + r]);      // {64 + z, s} of row r
                const float2 q_hi = __half22float2(qs[w * 32 + a * 16 + r + 8]);  // row r + 8
                zl[w][a] = 960.f + q_lo.x;  // 1024 + z
                zh[w][a] = 16.f * q_hi.x;   // 1024 + 16 z
                sl[w][a] = q_lo.y;
                sh[w][a] = q_hi.y * 0.0625f;
            }
        }
        float acc[TILES][2][4];
        float sx[4];
        if (kOne) {
            float part = (__half2float(__ushort_as_half((unsigned short)(xs.x & 0xffffu))) + __half2float(__ushort_as_half((unsigned short)(xs.x >> 16))))
                         + (__half2float(__ushort_as_half((unsigned short)(xs.y & 0xffffu))) + __half2float(__ushort_as_half((unsigned short)(xs.y >> 16))));
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            sx[0] = sx[1] = sx[2] = sx[3] = part;  // every column is the one token
        }
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            if (!kOne) {
                // group sum of the activations, in the accumulator layout (every row alike)
                if (h == 0) {
                    mma_m16n8k16_init(sx, ones, bf[h][0], bf[h][1]);
                }
                else {
                    mma_m16n8k16(sx, ones, bf[h][0], bf[h][1]);
                }
                mma_m16n8k16(sx, ones, bf[h][2], bf[h][3]);
            }
            uint32_t af[TILES][4][4];
#pragma unroll
            for (int w = 0; w < TILES; ++w) {
                const uint4    wq    = *reinterpret_cast<const uint4*>(sb + h * kSlab + w * kTileBytes + lane * 16);
                const uint32_t wv[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) unpack_s4_biased(wv[wi], af[w][wi]);
            }
#pragma unroll
            for (int k16 = 0; k16 < 2; ++k16) {
#pragma unroll
                for (int w = 0; w < TILES; ++w) {
#pragma unroll
                    for (int a = 0; a < 2; ++a) {
                        if (h == 0 && k16 == 0) {
                            mma_m16n8k16_init(acc[w][a], af[w][2 * k16 + a], bf[h][0], bf[h][1]);
                        }
                        else {
                            mma_m16n8k16(acc[w][a], af[w][2 * k16 + a], bf[h][2 * k16], bf[h][2 * k16 + 1]);
                        }
                    }
                }
            }
        }
        // end of the group: remove offsets and zero point, apply the scale
#pragma unroll
        for (int w = 0; w < TILES; ++w)
#pragma unroll
            for (int a = 0; a < 2; ++a) {
                tot[w][a][0] = fmaf(sl[w][a], fmaf(-zl[w][a], sx[0], acc[w][a][0]), tot[w][a][0]);
                tot[w][a][1] = fmaf(sl[w][a], fmaf(-zl[w][a], sx[1], acc[w][a][1]), tot[w][a][1]);
                tot[w][a][2] = fmaf(sh[w][a], fmaf(-zh[w][a], sx[0], acc[w][a][2]), tot[w][a][2]);
                tot[w][a][3] = fmaf(sh[w][a], fmaf(-zh[w][a], sx[1], acc[w][a][3]), tot[w][a][3]);
            }
        slot = (slot == ST - 1) ? 0 : slot + 1;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();  // the rings are free: they now hold the eight warps' partial sums, [warp][TILES x 8 values][lane]
    constexpr int kVals = TILES * 8;
    float*        red   = reinterpret_cast<float*>(smem_raw);
#pragma unroll
    for (int w = 0; w < TILES; ++w)
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int i = 0; i < 4; ++i) red[(warp * kVals + (w * 2 + a) * 4 + i) * 32 + lane] = tot[w][a][i];
    __syncthreads();
    for (int e = warp; e < kVals; e += kWarps) {
        float v = 0.f;
#pragma unroll
        for (int wp = 0; wp < kWarps; ++wp) v += red[(wp * kVals + e) * 32 + lane];  // fixed order
        const int  w     = e >> 3, a = (e >> 2) & 1, i = e & 3;
        const int  n     = (tile0 + w) * kColsPerTile + a * 16 + r + (i >> 1) * 8;
        const int  t     = 2 * c + (i & 1);
        const bool valid = tile0 + w < n_tiles32 && t < p.T;
        if (p.fused_silu) {
            // kernels/gemm_s_f16/gemm_s4_f16.cu:31-43 on the fp16-rounded pair; the partner column n ^ 1 lives in lane ^ 4
            const float mine  = __half2float(__float2half_rn(v));
            const float other = __shfl_xor_sync(0xffffffffu, mine, 4);
            if ((r & 1) == 0 && valid) {
                const float silu = mine / (1.f + __expf(-mine));
                p.C[(size_t)t * (p.N / 2) + n / 2] = __float2half_rn(silu * other);
            }
        }
        else if (valid) {
            p.C[(size_t)t * p.N + n] = __float2half_rn(v);
        }
    }
}

}  // namespace

size_t gemm_small_smem_bytes(int nt)
{
    const int st = stages_for(nt);
    return (size_t)st * (kWarps * kWarpStage + 2 * nt * 512) + 16;
}

GemmSmallPlan gemm_small_plan(int N, int T, int K, int sm_count, int max_smem, int cols_variant)
{
    (void)max_smem;
    GemmSmallPlan pl{};
    pl.nt = T <= 8 ? 1 : (T <= 16 ? 2 : 4);
    const int tp   = pl.nt * 8;
    pl.t_chunks    = (T + tp - 1) / tp;
    pl.n_col_tiles = (N / kColsPerTile + kTilesPerUnit - 1) / kTilesPerUnit;
    const int G    = K / kUnitRows;
    pl.total_units = pl.n_col_tiles * G;
    const int slots = sm_count * ctas_per_sm_for(pl.nt);  // co-resident CTAs
    int       ctas  = slots < pl.total_units ? slots : pl.total_units;
    pl.units_per_cta    = (pl.total_units + ctas - 1) / ctas;
    pl.units_per_cta += pl.units_per_cta & 1;  // whole 128-row groups: two units
    pl.ctas             = (pl.total_units + pl.units_per_cta - 1) / pl.units_per_cta;
    pl.slots_per_chunk  = pl.ctas + pl.n_col_tiles;
    pl.stages           = stages_for(pl.nt);
    pl.smem_bytes       = gemm_small_smem_bytes(pl.nt);
    pl.workspace_floats = (size_t)pl.t_chunks * pl.slots_per_chunk * tp * kUnitCols;
    pl.counter_ints     = (size_t)pl.t_chunks * pl.n_col_tiles;
    // Enough column strips to give every SM one: the column-owner kernel, which splits nothing between CTAs.  The
    // scratch sizes above stay (unused) so that a caller's workspace is sized the same way for both kernels.
    // Variant 1: 32-column strips, three CTAs per SM, a ring of up to four groups per warp (the whole K range of a
    // 4096-row weight is requested at once); variant 2: 64-column strips, two CTAs per SM, three groups.
    const int tiles  = cols_variant == 2 ? 2 : 1;
    const int strips = (N / kColsPerTile + tiles - 1) / tiles;
    // Measured on the 7B shapes: with all strips resident at once (qkv: 384 strips for 444 slots) it wins at every
    // token count up to 8; with more strips than slots (gate/up: 688) it wins at one token, ties up to four and loses at
    // eight, where every CTA re-reads 64 KB of activations.
    const int  co_slots   = sm_count * (tiles == 2 ? 2 : 3);
    const bool worthwhile = strips >= sm_count && (strips <= co_slots || T == 1);
    pl.cols_tiles         = (cols_variant != 0 && T <= 8 && worthwhile) ? tiles : 0;
    if (pl.cols_tiles) {
        const int per_warp = (K / 128 + kWarps - 1) / kWarps;  // groups of the busiest warp
        pl.ctas       = strips;
        pl.stages     = tiles == 2 ? 3 : (per_warp < 2 ? 2 : (per_warp > 4 ? 4 : per_warp));
        pl.smem_bytes = (size_t)kWarps * pl.stages * co_stage_bytes(tiles);
    }
    return pl;
}

cudaError_t gemm_small_prepare(int max_smem)
{
    cudaError_t e;
    e = cudaFuncSetAttribute(gemm_s4_f16_small_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(gemm_s4_f16_small_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e != cudaSuccess) return e;
    constexpr int kCoSmemMax = kWarps * 4 * co_stage_bytes(2);
    e = cudaFuncSetAttribute(gemm_s4_f16_cols_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCoSmemMax);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(gemm_s4_f16_cols_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCoSmemMax);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(gemm_s4_f16_cols_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCoSmemMax);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(gemm_s4_f16_cols_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCoSmemMax);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(gemm_s4_f16_small_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
}

cudaError_t gemm_small_launch(const GemmSmallPlan& pl, GemmSmallParams p, cudaStream_t st, bool pdl)
{
    p.units_per_cta   = pl.units_per_cta;
    p.total_units     = pl.total_units;
    p.slots_per_chunk = pl.slots_per_chunk;
    p.n_col_tiles     = pl.n_col_tiles;
    p.stages          = pl.stages;
    dim3 grid(pl.ctas, pl.t_chunks);
    dim3 block(kThreads);
    if (pl.cols_tiles == 1) {
        return p.T == 1 ? launch_kernel(gemm_s4_f16_cols_kernel<1, true>, grid, block, pl.smem_bytes, st, pdl, p) :
                          launch_kernel(gemm_s4_f16_cols_kernel<1, false>, grid, block, pl.smem_bytes, st, pdl, p);
    }
    if (pl.cols_tiles == 2) {
        return p.T == 1 ? launch_kernel(gemm_s4_f16_cols_kernel<2, true>, grid, block, pl.smem_bytes, st, pdl, p) :
                          launch_kernel(gemm_s4_f16_cols_kernel<2, false>, grid, block, pl.smem_bytes, st, pdl, p);
    }
    switch (pl.nt) {
        case 1: return launch_kernel(gemm_s4_f16_small_kernel<1>, grid, block, pl.smem_bytes, st, pdl, p);
        case 2: return launch_kernel(gemm_s4_f16_small_kernel<2>, grid, block, pl.smem_bytes, st, pdl, p);
        default: return launch_kernel(gemm_s4_f16_small_kernel<4>, grid, block, pl.smem_bytes, st, pdl, p);
    }
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
