// W4A16 GEMM for more than 16 tokens: tcgen05 tensor-core tiles with the accumulators in TMEM.
//
// A CTA computes C^T tiles of 256 output features (two 128-feature UMMA tiles that share one
// activation slice) x up to 128 tokens.  It is persistent and stream-K balanced over
// (256-feature tile, 128-row quantisation group) units, like the small-token kernel.  Warp roles:
//   warp 0       one lane streams the activation slices: two tensor-map copies (TMA, 128-byte
//                swizzle, tokens beyond T read as zero) per unit, completion on an mbarrier
//   warps 1, 2   one issuer per 128-feature tile (warp 1 also allocates TMEM): an elected lane issues
//                tcgen05.mma (M = 128, N = token tile, K = 16 per instruction, fp16 x fp16 -> fp32, A
//                from TMEM, B from shared memory) and commits completions to mbarriers
//   warps 3..18  two teams of eight, one per 128-feature tile.  Every warp streams its own share of
//                the packed weight through a private cp.async ring and expands it (lop3 nibble
//                unpack, exact (q - z) in fp16) straight into TMEM with tcgen05.st, from where the
//                tensor core takes its A operand (no shared-memory round trip); the same warps read
//                the accumulators back with tcgen05.ld and store C (optionally through the
//                SiLU(gate) * up epilogue) or the split-K partial
// Two variants (template parameter FOLD):
//   FOLD (token tile <= 64)  The tensor core sees the integers (q - z); every 128-row group gets a
//                fresh accumulator (two per team, used in turn) and the expanding warps add it,
//                times the group's scale, to fp32 sums they keep in registers:
//                    y[n][t] += s[g][n] * sum_{k in g} (q - z)[k][n] x[t][k]
//                This takes the scale multiplies out of the expansion (9 instead of 13 instructions
//                per packed word); the weight differs from the reference's fp16_rn((q - z) s) by that
//                one rounding (the products are exact in fp32 here), as in the small-token kernel.
//   !FOLD (token tile 65..128)  The expansion multiplies by the scale in fp16, bit-identical to the
//                reference's dequantised weight (kernels/gemm_s_f16/common.h:115-156, 218-235), and a
//                column tile accumulates over all of its groups in TMEM (two accumulators of 128
//                columns leave no room for per-group accumulators).
// Partial tiles of CTAs that share a column tile meet in scratch memory; every CTA of the tile then
// sums its own share of the feature rows in a fixed order.  Every wait is bounded.
//
// Replaces the large-n end of GemmS4F16::Run (src/turbomind/kernels/gemm_s_f16/gemm_s4_f16.cu:
// 208-234; mma.sync tiles of gemm_template.h:338-444).
#include "common.cuh"
#include "gemm_s4_f16.h"

#include <cuda.h>  // CUtensorMap (types only: the encoder is looked up through the runtime)

#ifdef TM_B200_GEMM_TRACE
// Developer build only (never defined by lmdeploy_b200/build.py): time stamps of selected warps of selected CTAs.
__device__ long long g_tc_trace[8][2048];
__device__ int       g_tc_trace_n[8];
extern "C" __attribute__((visibility("default"))) int tm_dev_gemm_trace(long long* out, int* counts)
{
    cudaMemcpyFromSymbol(out, g_tc_trace, sizeof(long long) * 8 * 2048);
    cudaMemcpyFromSymbol(counts, g_tc_trace_n, sizeof(int) * 8);
    int zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    cudaMemcpyToSymbol(g_tc_trace_n, zero, sizeof(zero));
    return 0;
}
#define TC_TRACE(row, tag, unit)                                                                                       \
    do {                                                                                                                   \
        if ((row) >= 0 && (threadIdx.x & 31) == 0 && trace_i < 2046) {                                                     \
            g_tc_trace[row][trace_i]     = ((long long)(tag) << 32) | (unsigned)(unit);                                    \
            g_tc_trace[row][trace_i + 1] = clock64();                                                                      \
            trace_i += 2;                                                                                                  \
            g_tc_trace_n[row] = trace_i;                                                                                   \
        }                                                                                                                  \
    } while (0)
#else
#define TC_TRACE(row, tag, unit) do { } while (0)
#endif

namespace tmb {
namespace {

constexpr int kTileN     = 128;  // output features per UMMA tile (UMMA M)
constexpr int kTeams     = 2;    // UMMA tiles per CTA tile
constexpr int kSuperN    = kTileN * kTeams;
constexpr int kGroup     = 128;  // K extent of a unit
constexpr int kTileBytes = 512;
constexpr int kACols     = kGroup / 2;           // TMEM columns of one expanded weight stage (128 k as fp16 pairs)
constexpr int kWarpStage = 2 * kTileBytes + 128; // per expanding warp and unit: 2 x 512 B of weight + 32 {zero, scale}
constexpr int kWST       = 5;                    // stages of those private rings (cp.async groups in flight <= 4)
constexpr int kASTMax    = 2;                    // expanded-weight stages per team (in TMEM)
constexpr int kXSTMax    = 6;                    // activation stages
constexpr int kTeamWarps = 8;
constexpr int kDqWarps   = kTeams * kTeamWarps;
constexpr int kDqThreads = kDqWarps * 32;
constexpr int kDqWarp0   = 1 + kTeams;           // first expanding warp
constexpr int kThreads   = (kDqWarp0 + kDqWarps) * 32;
constexpr int kTmemCols  = 512;                  // accumulators + expanded-weight stages, power of two

struct Bars {
    uint64_t a_full[kTeams][kASTMax], a_empty[kTeams][kASTMax];
    uint64_t x_full[kXSTMax], x_empty[kXSTMax];
    uint64_t acc_full[kTeams][2], acc_empty[kTeams][2];  // per team and accumulator
    uint32_t tmem_base;
    int      flag;
};

__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr)
{
    // K-major, 128-byte swizzle: 8-row groups 1024 B apart (SBO), leading offset 1, descriptor version 1
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46)
           | ((uint64_t)2 << 61);
}

// D(tmem) (+)= A(tmem) x B(smem descriptor)
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a),
        "l"(desc_b),
        "r"(idesc),
        "r"(accumulate)
        : "memory");
}

// 16 TMEM lanes x 8 columns from an mma A-fragment: regs = {rows r | k pair c, rows r+8 | k pair c,
// rows r | k pair c+4, rows r+8 | k pair c+4} with r = lane / 4, c = lane % 4
__device__ __forceinline__ void tmem_st_16x128b_x2(uint32_t taddr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3)
{
    asm volatile("tcgen05.st.sync.aligned.16x128b.x2.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
                 : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// One box of the activation tensor map -> shared memory, completion counted on an mbarrier
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(map)),
                 "r"(x),
                 "r"(y),
                 "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8])
{
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ uint32_t hmul2_ftz(uint32_t a, uint32_t b)
{
    uint32_t r;
    asm("mul.ftz.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// Bounded wait of a whole warp; on a time-out the warp records `bit` and plays dead from then on.
__device__ __forceinline__ void warp_wait(uint64_t* bar, uint32_t parity, bool& dead, unsigned* status, unsigned bit)
{
    if (dead) return;
    // one lane polls; the shuffle hands the outcome (and, as a warp-level sync, the ordering) to the rest
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity) ? 1 : 0;  // suspending wait: leaves the issue slots to the busy warps
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok) {
        if ((threadIdx.x & 31) == 0) atomicOr(status, bit);
        dead = true;
    }
}

// eight fp32 columns of this thread's TMEM lane, no wait (pair with tmem_ld_wait)
__device__ __forceinline__ void tmem_ld8_nowait(uint32_t taddr, float* v)
{
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template<bool FOLD>
__global__ void __launch_bounds__(kThreads, 1) gemm_s4_f16_tc_kernel(GemmTcParams p, const __grid_constant__ CUtensorMap x_map)
{
    const int kXST = p.x_stages;
    constexpr int kAST = 2;         // expanded-weight stages per team (in TMEM)
    const int accS = p.acc_stride;  // TMEM columns of one accumulator
    extern __shared__ unsigned char smem_dyn[];
    // tiles the tensor core reads must sit on 1024-byte boundaries (the swizzle is a function of
    // the address bits)
    const uint32_t raw  = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* sm   = smem_dyn + (base - raw);

    const int TT      = p.token_tile;             // UMMA N, multiple of 16, <= 128 (<= 64 with FOLD)
    const int x_bytes = 2 * TT * 128;             // two K blocks of TT rows x 128 B
    unsigned char* x_ring = sm;                                   // kXST x x_bytes (multiples of 1024)
    unsigned char* w_ring = x_ring + kXST * x_bytes;              // kDqWarps x kWST x kWarpStage
    Bars*          bars   = reinterpret_cast<Bars*>(w_ring + kWST * kDqWarps * kWarpStage);

    const int tid  = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
#ifdef TM_B200_GEMM_TRACE
    int trow = -1, trace_i = 0;
    if (blockIdx.x == 0 && blockIdx.y == 0) trow = warp == 0 ? 0 : warp == 1 ? 1 : warp == kDqWarp0 ? 2 : warp == kDqWarp0 + 8 ? 3 : -1;
    if (blockIdx.x == 64 && blockIdx.y == 0) trow = warp == kDqWarp0 ? 4 : warp == 1 ? 5 : warp == kDqWarp0 + 5 ? 6 : -1;
    if (blockIdx.x == gridDim.x - 1 && blockIdx.y == 0) trow = warp == kDqWarp0 ? 7 : trow;
    TC_TRACE(trow, 1, 0);
#endif

    const int t0     = blockIdx.y * 128;
    const int t_rows = min(TT, p.T - t0);

    const int G         = p.K / kGroup;
    const int upc       = p.units_per_cta;
    const int u_begin   = blockIdx.x * upc;
    const int n_units   = min(u_begin + upc, p.total_units) - u_begin;
    const int n_tiles32 = p.N / 32;

    // ---- expanding warps: identity and the state of their copy front ---------------------------
    const int  dw   = warp - kDqWarp0; // 0..15 for the expanding warps
    const int  m_dq = (dw >> 3) & 1;   // team = 128-feature tile of the unit
    const int  q    = warp & 3;        // TMEM lane quarter this warp may access = its 32-feature tile
    const int  kh   = (dw >> 2) & 1;   // which pair of 32-row slabs of the group it expands,
                                       // and which half of the token columns it drains
    // private ring of this warp: per unit its own 2 x 512 B of packed weight (32-feature tile,
    // 32-row slabs 2 kh, 2 kh + 1 of the group) + the 128 B of {zero, scale} of its 32 features
    const uint32_t       my_ring   = base + (uint32_t)(w_ring - sm) + (uint32_t)(dw < 0 ? 0 : dw) * kWST * kWarpStage;
    const unsigned char* my_ring_g = w_ring + (dw < 0 ? 0 : dw) * kWST * kWarpStage;
    // the copy front runs kWST - 1 units ahead of the expansion: this lane's 16 bytes of the warp's
    // first slab and of the {zero, scale} row.  A warp whose tile lies beyond N re-reads the last
    // tile; what it produces is never stored.
    int                  i_js = u_begin / G, i_g = u_begin - i_js * G;
    const unsigned char* i_w  = nullptr;
    const unsigned char* i_q  = nullptr;
    const size_t         slab_b  = (size_t)n_tiles32 * kTileBytes;  // bytes between 32-row slabs
    const size_t         q_row_b = (size_t)p.N * 4;                 // bytes between {zero, scale} rows
    auto i_seek = [&]() {
        const int tile = min((i_js * kTeams + m_dq) * 4 + q, n_tiles32 - 1);
        i_w = p.A + (((size_t)i_g * 4 + kh * 2) * n_tiles32 + tile) * kTileBytes + lane * 16;
        i_q = p.Q + ((size_t)i_g * p.N + (size_t)tile * 32) * 4 + (lane & 7) * 16;
    };
    int to_issue = n_units;
    auto issue_unit = [&](int stage) {
        const uint32_t dst = my_ring + stage * kWarpStage + lane * 16;
        cp_async16(dst, i_w);
        cp_async16(dst + kTileBytes, i_w + slab_b);
        if (lane < 8) cp_async16(dst + 2 * kTileBytes, i_q);
        i_w += 4 * slab_b;
        i_q += q_row_b;
        if (++i_g == G) {
            i_g = 0;
            ++i_js;
            i_seek();
        }
    };
    if (dw >= 0) {
        // The packed weights are written by no kernel: their first copies start at once, ahead of the
        // barrier and TMEM set-up and of the wait for the kernel before this one.
        i_seek();
#pragma unroll
        for (int sidx = 0; sidx < kWST - 1; ++sidx) {
            if (to_issue > 0) issue_unit(sidx);
            --to_issue;
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
    }

    if (tid == 0) {
        for (int m = 0; m < kTeams; ++m) {
            for (int s = 0; s < kASTMax; ++s) {
                mbar_init(&bars->a_full[m][s], kTeamWarps);
                mbar_init(&bars->a_empty[m][s], 1);
            }
            for (int b = 0; b < 2; ++b) {
                mbar_init(&bars->acc_full[m][b], 1);
                mbar_init(&bars->acc_empty[m][b], kTeamWarps);
            }
        }
        for (int s = 0; s < kXSTMax; ++s) {
            mbar_init(&bars->x_full[s], 1);
            mbar_init(&bars->x_empty[s], kTeams);
        }
        fence_mbar_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                     "n"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem   = bars->tmem_base;
    TC_TRACE(trow, 2, 0);
    // TMEM columns: accumulators [team][FOLD ? 2 : 1] x accS, then the expanded-weight stages
    const uint32_t a_base = tmem + kTeams * (FOLD ? 2 : 1) * accS;

    if (warp == 0) {
        // ================================================================== activation loader
        // slice [TT tokens][128 k] of a group -> two 64-wide K blocks, rows of 128 B with their 16-byte
        // chunks XOR-swizzled by (row & 7): the layout the tensor core expects and the one a tensor-map
        // copy with 128-byte swizzle writes.  One slice serves both feature tiles of the unit.
        bool dead = false;
        int  g    = u_begin % G;
        pdl_wait();  // the activations come from the kernel before this one
        pdl_launch_dependents();
        for (int it = 0; it < n_units; ++it) {
            const int sx = it % kXST;
            TC_TRACE(trow, 10, it);
            if (it >= kXST) warp_wait(&bars->x_empty[sx], ((it / kXST) - 1) & 1, dead, p.status, kStatusGemmPipeWait);
            if (!dead && lane == 0) {
                const uint32_t xb = base + (uint32_t)(x_ring - sm) + sx * x_bytes;
                mbar_arrive_expect_tx(&bars->x_full[sx], (uint32_t)x_bytes);
                tma_load_2d(xb, &x_map, g * kGroup, t0, &bars->x_full[sx]);
                tma_load_2d(xb + TT * 128, &x_map, g * kGroup + 64, t0, &bars->x_full[sx]);
            }
            __syncwarp();
            if (++g == G) g = 0;
        }
    }
    else if (warp <= kTeams) {
        // ================================================================== MMA issuers, one per team
        // A single lane runs the whole loop: waits, eight MMAs, commits.  Nothing here needs the warp.
        if (lane == 0) {
            const int      m       = warp - 1;
            const uint32_t idesc   = (1u << 4) | ((uint32_t)(TT >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);
            const uint32_t kb_step = (uint32_t)(TT * 128) >> 4;  // descriptor units (16 B) between the two K blocks
            const uint64_t d_ring  = make_desc(base + (uint32_t)(x_ring - sm));
            const uint32_t x_step  = (uint32_t)x_bytes >> 4;
            int  seg_idx = 0;
            bool first   = true;  // !FOLD: first MMA of the current segment overwrites the accumulator
            int  g       = u_begin % G;
            int  sa = 0, sx = 0;
            uint32_t pa = 0, px = 0;  // phase parity of the weight / activation rings
            for (int it = 0; it < n_units; ++it) {
                bool ok = true;
                const int buf = FOLD ? (it & 1) : 0;
                if (FOLD) {
                    // the expanding warps must have read what this accumulator held two units ago
                    if (it >= 2) ok = mbar_wait(&bars->acc_empty[m][buf], ((it >> 1) - 1) & 1);
                }
                else if (first && seg_idx > 0) {
                    // the epilogue of the previous segment must have drained the accumulator
                    ok = mbar_wait(&bars->acc_empty[m][0], (seg_idx - 1) & 1);
                }
                ok = ok && mbar_wait(&bars->x_full[sx], px) && mbar_wait(&bars->a_full[m][sa], pa);
                if (!ok) {
                    atomicOr(p.status, kStatusGemmPipeWait);
                    break;
                }
                tc_fence_after();
                TC_TRACE(trow, 20, it);
                const uint32_t d_tmem = tmem + (uint32_t)((FOLD ? m * 2 + buf : m) * accS);
                const uint32_t a_tmem = a_base + (m * kAST + sa) * kACols;
                const uint64_t d0     = d_ring + (uint64_t)(sx * x_step);
                uint32_t       accum  = (FOLD || first) ? 0u : 1u;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    // K block j / 4, 16-wide K step j % 4 (32 bytes inside the 128-byte rows)
                    umma_f16_ts(d_tmem, a_tmem + j * 8, d0 + (uint64_t)((j >> 2) * kb_step + (j & 3) * 2), idesc, accum);
                    accum = 1u;
                }
                umma_commit(&bars->a_empty[m][sa]);
                umma_commit(&bars->x_empty[sx]);
                TC_TRACE(trow, 21, it);
                first = false;
                if (FOLD) {
                    umma_commit(&bars->acc_full[m][buf]);
                }
                else if ((it == n_units - 1) || (g == G - 1)) {
                    umma_commit(&bars->acc_full[m][0]);
                    ++seg_idx;
                    first = true;
                }
                if (++g == G) g = 0;
                if (++sa == kAST) { sa = 0; pa ^= 1; }
                if (++sx == kXST) { sx = 0; px ^= 1; }
            }
        }
        __syncwarp();
    }
    else {
        // ================================================================== expand + epilogue
        const int  m    = m_dq;
        const int  r    = lane >> 2;
        bool       dead = false;
        int        seg_idx = 0;
        const int  dtid = tid - kDqWarp0 * 32;

        // What follows reads and writes scratch, tickets and the output, which the kernel before this
        // one may still be using.
        pdl_wait();

        // split-K: [slot][128 tokens][256 feature rows] fp32 partial tiles (a warp touches 128 contiguous
        // bytes per token), per tile a count of CTAs whose partial is complete and a count of CTAs that
        // are done reading.  Tiles this CTA shares with others are reduced after its last unit.
        float* const slots  = p.workspace + (size_t)blockIdx.y * p.slots_per_chunk * (size_t)(128 * kSuperN);
        int* const   arrive = p.counters + (size_t)blockIdx.y * p.n_col_tiles;
        int* const   done   = p.counters + (size_t)(gridDim.y + blockIdx.y) * p.n_col_tiles;
        constexpr int kMaxPending = 4;
        int           pend[kMaxPending] = {0, 0, 0, 0};
        int           n_pend = 0;
        // Every CTA of a split tile reduces its own share of the feature rows, once all partials of the
        // tile are in scratch: nobody reads more than one tile's worth, and the sum runs in CTA order.
        auto reduce_share = [&](int tjs) {
            const int c_first = (tjs * G) / upc;
            const int c_last  = ((tjs + 1) * G - 1) / upc;
            const int n_split = c_last - c_first + 1;
            const int col0    = tjs * kSuperN;
            if (dtid == 0) {
                // Bounded wait for the other CTAs of the tile.  The plan splits tiles between CTAs only
                // when the whole grid is one wave of at most one CTA per SM (gemm_tc_plan), so the
                // partners are running or waiting for an SM that a kernel ahead in the stream still
                // holds; that kernel does not depend on this one.
                int             seen = 0;
                const long long t_begin = clock64();
                for (;;) {
                    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(arrive + tjs) : "memory");
                    if (seen >= n_split || clock64() - t_begin > p.max_wait_cycles) break;
                }
                if (seen < n_split) atomicOr(p.status, kStatusGemmTmemWait);
                bars->flag = seen >= n_split;
            }
            named_bar_sync(1, kDqThreads);
            TC_TRACE(trow, 42, tjs);
            if (bars->flag) {
                const int j      = blockIdx.x - c_first;
                const int n_cols = min(kSuperN, p.N - col0);  // N % 32 == 0
                const int f0     = (n_cols * j / n_split) & ~3;
                const int f1     = j == n_split - 1 ? n_cols : ((n_cols * (j + 1) / n_split) & ~3);
                const int quads  = (f1 - f0) / 4;
                const int items  = t_rows * quads;
                for (int i = dtid; i < items; i += kDqThreads) {
                    const int    t    = i / quads;
                    const int    n    = f0 + (i - t * quads) * 4;
                    const float* src  = slots + (size_t)t * kSuperN + n;
                    float4       acc  = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int cc = c_first; cc <= c_last; cc += 4) {
                        float4 part[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            part[e] = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (cc + e <= c_last) {
                                part[e] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(cc + e + tjs) * (size_t)(128 * kSuperN)));
                            }
                        }
#pragma unroll
                        for (int e = 0; e < 4; ++e) {  // absent slots add +0
                            acc.x += part[e].x, acc.y += part[e].y, acc.z += part[e].z, acc.w += part[e].w;
                        }
                    }
                    const __half2 h0 = __floats2half2_rn(acc.x, acc.y), h1 = __floats2half2_rn(acc.z, acc.w);
                    if (p.fused_silu) {
                        // kernels/gemm_s_f16/gemm_s4_f16.cu:31-43 on the fp16-rounded pairs (gate, up)
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
            named_bar_sync(1, kDqThreads);  // everyone is done reading; the flag may be reused
            if (dtid == 0) {
                // the last reader of the tile resets both counts for the next launch; a CTA that gave up
                // on the wait counts as a reader too, so the counts recover after a time-out
                if (atomicAdd(done + tjs, 1) == n_split - 1) {
                    arrive[tjs] = 0;
                    done[tjs]   = 0;
                }
            }
        };

        const int      ccount = TT / 2;  // token columns per warp: [kh * ccount, +ccount)
        const int      n_row  = m * kTileN + q * 32 + lane;  // feature row of the CTA tile held by this thread
        // fp32 sums of this thread's feature row over the units of the current segment (FOLD)
        float y[FOLD ? 32 : 1];
#pragma unroll
        for (int i = 0; i < (FOLD ? 32 : 1); ++i) y[i] = 0.f;
        float s_prev = 0.f;   // scale of this thread's feature row for the unit expanded last (FOLD)
        int   prev_js = 0;
        bool  prev_end = false;

        // output of a finished segment: `get(col, v)` delivers eight token columns of this thread's row
        auto finish_segment = [&](int this_js, auto&& get) {
            const int c_first = (this_js * G) / upc;
            const int c_last  = ((this_js + 1) * G - 1) / upc;
            const int n_split = c_last - c_first + 1;
            const int col0    = this_js * kSuperN;
            const int n_glob  = col0 + n_row;
            // eight token columns of this thread's feature row -> C
            auto store_c = [&](const float (&v)[8], int col) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int t = t0 + col + i;
                    if (p.fused_silu) {
                        // kernels/gemm_s_f16/gemm_s4_f16.cu:31-43 on the fp16-rounded pair (gate, up) = rows (n, n + 1)
                        const float mine  = __half2float(__float2half_rn(v[i]));
                        const float other = __shfl_down_sync(0xffffffffu, mine, 1);
                        if ((lane & 1) == 0 && t < p.T && n_glob < p.N) {
                            const float silu = mine / (1.f + __expf(-mine));
                            p.C[(size_t)t * (p.N / 2) + n_glob / 2] = __float2half_rn(silu * other);
                        }
                    }
                    else if (t < p.T && n_glob < p.N) {
                        p.C[(size_t)t * p.N + n_glob] = __float2half_rn(v[i]);
                    }
                }
            };
            if (!dead) {
                float* mine = slots + (size_t)(blockIdx.x + this_js) * (size_t)(128 * kSuperN) + n_row;
                for (int cb = 0; cb < ccount; cb += 8) {
                    const int col = kh * ccount + cb;
                    float     v[8];
                    get(cb, col, v);
                    if (n_split > 1) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) __stcg(mine + (size_t)(col + i) * kSuperN, v[i]);
                    }
                    else {
                        store_c(v, col);
                    }
                }
            }
            return n_split;
        };
        // after the segment's values have left the accumulators / registers
        auto publish_segment = [&](int this_js, int n_split) {
            if (n_split > 1) {
                // publish the partial; its reduction waits until this CTA has no units left
                __threadfence();
                named_bar_sync(1, kDqThreads);
                if (dtid == 0) {
                    __threadfence();  // release: the partial of every thread, ordered before by the barrier
                    atomicAdd(arrive + this_js, 1);
                }
                if (n_pend == kMaxPending) {
                    reduce_share(pend[0]);
                    for (int i = 1; i < kMaxPending; ++i) pend[i - 1] = pend[i];
                    --n_pend;
                }
                pend[n_pend++] = this_js;
            }
        };

        int      js = u_begin / G, g = u_begin - js * G;
        int      sw = 0, sw_fill = kWST - 1;  // ring slot read now / refilled now (the one read one unit ago)
        int      sa = 0;
        uint32_t pa = 0;                      // phase parity of the team's expanded-weight ring
        const int n_iter = FOLD ? n_units + 1 : n_units;  // FOLD: the accumulator of a unit is folded one iteration later
        for (int it = 0; it < n_iter; ++it) {
            float s_cur    = 0.f;
            int   this_js  = js;
            bool  seg_end  = false;
            if (it < n_units) {
                TC_TRACE(trow, 30, it);
                asm volatile("cp.async.wait_group %0;" ::"n"(kWST - 2) : "memory");
                __syncwarp();
                TC_TRACE(trow, 31, it);
                // the tensor core must be done with what this TMEM stage held kAST units ago (the first
                // round passes at once: a fresh barrier counts as having completed the phase before)
                warp_wait(&bars->a_empty[m][sa], pa ^ 1u, dead, p.status, kStatusGemmPipeWait);
                tc_fence_after();
                TC_TRACE(trow, 32, it);
                {
                    const unsigned char* sb = my_ring_g + sw * kWarpStage;
                    const __half2*       qs = reinterpret_cast<const __half2*>(sb + 2 * kTileBytes);
                    uint32_t z1024[2], nz64[2], s_lo[2], s_hi[2];
#pragma unroll
                    for (int a = 0; a < 2; ++a) {
                        const __half2 q_lo = qs[a * 16 + r];
                        const __half2 q_hi = qs[a * 16 + r + 8];
                        const __half2 zl2  = __half2half2(__hadd(__low2half(q_lo), __float2half_rn(960.f)));
                        const __half2 zh2  = __half2half2(__hneg(__low2half(q_hi)));
                        z1024[a] = reinterpret_cast<const uint32_t&>(zl2);
                        nz64[a]  = reinterpret_cast<const uint32_t&>(zh2);
                        if (!FOLD) {
                            const __half2 sl2 = __half2half2(__high2half(q_lo));
                            const __half2 sh2 = __half2half2(__high2half(q_hi));
                            s_lo[a] = reinterpret_cast<const uint32_t&>(sl2);
                            s_hi[a] = reinterpret_cast<const uint32_t&>(sh2);
                        }
                    }
                    if (FOLD) s_cur = __half2float(__high2half(qs[lane]));  // feature row q * 32 + lane of the team's tile
                    const uint32_t a_tmem = a_base + (m * kAST + sa) * kACols + ((uint32_t)(q * 32) << 16);
                    // one 32-row slab at a time: its four fragments first (independent chains the scheduler can
                    // interleave), then their stores
#pragma unroll
                    for (int kk = 0; kk < 2; ++kk) {
                        const int      k32   = kh * 2 + kk;  // 32-row slab of the group: k = 32 k32 .. +31
                        const uint4    w     = reinterpret_cast<const uint4*>(sb)[kk * 32 + lane];
                        const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
                        uint32_t       f[4][4];
#pragma unroll
                        for (int wi = 0; wi < 4; ++wi) {
                            const int a = wi & 1;
                            unpack_s4_minus_zero(wv[wi], z1024[a], nz64[a], f[wi]);
                            if (!FOLD) {
                                f[wi][0] = hmul2_ftz(f[wi][0], s_lo[a]);
                                f[wi][1] = hmul2_ftz(f[wi][1], s_hi[a]);
                                f[wi][2] = hmul2_ftz(f[wi][2], s_lo[a]);
                                f[wi][3] = hmul2_ftz(f[wi][3], s_hi[a]);
                            }
                        }
#pragma unroll
                        for (int wi = 0; wi < 4; ++wi) {
                            const int k16 = wi >> 1;
                            const int a   = wi & 1;
                            // rows q*32 + a*16 .. +15 (TMEM lanes), k = 32 k32 + 16 k16 .. +15 (8 columns)
                            tmem_st_16x128b_x2(a_tmem + ((uint32_t)(a * 16) << 16) + (uint32_t)(k32 * 16 + k16 * 8), f[wi][0], f[wi][1],
                                               f[wi][2], f[wi][3]);
                        }
                    }
                }
                // expanded tile visible to the tensor core; packed stage free again
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->a_full[m][sa]);
                TC_TRACE(trow, 33, it);
                // refill the slot that was read one unit ago (everyone in the warp is past its reads)
                if (to_issue > 0) issue_unit(sw_fill);
                --to_issue;
                asm volatile("cp.async.commit_group;" ::: "memory");
                sw      = (sw == kWST - 1) ? 0 : sw + 1;
                sw_fill = (sw_fill == kWST - 1) ? 0 : sw_fill + 1;
                if (++sa == kAST) {
                    sa = 0;
                    pa ^= 1u;
                }
                seg_end = (it == n_units - 1) || (g == G - 1);
                if (++g == G) {
                    g = 0;
                    ++js;
                }
            }

            if (FOLD) {
                if (it >= 1) {
                    // ---- fold the accumulator of unit it - 1 into the fp32 sums ---------------------
                    const int u   = it - 1;
                    const int buf = u & 1;
                    TC_TRACE(trow, 34, it);
                    warp_wait(&bars->acc_full[m][buf], (uint32_t)(u >> 1) & 1u, dead, p.status, kStatusGemmTmemWait);
                    tc_fence_after();
                    TC_TRACE(trow, 35, it);
                    const uint32_t my_acc = tmem + (uint32_t)((m * 2 + buf) * accS) + ((uint32_t)(q * 32) << 16) + (uint32_t)(kh * ccount);
                    // two halves of up to 16 columns each (registers): load, wait, accumulate
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        float v[16];
                        if (!dead) {
#pragma unroll
                            for (int cb = 0; cb < 16; cb += 8) {
                                if (hf * 16 + cb < ccount) tmem_ld8_nowait(my_acc + (uint32_t)(hf * 16 + cb), v + cb);
                            }
                            tmem_ld_wait();
                        }
                        if (hf == 1) {
                            // the accumulator may be overwritten now
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0 && !dead) mbar_arrive(&bars->acc_empty[m][buf]);
                        }
                        if (!dead) {
#pragma unroll
                            for (int cb = 0; cb < 16; cb += 8) {
                                if (hf * 16 + cb < ccount) {
#pragma unroll
                                    for (int i = 0; i < 8; ++i) y[hf * 16 + cb + i] = fmaf(s_prev, v[cb + i], y[hf * 16 + cb + i]);
                                }
                            }
                        }
                    }
                    TC_TRACE(trow, 36, it);
                    if (prev_end) {
                        // ---- 256-feature tile prev_js finished for this CTA --------------------------
                        const int n_split = finish_segment(prev_js, [&](int cb, int, float (&o)[8]) {
#pragma unroll
                            for (int cc = 0; cc < 32; cc += 8) {
                                if (cc == cb) {
#pragma unroll
                                    for (int i = 0; i < 8; ++i) o[i] = y[cc + i];
                                }
                            }
                        });
#pragma unroll
                        for (int i = 0; i < 32; ++i) y[i] = 0.f;
                        TC_TRACE(trow, 37, it);
                        publish_segment(prev_js, n_split);
                        TC_TRACE(trow, 38, it);
                    }
                }
                s_prev   = s_cur;
                prev_js  = this_js;
                prev_end = seg_end;
                continue;
            }

            if (!seg_end) continue;

            // ---- !FOLD: 256-feature tile this_js finished for this CTA: drain the accumulator --------
            warp_wait(&bars->acc_full[m][0], seg_idx & 1, dead, p.status, kStatusGemmTmemWait);
            tc_fence_after();
            const uint32_t my_acc  = tmem + m * accS + ((uint32_t)(q * 32) << 16);
            const int      n_split = finish_segment(this_js, [&](int, int col, float (&o)[8]) { tmem_ld8(my_acc + (uint32_t)col, o); });
            ++seg_idx;
            // the accumulator may be overwritten now
            tc_fence_before();
            __syncwarp();
            if (lane == 0 && !dead) mbar_arrive(&bars->acc_empty[m][0]);
            publish_segment(this_js, n_split);
        }
        TC_TRACE(trow, 40, 0);
        for (int i = 0; i < n_pend; ++i) {
            reduce_share(pend[i]);
            TC_TRACE(trow, 41, i);
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(kTmemCols) : "memory");
    }
}

using PFN_encodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                     const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// the driver's tensor-map encoder, found through the runtime so that the library does not link libcuda
PFN_encodeTiled lookup_encode_tiled()
{
    void*                           fn = nullptr;
    cudaDriverEntryPointQueryResult q{};
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess
        || q != cudaDriverEntryPointSuccess) {
        return nullptr;
    }
    return reinterpret_cast<PFN_encodeTiled>(fn);
}

int x_stages_for(int token_tile) { return token_tile > 64 ? 3 : kXSTMax; }
int acc_stride_for(int token_tile) { return token_tile > 64 ? 128 : 64; }

}  // namespace

size_t gemm_tc_smem_bytes(int token_tile)
{
    return 1024 + (size_t)x_stages_for(token_tile) * 2 * token_tile * 128 + (size_t)kWST * kDqWarps * kWarpStage + sizeof(Bars) + 64;
}

GemmTcPlan gemm_tc_plan(int N, int T, int K, int sm_count)
{
    GemmTcPlan pl{};
    pl.token_tile  = T >= 128 ? 128 : ((T + 15) / 16) * 16;
    pl.t_chunks    = (T + 127) / 128;
    pl.n_col_tiles = (N + kSuperN - 1) / kSuperN;
    const int G    = K / kGroup;
    pl.total_units = pl.n_col_tiles * G;
    if ((long long)pl.t_chunks * pl.n_col_tiles >= sm_count) {
        // enough whole column tiles to fill the device: one per CTA, nothing is split, nobody waits
        pl.units_per_cta = G;
    }
    else {
        // K is split between CTAs only while the whole grid is a single wave of one CTA per SM: CTAs
        // that share a column tile wait for one another, so all of them must be able to run together
        int ctas = sm_count / pl.t_chunks;
        if (ctas > pl.total_units) ctas = pl.total_units;
        pl.units_per_cta = (pl.total_units + ctas - 1) / ctas;
    }
    pl.ctas            = (pl.total_units + pl.units_per_cta - 1) / pl.units_per_cta;
    pl.slots_per_chunk = pl.ctas + pl.n_col_tiles;
    pl.smem_bytes      = gemm_tc_smem_bytes(pl.token_tile);
    pl.workspace_floats = pl.units_per_cta % G == 0 ? 0 : (size_t)pl.t_chunks * pl.slots_per_chunk * 128 * kSuperN;
    pl.counter_ints     = (size_t)2 * pl.t_chunks * pl.n_col_tiles;  // arrivals and finished readers per tile
    return pl;
}

cudaError_t gemm_tc_prepare(int max_smem)
{
    cudaError_t e = cudaFuncSetAttribute(gemm_s4_f16_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(gemm_s4_f16_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
}

cudaError_t gemm_tc_launch(const GemmTcPlan& pl, GemmTcParams p, cudaStream_t st, bool pdl)
{
    p.units_per_cta   = pl.units_per_cta;
    p.total_units     = pl.total_units;
    p.slots_per_chunk = pl.slots_per_chunk;
    p.n_col_tiles     = pl.n_col_tiles;
    p.token_tile      = pl.token_tile;
    p.x_stages        = x_stages_for(pl.token_tile);
    if (p.max_wait_cycles <= 0) p.max_wait_cycles = kMaxWaitCycles;
    p.acc_stride      = acc_stride_for(pl.token_tile);

    // Activations as a 2-D tensor [T][K] of fp16; one box = 64 k (128 bytes, the swizzle span) x token tile.
    static const PFN_encodeTiled encode = lookup_encode_tiled();
    if (encode == nullptr) return cudaErrorNotSupported;
    CUtensorMap       x_map;
    const cuuint64_t  dims[2]    = {(cuuint64_t)p.K, (cuuint64_t)p.T};
    const cuuint64_t  strides[1] = {(cuuint64_t)p.K * 2};
    const cuuint32_t  box[2]     = {64u, (cuuint32_t)pl.token_tile};
    const cuuint32_t  estr[2]    = {1u, 1u};
    if (encode(&x_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<unsigned char*>(p.X), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
        != CUDA_SUCCESS) {
        return cudaErrorInvalidValue;
    }
    dim3 grid(pl.ctas, pl.t_chunks);
    if (pl.token_tile <= 64) {
        return launch_kernel(gemm_s4_f16_tc_kernel<true>, grid, dim3(kThreads), pl.smem_bytes, st, pdl, p, x_map);
    }
    return launch_kernel(gemm_s4_f16_tc_kernel<false>, grid, dim3(kThreads), pl.smem_bytes, st, pdl, p, x_map);
}

}  // namespace tmb
