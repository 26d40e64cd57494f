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
//                the packed weight through a private cp.async ring and expands it: lop3 nibble
//                unpack, exact (q - z) in fp16, one fp16 multiply by the scale (bit-identical to the
//                reference's dequantised weight, kernels/gemm_s_f16/common.h:115-156, 218-235),
//                tcgen05.st of the fragments straight into TMEM, from where the tensor core takes
//                its A operand (no shared-memory round trip); at the end of a column tile the
//                warps read the accumulators with tcgen05.ld and store C (optionally through the
//                SiLU(gate) * up epilogue) or the split-K partial
// A waiting thread sleeps in the mbarrier (try_wait with a time hint): the three single-lane roles
// would otherwise take a quarter of the issue slots from the expanding warps.
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
__device__ unsigned long long g_tc_span[512][2];  // per launch: first CTA start, last CTA end (globaltimer ns)
__device__ int                g_tc_launch;
__device__ unsigned long long g_tc_cta[160][4];   // launch 5: per CTA start, end (ns), smid, units
extern "C" __attribute__((visibility("default"))) int tm_dev_gemm_ctas(unsigned long long* out)
{
    cudaMemcpyFromSymbol(out, g_tc_cta, sizeof(unsigned long long) * 640);
    return 0;
}
extern "C" __attribute__((visibility("default"))) int tm_dev_gemm_spans(unsigned long long* out, int reset)
{
    cudaMemcpyFromSymbol(out, g_tc_span, sizeof(unsigned long long) * 1024);
    if (reset) {
        static unsigned long long init[1024];
        for (int i = 0; i < 512; ++i) { init[2 * i] = ~0ull; init[2 * i + 1] = 0ull; }
        cudaMemcpyToSymbol(g_tc_span, init, sizeof(init));
        int z = 0;
        cudaMemcpyToSymbol(g_tc_launch, &z, sizeof(z));
    }
    return 0;
}
__device__ __forceinline__ unsigned long long tc_globaltimer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
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
constexpr int kIssuers   = 2 * kTeams;           // issuer warps: (team, K half); the second halves idle at token tiles > 64
constexpr int kDqWarp0   = 1 + kIssuers;         // first expanding warp
constexpr int kThreads   = (kDqWarp0 + kDqWarps) * 32;
constexpr int kTmemCols  = 512;                  // accumulators + expanded-weight stages, power of two

struct Bars {
    uint64_t a_full[kTeams][kASTMax], a_empty[kTeams][kASTMax];
    uint64_t x_full[kXSTMax], x_empty[kXSTMax];
    uint64_t acc_full[kTeams], acc_empty[kTeams];  // per team
    uint32_t tmem_base;
    int      flag;
};

__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr)
{
    // K-major, 128-byte swizzle: 8-row groups 1024 B apart (SBO), leading offset 1, descriptor version 1
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46)
           | ((uint64_t)2 << 61);
}

// Four MMAs: one 64-wide K block (four 16-wide steps) of a unit, operands precomputed so that an MMA costs the
// issuing thread three instructions.  `first`: the first MMA overwrites the accumulator.
__device__ __forceinline__ void umma_f16_ts_x4(uint32_t tmem_d, uint32_t tmem_a, uint32_t desc_lo, uint32_t desc_hi, uint32_t idesc,
                                               uint32_t first)
{
    asm volatile(
        "{\n"
        ".reg .pred p, t;\n"
        ".reg .b64 d;\n"
        ".reg .b32 a, l;\n"
        "setp.eq.b32 p, %5, 0;\n"      // accumulate unless first
        "setp.eq.b32 t, 0, 0;\n"       // always accumulate
        "mov.b64 d, {%2, %3};\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], d, %4, p;\n"
        "add.u32 a, %1, 8;\n  add.u32 l, %2, 2;\n  mov.b64 d, {l, %3};\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %4, t;\n"
        "add.u32 a, %1, 16;\n add.u32 l, %2, 4;\n  mov.b64 d, {l, %3};\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %4, t;\n"
        "add.u32 a, %1, 24;\n add.u32 l, %2, 6;\n  mov.b64 d, {l, %3};\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], d, %4, t;\n"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a),
        "r"(desc_lo),
        "r"(desc_hi),
        "r"(idesc),
        "r"(first)
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

// sixteen fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16])
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
    // Usually the phase is complete already: every lane tests it (same answer in every lane, no divergence).
    if (mbar_try_wait(bar, parity)) return;
    // Otherwise one lane sleeps in the barrier; the shuffle hands the outcome (and, as a warp-level sync, the
    // ordering) to the rest.
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok) {
        if ((threadIdx.x & 31) == 0) atomicOr(status, bit);
        dead = true;
    }
}

__global__ void __launch_bounds__(kThreads, 1) gemm_s4_f16_tc_kernel(GemmTcParams p, const __grid_constant__ CUtensorMap x_map)
{
    const int kXST = p.x_stages;
    const int kAST = p.a_stages;    // per team
    const int accS = p.acc_stride;  // TMEM columns of one accumulator
    const int KS   = p.k_split;     // issuers (and accumulators) per team: 2 at token tiles <= 64, else 1
    extern __shared__ unsigned char smem_dyn[];
    // tiles the tensor core reads must sit on 1024-byte boundaries (the swizzle is a function of
    // the address bits)
    const uint32_t raw  = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* sm   = smem_dyn + (base - raw);

    const int TT      = p.token_tile;             // UMMA N, multiple of 16, <= 128
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
    const int launch_idx = *(volatile int*)&g_tc_launch;
    const long long clk_begin = clock64();
    const unsigned long long gt_begin = tc_globaltimer();
    if (tid == 0 && launch_idx < 512) atomicMin(&g_tc_span[launch_idx][0], gt_begin);
#endif

    const int t0     = blockIdx.y * 128;
    const int t_rows = min(TT, p.T - t0);

    const int G         = p.K / kGroup;
    const int upc       = p.units_per_cta;
    // Two ways of dealing the (column tile, group) units to the CTAs: `parts` CTAs per column tile, each with up
    // to `upc` consecutive groups of it (no CTA touches two tiles); or, with parts == 0, the flat unit list cut
    // into runs of `upc` (a run may end one tile and begin the next).
    const int parts     = p.parts_per_tile;
    const int u_begin   = parts ? (blockIdx.x / parts) * G + (blockIdx.x % parts) * upc : blockIdx.x * upc;
    const int n_units   = parts ? min(upc, G - (int)(blockIdx.x % parts) * upc) : min(u_begin + upc, p.total_units) - u_begin;
    // the CTAs that share column tile `tile`: first CTA and how many
    auto tile_ctas = [&](int tile, int& c_first) {
        if (parts) {
            c_first = tile * parts;
            return parts;
        }
        c_first = (tile * G) / upc;
        return ((tile + 1) * G - 1) / upc - c_first + 1;
    };
    const int n_tiles32 = p.N / 32;

    // ---- expanding warps: identity and the state of their copy front ---------------------------
    const int  dw   = warp - kDqWarp0; // 0..15 for the expanding warps
    const int  m_dq = (dw >> 3) & 1;   // team = 128-feature tile of the unit
    const int  q    = warp & 3;        // TMEM lane quarter this warp may access = its 32-feature tile
    const int  kh   = (dw >> 2) & 1;   // which pair of 32-row slabs of the group it expands,
                                       // and which half of the token columns it drains
    // private ring of this warp: per unit its own 2 x 512 B of packed weight (32-feature tile,
    // 32-row slabs 2 kh, 2 kh + 1 of the group) + the 128 B of {zero, scale} of its 32 features
    const uint32_t       my_ring   = base + (uint32_t)(w_ring - sm) + (uint32_t)(dw < 0 ? 0 : dw) * kWST * kWarpStage + lane * 16;
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
        const uint32_t dst = my_ring + stage * kWarpStage;
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
                mbar_init(&bars->a_empty[m][s], KS);
            }
            mbar_init(&bars->acc_full[m], KS);
            mbar_init(&bars->acc_empty[m], kTeamWarps);
        }
        for (int s = 0; s < kXSTMax; ++s) {
            mbar_init(&bars->x_full[s], 1);
            mbar_init(&bars->x_empty[s], kTeams * KS);
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
    const uint32_t a_base = tmem + kTeams * KS * accS;  // first expanded-weight stage

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
    else if (warp <= kIssuers) {
        // ================================================================== MMA issuers
        // One lane per (team, K half) runs the whole loop: waits, four (or eight) MMAs, commits.  The issue rate
        // of one thread among busy warps (about 100 cycles per MMA), not the tensor pipe (about 35 at 64 tokens),
        // bounds the MMA throughput of small token tiles: four issuers on four different schedulers share the
        // work there, each half of K with an accumulator of its own (summed by the epilogue).
        const int m = (warp - 1) & 1;
        const int h = (warp - 1) >> 1;
        if (lane == 0 && h < KS) {
            const uint32_t idesc   = (1u << 4) | ((uint32_t)(TT >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);
            const uint32_t d_tmem  = tmem + (m * KS + h) * accS;
            const uint32_t kb_step = (uint32_t)(TT * 128) >> 4;  // descriptor units (16 B) between the two K blocks
            const uint64_t d_ring  = make_desc(base + (uint32_t)(x_ring - sm));
            const uint32_t d_hi    = (uint32_t)(d_ring >> 32);
            // (the low word of the descriptor carries the address: 14 bits of 16-byte units, never a carry out)
            const uint32_t d_lo    = (uint32_t)d_ring + (uint32_t)h * kb_step;
            const uint32_t x_step  = (uint32_t)x_bytes >> 4;
            int  seg_idx = 0;
            bool first   = true;  // first MMA of the current segment overwrites the accumulator
            int  g       = u_begin % G;
            int  sa = 0, sx = 0;
            uint32_t pa = 0, px = 0;  // phase parity of the weight / activation rings
            for (int it = 0; it < n_units; ++it) {
                bool ok = true;
                if (first && seg_idx > 0) {
                    // the epilogue of the previous segment must have drained the accumulators
                    ok = mbar_wait(&bars->acc_empty[m], (seg_idx - 1) & 1);
                }
                ok = ok && mbar_wait(&bars->x_full[sx], px) && mbar_wait(&bars->a_full[m][sa], pa);
                if (!ok) {
                    atomicOr(p.status, kStatusGemmPipeWait);
                    break;
                }
                tc_fence_after();
                TC_TRACE(trow, 20, it);
                const uint32_t a_tmem = a_base + (m * kAST + sa) * kACols + (uint32_t)h * 32;
                const uint32_t lo     = d_lo + (uint32_t)sx * x_step;
                umma_f16_ts_x4(d_tmem, a_tmem, lo, d_hi, idesc, first ? 1u : 0u);
                if (KS == 1) umma_f16_ts_x4(d_tmem, a_tmem + 32, lo + kb_step, d_hi, idesc, 0u);
                umma_commit(&bars->a_empty[m][sa]);
                umma_commit(&bars->x_empty[sx]);
                TC_TRACE(trow, 21, it);
                first = false;
                if ((it == n_units - 1) || (g == G - 1)) {
                    umma_commit(&bars->acc_full[m]);
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

        // split-K: [slot][TT tokens][256 feature rows] fp32 partial tiles (a warp touches 128 contiguous
        // bytes per token: whole sectors), per tile a count of CTAs whose partial is complete and a count of
        // CTAs that are done reading.  Tiles this CTA shares with others are reduced after its last unit.
        const size_t slot_floats = (size_t)kSuperN * TT;
        float* const slots  = p.workspace + (size_t)blockIdx.y * p.slots_per_chunk * slot_floats;
        int* const   arrive = p.counters + (size_t)blockIdx.y * p.n_col_tiles;
        int* const   done   = p.counters + (size_t)(gridDim.y + blockIdx.y) * p.n_col_tiles;
        constexpr int kMaxPending = 4;
        int           pend[kMaxPending] = {0, 0, 0, 0};
        int           n_pend = 0;
        // Every CTA of a split tile reduces its own share of the feature rows, once all partials of the
        // tile are in scratch: nobody reads more than one tile's worth, and the sum runs in CTA order.
        auto reduce_share = [&](int tjs) {
            int       c_first;
            const int n_split = tile_ctas(tjs, c_first);
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
                    __nanosleep(64);
                }
                if (seen < n_split) atomicOr(p.status, kStatusGemmTmemWait);
                bars->flag = seen >= n_split;
            }
            // producer side of a folded norm: per-token sums of squares of this CTA's share, in fixed point, kept in the
            // (by now idle) activation ring until they go out with one atomic per token
            unsigned long long* s_ssq = reinterpret_cast<unsigned long long*>(x_ring);
            if (p.norm.ssq_out && dtid < t_rows) s_ssq[dtid] = 0ull;
            named_bar_sync(1, kDqThreads);
            TC_TRACE(trow, 42, tjs);
            const bool tile_ok = bars->flag != 0;  // read between the barriers: the next call may rewrite the flag
            if (tile_ok) {
                const int j      = blockIdx.x - c_first;
                const int n_cols = min(kSuperN, p.N - col0);  // N % 32 == 0
                const int f0     = (n_cols * j / n_split) & ~3;
                const int f1     = j == n_split - 1 ? n_cols : ((n_cols * (j + 1) / n_split) & ~3);
                const int quads  = (f1 - f0) / 4;
                const int items  = t_rows * quads;
                const float* tile_slots = slots + (size_t)(c_first + tjs) * slot_floats;
                for (int i = dtid; i < items; i += kDqThreads) {
                    const int    t    = i / quads;
                    const int    n    = f0 + (i - t * quads) * 4;
                    const float* src  = tile_slots + (size_t)t * kSuperN + n;
                    float4       acc  = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int cc = 0; cc < n_split; cc += 8) {
                        float4 part[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            part[e] = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (cc + e < n_split) part[e] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(cc + e) * slot_floats));
                        }
#pragma unroll
                        for (int e = 0; e < 8; ++e) {  // absent slots add +0
                            acc.x += part[e].x, acc.y += part[e].y, acc.z += part[e].z, acc.w += part[e].w;
                        }
                    }
                    if (p.norm.ssq_in) {
                        // consumer side: the row's 1 / rms completes the normalisation of this GEMM's input
                        const float ssq = (float)__ldcg(p.norm.ssq_in + t0 + t) * (1.f / 1048576.f);
                        const float inv = rsqrtf(ssq * p.norm.inv_n + p.norm.eps);
                        acc.x *= inv, acc.y *= inv, acc.z *= inv, acc.w *= inv;
                    }
                    const __half2 h0 = __floats2half2_rn(acc.x, acc.y), h1 = __floats2half2_rn(acc.z, acc.w);
                    if (p.norm.ssq_out) {
                        // producer side (llama_decoder_kernels.cu:104-160 split in two): residual += y in fp32, stored as
                        // fp16; the sum of squares is taken before that rounding, the norm weight applied to the stored value
                        __half2*       rp = reinterpret_cast<__half2*>(p.norm.residual + (size_t)(t0 + t) * p.N + col0 + n);
                        const __half2* gp = reinterpret_cast<const __half2*>(p.norm.norm_weight + col0 + n);
                        const float2   r0 = __half22float2(rp[0]), r1 = __half22float2(rp[1]);
                        const float2   y0 = __half22float2(h0), y1 = __half22float2(h1);
                        const float2   s0 = make_float2(r0.x + y0.x, r0.y + y0.y), s1 = make_float2(r1.x + y1.x, r1.y + y1.y);
                        const float    ss = (s0.x * s0.x + s0.y * s0.y) + (s1.x * s1.x + s1.y * s1.y);
                        const __half2  n0 = __float22half2_rn(s0), n1 = __float22half2_rn(s1);
                        rp[0] = n0, rp[1] = n1;
                        const float2 a0 = __half22float2(n0), a1 = __half22float2(n1);
                        const float2 g0 = __half22float2(gp[0]), g1 = __half22float2(gp[1]);
                        __half2*     dst = reinterpret_cast<__half2*>(p.C + (size_t)(t0 + t) * p.N + col0 + n);
                        dst[0]           = __floats2half2_rn(a0.x * g0.x, a0.y * g0.y);
                        dst[1]           = __floats2half2_rn(a1.x * g1.x, a1.y * g1.y);
                        atomicAdd(s_ssq + t, (unsigned long long)__float2ll_rn(ss * 1048576.f));
                    }
                    else if (p.fused_silu) {
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
            if (p.norm.ssq_out && tile_ok && dtid < t_rows && s_ssq[dtid]) atomicAdd(p.norm.ssq_out + t0 + dtid, s_ssq[dtid]);
            if (dtid == 0) {
                // the last reader of the tile resets both counts for the next launch; a CTA that gave up
                // on the wait counts as a reader too, so the counts recover after a time-out
                if (atomicAdd(done + tjs, 1) == n_split - 1) {
                    arrive[tjs] = 0;
                    done[tjs]   = 0;
                }
            }
        };

        const int      ccount = TT / 2;                      // token columns per warp: [kh * ccount, +ccount)
        const int      n_row  = m * kTileN + q * 32 + lane;  // feature row of the CTA tile held by this thread
        const uint32_t a_lane = ((uint32_t)(q * 32) << 16) + (uint32_t)(kh * 32);  // TMEM lanes and first column of this warp's share of a stage

        int      js = u_begin / G, g = u_begin - js * G;
        int      sw = 0, sw_fill = kWST - 1;  // ring slot read now / refilled now (the one read one unit ago)
        int      sa = 0;
        uint32_t pa = 0;                      // phase parity of the team's expanded-weight ring
        for (int it = 0; it < n_units; ++it) {
            TC_TRACE(trow, 30, it);
            asm volatile("cp.async.wait_group %0;" ::"n"(kWST - 2) : "memory");
            __syncwarp();
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
                    const __half2 sl2  = __half2half2(__high2half(q_lo));
                    const __half2 sh2  = __half2half2(__high2half(q_hi));
                    z1024[a] = reinterpret_cast<const uint32_t&>(zl2);
                    nz64[a]  = reinterpret_cast<const uint32_t&>(zh2);
                    s_lo[a]  = reinterpret_cast<const uint32_t&>(sl2);
                    s_hi[a]  = reinterpret_cast<const uint32_t&>(sh2);
                }
                const uint32_t a_tmem = a_base + (m * kAST + sa) * kACols + a_lane;
                // all fragments first (independent chains the scheduler can interleave), then the stores
                uint32_t f[8][4];
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    const uint4    w     = reinterpret_cast<const uint4*>(sb)[kk * 32 + lane];
                    const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int wi = 0; wi < 4; ++wi) {
                        const int a = wi & 1;
                        uint32_t (&fr)[4] = f[kk * 4 + wi];
                        unpack_s4_minus_zero(wv[wi], z1024[a], nz64[a], fr);
                        fr[0] = hmul2_ftz(fr[0], s_lo[a]);
                        fr[1] = hmul2_ftz(fr[1], s_hi[a]);
                        fr[2] = hmul2_ftz(fr[2], s_lo[a]);
                        fr[3] = hmul2_ftz(fr[3], s_hi[a]);
                    }
                }
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
                    for (int wi = 0; wi < 4; ++wi) {
                        const int k16 = wi >> 1;
                        const int a   = wi & 1;
                        const uint32_t (&fr)[4] = f[kk * 4 + wi];
                        // rows q*32 + a*16 .. +15 (TMEM lanes), k = 32 (2 kh + kk) + 16 k16 .. +15 (8 columns)
                        tmem_st_16x128b_x2(a_tmem + ((uint32_t)(a * 16) << 16) + (uint32_t)(kk * 16 + k16 * 8), fr[0], fr[1], fr[2], fr[3]);
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

            const int  this_js = js;
            const bool seg_end = (it == n_units - 1) || (g == G - 1);
            if (++g == G) {
                g = 0;
                ++js;
            }
            if (!seg_end) continue;

            // ---- 256-feature tile this_js finished for this CTA: drain the accumulators -----------
            int       c_first;
            const int n_split = tile_ctas(this_js, c_first);
            const int col0    = this_js * kSuperN;
            TC_TRACE(trow, 34, it);
            warp_wait(&bars->acc_full[m], seg_idx & 1, dead, p.status, kStatusGemmTmemWait);
            tc_fence_after();
            TC_TRACE(trow, 35, it);
            const int n_glob = col0 + n_row;
            const uint32_t my_acc = tmem + m * KS * accS + ((uint32_t)(q * 32) << 16);
            if (!dead) {
                float* mine = slots + (size_t)(blockIdx.x + this_js) * slot_floats + n_row;
                for (int cb = 0; cb < ccount; cb += 16) {
                    // sixteen token columns of this thread's feature row (eight, twice, where ccount is not a
                    // multiple of 16: the second half then repeats columns the other warp owns and is dropped)
                    const int col = kh * ccount + cb;
                    float     v[16];
                    tmem_ld16(my_acc + (uint32_t)col, v);
                    if (KS == 2) {
                        float v2[16];
                        tmem_ld16(my_acc + (uint32_t)(accS + col), v2);
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] += v2[i];
                    }
                    const int valid = min(16, ccount - cb);  // 8 or 16
                    if (n_split > 1) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            if (i < valid) __stcg(mine + (size_t)(col + i) * kSuperN, v[i]);
                        }
                    }
                    else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int t = t0 + col + i;
                            const bool in = i < valid && t < p.T && n_glob < p.N;
                            if (p.fused_silu) {
                                // kernels/gemm_s_f16/gemm_s4_f16.cu:31-43 on the fp16-rounded pair (gate, up) = rows (n, n + 1)
                                const float mine_v = __half2float(__float2half_rn(v[i]));
                                const float other  = __shfl_down_sync(0xffffffffu, mine_v, 1);
                                if ((lane & 1) == 0 && in) {
                                    const float silu = mine_v / (1.f + __expf(-mine_v));
                                    p.C[(size_t)t * (p.N / 2) + n_glob / 2] = __float2half_rn(silu * other);
                                }
                            }
                            else if (in) {
                                p.C[(size_t)t * p.N + n_glob] = __float2half_rn(v[i]);
                            }
                        }
                    }
                }
            }
            ++seg_idx;
            // the accumulators may be overwritten now
            tc_fence_before();
            __syncwarp();
            if (lane == 0 && !dead) mbar_arrive(&bars->acc_empty[m]);
            TC_TRACE(trow, 37, it);
            if (n_split > 1) {
                // publish the partial (its reduction waits until this CTA has no units left): the barrier orders
                // every thread's stores before the fence of the one thread that then counts the CTA in
                named_bar_sync(1, kDqThreads);
                if (dtid == 0) {
                    __threadfence();
                    atomicAdd(arrive + this_js, 1);
                }
                if (n_pend == kMaxPending) {
                    reduce_share(pend[0]);
                    for (int i = 1; i < kMaxPending; ++i) pend[i - 1] = pend[i];
                    --n_pend;
                }
                pend[n_pend++] = this_js;
            }
            TC_TRACE(trow, 38, it);
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
#ifdef TM_B200_GEMM_TRACE
    if (tid == 0 && launch_idx < 512) {
        atomicMax(&g_tc_span[launch_idx][1], tc_globaltimer());
        if (launch_idx == 5 && blockIdx.x < 160 && blockIdx.y == 0) {
            unsigned smid;
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            g_tc_cta[blockIdx.x][0] = gt_begin;
            g_tc_cta[blockIdx.x][1] = tc_globaltimer();
            g_tc_cta[blockIdx.x][2] = smid;
            g_tc_cta[blockIdx.x][3] = (unsigned long long)n_units;
        }
        if (blockIdx.x == 0 && blockIdx.y == 0) {
            if (launch_idx + 256 < 512) {   // CTA 0's own duration in SM cycles and in ns, stored 256 rows further down
                g_tc_span[launch_idx + 256][0] = (unsigned long long)(clock64() - clk_begin);
                g_tc_span[launch_idx + 256][1] = tc_globaltimer() - gt_begin;
            }
            // the last thing CTA 0 does; every CTA of the launch has long read the index
            __threadfence();
            atomicAdd(&g_tc_launch, 1);
        }
    }
#endif
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
int a_stages_for(int token_tile) { (void)token_tile; return 2; }
int k_split_for(int token_tile) { return token_tile > 64 ? 1 : 2; }
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
    pl.parts_per_tile = 0;
    if ((long long)pl.t_chunks * pl.n_col_tiles >= sm_count) {
        // enough whole column tiles to fill the device: one per CTA, nothing is split, nobody waits
        pl.units_per_cta = G;
        pl.ctas          = pl.n_col_tiles;
    }
    else {
        // K is split between CTAs only while the whole grid is a single wave of one CTA per SM: CTAs
        // that share a column tile wait for one another, so all of them must be able to run together
        int ctas = sm_count / pl.t_chunks;
        if (ctas > pl.total_units) ctas = pl.total_units;
        const int flat = (pl.total_units + ctas - 1) / ctas;  // units per CTA when the flat unit list is cut evenly
        // Prefer a whole number of CTAs per column tile when that costs at most one unit more per CTA: a CTA whose
        // run of units crosses from one tile into the next publishes and reduces two partial tiles instead of one.
        const int per_tile = ctas / pl.n_col_tiles;            // >= 1 here
        const int part     = (G + per_tile - 1) / per_tile;    // units per CTA with per_tile CTAs on every tile
        if (per_tile >= 2 && part <= flat + 1) {
            pl.parts_per_tile = (G + part - 1) / part;
            pl.units_per_cta  = part;
            pl.ctas           = pl.n_col_tiles * pl.parts_per_tile;
        }
        else {
            pl.units_per_cta = flat;
            pl.ctas          = (pl.total_units + flat - 1) / flat;
        }
    }
    pl.slots_per_chunk = pl.ctas + pl.n_col_tiles;
    pl.smem_bytes      = gemm_tc_smem_bytes(pl.token_tile);
    pl.workspace_floats = pl.units_per_cta % G == 0 ? 0 : (size_t)pl.t_chunks * pl.slots_per_chunk * pl.token_tile * kSuperN;
    pl.counter_ints     = (size_t)2 * pl.t_chunks * pl.n_col_tiles;  // arrivals and finished readers per tile
    return pl;
}

bool gemm_tc_all_tiles_split(const GemmTcPlan& pl, int K)
{
    if (pl.t_chunks != 1) return false;
    if (pl.parts_per_tile) return pl.parts_per_tile >= 2;
    return pl.units_per_cta < K / kGroup && pl.ctas > 1;  // a run of the flat list is shorter than a tile: every tile has several owners
}

cudaError_t gemm_tc_prepare(int max_smem)
{
    return cudaFuncSetAttribute(gemm_s4_f16_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
}

cudaError_t gemm_tc_launch(const GemmTcPlan& pl, GemmTcParams p, cudaStream_t st, bool pdl)
{
    p.units_per_cta   = pl.units_per_cta;
    p.parts_per_tile  = pl.parts_per_tile;
    p.total_units     = pl.total_units;
    p.slots_per_chunk = pl.slots_per_chunk;
    p.n_col_tiles     = pl.n_col_tiles;
    p.token_tile      = pl.token_tile;
    p.x_stages        = x_stages_for(pl.token_tile);
    p.a_stages        = a_stages_for(pl.token_tile);
    p.k_split         = k_split_for(pl.token_tile);
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
    return launch_kernel(gemm_s4_f16_tc_kernel, grid, dim3(kThreads), pl.smem_bytes, st, pdl, p, x_map);
}

}  // namespace tmb
