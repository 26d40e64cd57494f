// W4A16 GEMM for more than 16 tokens: tcgen05 tensor-core tiles with the accumulator in TMEM.
//
// A CTA computes C^T tiles of 128 output features x up to 128 tokens.  It is persistent and
// stream-K balanced over (128-feature tile, 128-row quantisation group) units, like the
// small-token kernel.  Warp roles:
//   warp 0      producer: bulk copies (TMA, mbarrier completion) of the packed int4 weight and the
//               {zero, scale} row of a unit into a ring
//   warp 10     streams the activation slice of the unit with cp.async into the
//               128-byte-swizzled K-major layout the tensor core reads
//   warp 1      allocates TMEM; one elected lane issues tcgen05.mma (M = 128, N = token tile,
//               K = 16 per instruction, fp16 x fp16 -> fp32) and commits completions to mbarriers
//   warps 2..9  expand the packed weight: lop3 nibble unpack, exact (q - z) in fp16, one fp16
//               multiply by the scale (bit-identical to the reference's dequantised weight,
//               kernels/gemm_s_f16/common.h:115-156, 218-235), stmatrix into the swizzled A tile;
//               at the end of a column tile they read the accumulator with tcgen05.ld and store C
//               (optionally through the SiLU(gate) * up epilogue) or the split-K partial
// Partial tiles of CTAs that share a column tile meet in scratch memory; the last CTA to arrive
// reduces them in a fixed order.  Every wait is bounded.
//
// Replaces the large-n end of GemmS4F16::Run (src/turbomind/kernels/gemm_s_f16/gemm_s4_f16.cu:
// 208-234; mma.sync tiles of gemm_template.h:338-444).
#include "common.cuh"
#include "gemm_s4_f16.h"

namespace tmb {
namespace {

constexpr int kTileN     = 128;  // output features per CTA tile (UMMA M)
constexpr int kGroup     = 128;  // K extent of a unit
constexpr int kTileBytes = 512;
constexpr int kWBytes    = 4 * 4 * kTileBytes;  // [4 k32][4 column tiles][512 B]
constexpr int kQBytes    = kTileN * 4;
constexpr int kWStage    = kWBytes + kQBytes;    // 8704
constexpr int kABytes    = 2 * kTileN * 128;     // two 64-wide K blocks of 128 rows x 128 B
constexpr int kWSTMax    = 16;                   // packed-weight stages: as many as fit (the HBM latency is
                                                 // hidden by the bytes in flight, ~64 KB per SM)
constexpr int kAST       = 2;                    // expanded-weight stages
constexpr int kXSTMax    = 8;                    // activation stages: as many as fit (GemmTcPlan::x_stages), and a
                                                 // slice is published x_stages - 2 iterations after it was
                                                 // issued: that many loads are in flight, and publishing
                                                 // slice j waits at most for the MMA of slice j - 2
constexpr int kDqWarps   = 8;
constexpr int kXWarp     = 2 + kDqWarps;         // warp that streams the activations
constexpr int kThreads   = (3 + kDqWarps) * 32;
constexpr int kTmemCols  = 128;

struct Bars {
    uint64_t w_full[kWSTMax], w_empty[kWSTMax];
    uint64_t a_full[kAST], a_empty[kAST];
    uint64_t x_full[kXSTMax], x_empty[kXSTMax];
    uint64_t acc_full, acc_empty;
    uint32_t tmem_base;
    int      flag;
};

__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr)
{
    // K-major, 128-byte swizzle: 8-row groups 1024 B apart (SBO), leading offset 1, descriptor version 1
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46)
           | ((uint64_t)2 << 61);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a),
        "l"(desc_b),
        "r"(idesc),
        "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
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

__device__ __forceinline__ void stmatrix_x4(uint32_t addr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3)
{
    asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
                 : "memory");
}

__device__ __forceinline__ uint32_t hmul2_ftz(uint32_t a, uint32_t b)
{
    uint32_t r;
    asm("mul.ftz.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid)
{
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}

__device__ __forceinline__ void cp_async_wait_dyn(int n)
{
    switch (n) {
        case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
        case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
        case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
        case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
        case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    }
}

// bounded wait that also accumulates the cycles spent waiting (developer counters)
__device__ __forceinline__ bool timed_wait(uint64_t* bar, uint32_t parity, long long& acc)
{
    const long long t0 = clock64();
    const bool      ok = mbar_wait(bar, parity);
    acc += clock64() - t0;
    return ok;
}

__global__ void __launch_bounds__(kThreads, 1) gemm_s4_f16_tc_kernel(GemmTcParams p)
{
    long long dbg_w0 = 0, dbg_w1 = 0, dbg_w2 = 0;
    const long long dbg_t0 = clock64();
    const int kXST  = p.x_stages;
    const int kXLag = p.x_stages - 2;
    const int kWST  = p.w_stages;
    extern __shared__ unsigned char smem_dyn[];
    // tiles the tensor core reads must sit on 1024-byte boundaries (the swizzle is a function of
    // the address bits)
    const uint32_t raw  = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* sm   = smem_dyn + (base - raw);

    const int TT      = p.token_tile;             // UMMA N, multiple of 16, <= 128
    const int x_bytes = 2 * TT * 128;             // two K blocks of TT rows x 128 B
    unsigned char* a_ring = sm;                                   // kAST x kABytes
    unsigned char* x_ring = a_ring + kAST * kABytes;              // kXST x x_bytes (x_bytes % 1024 == 0 for TT % 8 == 0... TT*256)
    unsigned char* w_ring = x_ring + kXST * x_bytes;              // kWST x kWStage
    Bars*          bars   = reinterpret_cast<Bars*>(w_ring + kWST * kWStage);

    const int tid  = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    const int t0     = blockIdx.y * 128;
    const int t_rows = min(TT, p.T - t0);

    const int G       = p.K / kGroup;
    const int upc     = p.units_per_cta;
    const int u_begin = blockIdx.x * upc;
    const int u_end   = min(u_begin + upc, p.total_units);
    const int n_units = u_end - u_begin;
    const int n_tiles32 = p.N / 32;

    if (tid == 0) {
        for (int s = 0; s < kWSTMax; ++s) {
            mbar_init(&bars->w_full[s], 1);
            mbar_init(&bars->w_empty[s], kDqWarps);
        }
        for (int s = 0; s < kAST; ++s) {
            mbar_init(&bars->a_full[s], kDqWarps);
            mbar_init(&bars->a_empty[s], 1);
        }
        for (int s = 0; s < kXSTMax; ++s) {
            mbar_init(&bars->x_full[s], 32);
            mbar_init(&bars->x_empty[s], 1);
        }
        mbar_init(&bars->acc_full, 1);
        mbar_init(&bars->acc_empty, kDqWarps);
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
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0) {
        // ================================================================== weight producer
        const uint64_t pol_w = policy_evict_first();
        bool           dead  = false;
        int            jt = u_begin / G, g = u_begin - jt * G;
        for (int it = 0; it < n_units && !dead; ++it) {
            const int tile0 = jt * 4;
            const int ntw   = min(4, n_tiles32 - tile0);
            const int sw    = it % kWST;
            if (it >= kWST) {
                const bool ok = timed_wait(&bars->w_empty[sw], ((it / kWST) - 1) & 1, dbg_w0);
                if (!__all_sync(0xffffffffu, ok)) {
                    if (lane == 0) atomicOr(p.status, kStatusGemmPipeWait);
                    dead = true;
                    break;
                }
            }
            unsigned char* sb = w_ring + sw * kWStage;
            if (lane == 0) {
                mbar_arrive_expect_tx(&bars->w_full[sw], (uint32_t)(4 * ntw * kTileBytes + ntw * 128));
            }
            __syncwarp();
            if (lane < 4) {
                const size_t k32 = (size_t)g * 4 + lane;
                bulk_g2s_hint(sb + lane * 4 * kTileBytes, p.A + (k32 * n_tiles32 + tile0) * kTileBytes,
                              (uint32_t)(ntw * kTileBytes), &bars->w_full[sw], pol_w);
            }
            else if (lane == 4) {
                bulk_g2s_hint(sb + kWBytes, p.Q + ((size_t)g * p.N + (size_t)tile0 * 32) * 4, (uint32_t)(ntw * 128),
                              &bars->w_full[sw], pol_w);
            }
            if (++g == G) {
                g = 0;
                ++jt;
            }
        }
    }
    else if (warp == kXWarp) {
        // ================================================================== activation loader
        // slice [TT rows][128 k] of the unit's group -> two 64-wide K blocks, rows of 128 B with
        // their 16-byte chunks XOR-swizzled by (row & 7): the layout the tensor core expects.
        // Lane = (row & 3, chunk): 4 rows per pass.
        const int      ch   = lane & 7;
        const int      tr   = lane >> 3;
        const uint32_t sw0  = (uint32_t)((ch ^ tr) << 4);        // rows tr, tr + 8, ...
        const uint32_t sw1  = (uint32_t)((ch ^ (tr + 4)) << 4);  // rows tr + 4, tr + 12, ...
        bool           dead = false;
        int            g    = u_begin % G;
        for (int it = 0; it < n_units + kXLag; ++it) {
            if (it < n_units) {
                const int sx = it % kXST;
                if (!dead && it >= kXST) {
                    const bool ok = timed_wait(&bars->x_empty[sx], ((it / kXST) - 1) & 1, dbg_w0);
                    if (!__all_sync(0xffffffffu, ok)) {
                        if (lane == 0) atomicOr(p.status, kStatusGemmPipeWait);
                        dead = true;
                    }
                }
                if (!dead) {
                    const uint32_t       xb      = base + (uint32_t)(x_ring - sm) + sx * x_bytes;
                    const size_t         row_b   = (size_t)p.K * 2;
                    const unsigned char* src_col = p.X + ((size_t)g * kGroup + ch * 8) * 2;
#pragma unroll
                    for (int kb = 0; kb < 2; ++kb) {
                        const unsigned char* src = src_col + kb * 128 + (size_t)(t0 + tr) * row_b;
                        uint32_t             dst = xb + kb * (TT * 128) + tr * 128;
                        for (int t = tr; t < TT; t += 8) {
                            const bool ok0 = t < t_rows, ok1 = t + 4 < t_rows;
                            cp_async16_zfill(dst + sw0, ok0 ? src : p.X, ok0);
                            cp_async16_zfill(dst + 512 + sw1, ok1 ? src + 4 * row_b : p.X, ok1);
                            src += 8 * row_b;
                            dst += 1024;
                        }
                    }
                }
                if (++g == G) g = 0;
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            // the slice issued kXLag iterations ago has landed: publish it to the tensor core
            const int done = it - kXLag;
            if (done >= 0) {
                const long long tw = clock64();
                cp_async_wait_dyn(kXLag);
                dbg_w1 += clock64() - tw;
                fence_proxy_async_smem();
                if (!dead) mbar_arrive(&bars->x_full[done % kXST]);
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    else if (warp == 1) {
        // ================================================================== MMA issuer
        const uint32_t idesc = (1u << 4) | ((uint32_t)(TT >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);
        bool dead    = false;
        int  seg_idx = 0;
        bool first   = true;  // first MMA of the current segment overwrites the accumulator
        for (int it = 0; it < n_units; ++it) {
            const int u  = u_begin + it;
            const int g  = u % G;
            const int sa = it % kAST, sx = it % kXST;
            if (first && seg_idx > 0 && !dead) {
                // the epilogue of the previous segment must have drained the accumulator
                const bool ok = timed_wait(&bars->acc_empty, (seg_idx - 1) & 1, dbg_w2);
                if (!__all_sync(0xffffffffu, ok)) dead = true;
            }
            if (!dead) {
                const bool ok = timed_wait(&bars->a_full[sa], (it / kAST) & 1, dbg_w0)
                                && timed_wait(&bars->x_full[sx], (it / kXST) & 1, dbg_w1);
                if (!__all_sync(0xffffffffu, ok)) {
                    if (lane == 0) atomicOr(p.status, kStatusGemmPipeWait);
                    dead = true;
                }
            }
            tc_fence_after();
            if (!dead && lane == 0) {
                const uint32_t a_addr = base + (uint32_t)(a_ring - sm) + sa * kABytes;
                const uint32_t x_addr = base + (uint32_t)(x_ring - sm) + sx * x_bytes;
#pragma unroll
                for (int kb = 0; kb < 2; ++kb) {
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint64_t da = make_desc(a_addr + kb * (kTileN * 128) + ks * 32);
                        const uint64_t db = make_desc(x_addr + kb * (TT * 128) + ks * 32);
                        umma_f16(tmem, da, db, idesc, (first && kb == 0 && ks == 0) ? 0u : 1u);
                    }
                }
                umma_commit(&bars->a_empty[sa]);
                umma_commit(&bars->x_empty[sx]);
            }
            first = false;
            const bool seg_end = (it == n_units - 1) || (g == G - 1);
            if (seg_end) {
                if (!dead && lane == 0) umma_commit(&bars->acc_full);
                ++seg_idx;
                first = true;
            }
            __syncwarp();
        }
    }
    else {
        // ================================================================== expand + epilogue
        const int  dw   = warp - 2;       // 0..7
        const int  tile = dw & 3;         // 32-feature column tile expanded by this warp
        const int  kh   = dw >> 2;        // which pair of 32-row slabs of the group
        const int  r    = lane >> 2;
        const int  c    = lane & 3;
        const int  q4   = warp & 3;       // TMEM lane quarter this warp may read
        const int  chalf = dw >> 2;       // which half of the token columns it drains
        bool       dead = false;
        int        seg_idx = 0;
        const int  dtid = tid - 64;

        // stmatrix row address pattern: lane L supplies row (L & 7) of matrix (L >> 3):
        // matrices = {rows +0, k +0}, {rows +8, k +0}, {rows +0, k +8}, {rows +8, k +8}
        const int m_row = (lane & 7) + ((lane >> 3) & 1) * 8;  // row inside the 16-row half tile
        const int m_k8  = (lane >> 4) & 1;                     // which 8-wide k chunk of the 16

        for (int it = 0; it < n_units; ++it) {
            const int u     = u_begin + it;
            const int jt    = u / G;
            const int g     = u - jt * G;
            const int tile0 = jt * 4;
            const int ntw   = min(4, n_tiles32 - tile0);
            const int sw = it % kWST, sa = it % kAST;

            if (!dead) {
                bool ok = timed_wait(&bars->w_full[sw], (it / kWST) & 1, dbg_w0);
                if (ok && it >= kAST) ok = timed_wait(&bars->a_empty[sa], ((it / kAST) - 1) & 1, dbg_w1);
                if (!__all_sync(0xffffffffu, ok)) {
                    if (lane == 0) atomicOr(p.status, kStatusGemmPipeWait);
                    dead = true;
                }
            }
            if (!dead && tile < ntw) {
                tc_fence_after();
                const unsigned char* sb = w_ring + sw * kWStage;
                const __half2*       qs = reinterpret_cast<const __half2*>(sb + kWBytes) + tile * 32;
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
                const uint32_t a_addr = base + (uint32_t)(a_ring - sm) + sa * kABytes;
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    const int   k32 = kh * 2 + kk;  // 32-row slab of the group: k = 32 k32 .. +31
                    const uint4 w   = reinterpret_cast<const uint4*>(sb)[(k32 * 4 + tile) * 32 + lane];
                    const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int wi = 0; wi < 4; ++wi) {
                        const int k16 = wi >> 1;
                        const int a   = wi & 1;
                        uint32_t  f[4];
                        unpack_s4_minus_zero(wv[wi], z1024[a], nz64[a], f);
                        f[0] = hmul2_ftz(f[0], s_lo[a]);
                        f[1] = hmul2_ftz(f[1], s_hi[a]);
                        f[2] = hmul2_ftz(f[2], s_lo[a]);
                        f[3] = hmul2_ftz(f[3], s_hi[a]);
                        // destination row / 16-byte chunk of this lane's stmatrix row
                        const int n   = tile * 32 + a * 16 + m_row;           // row of the 128-row tile
                        const int k   = k32 * 32 + k16 * 16 + m_k8 * 8;       // 0..127 inside the group
                        const int kb  = k >> 6;
                        const int ch  = (k & 63) >> 3;
                        stmatrix_x4(a_addr + kb * (kTileN * 128) + n * 128 + ((ch ^ (n & 7)) << 4), f[0], f[1], f[2], f[3]);
                    }
                }
            }
            // expanded tile visible to the tensor core; packed stage free again
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && !dead) {
                mbar_arrive(&bars->a_full[sa]);
                mbar_arrive(&bars->w_empty[sw]);
            }

            const bool seg_end = (it == n_units - 1) || (g == G - 1);
            if (!seg_end) continue;

            // ---- column tile jt finished for this CTA: drain the accumulator ------------------
            const int c_first = (jt * G) / upc;
            const int c_last  = ((jt + 1) * G - 1) / upc;
            const int n_split = c_last - c_first + 1;
            const int col0    = jt * kTileN;
            if (!dead) {
                const bool ok = timed_wait(&bars->acc_full, seg_idx & 1, dbg_w2);
                if (!__all_sync(0xffffffffu, ok)) {
                    if (lane == 0) atomicOr(p.status, kStatusGemmTmemWait);
                    dead = true;
                }
            }
            tc_fence_after();
            const int n_row   = q4 * 32 + lane;         // feature row of the tile held by this thread
            const int n_glob  = col0 + n_row;
            const int ccount  = TT / 2;                 // token columns per warp
            float*    slot    = p.workspace + ((size_t)blockIdx.y * p.slots_per_chunk + blockIdx.x + jt) * (size_t)(128 * kTileN);
            if (!dead) {
                for (int cb = 0; cb < ccount; cb += 8) {
                    const int col = chalf * ccount + cb;
                    float     v[8];
                    tmem_ld8(tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)col, v);
                    if (n_split > 1) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) __stcg(slot + (size_t)(col + i) * kTileN + n_row, v[i]);
                    }
                    else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int t = t0 + col + i;
                            if (p.fused_silu) {
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
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0 && !dead) mbar_arrive(&bars->acc_empty);
            ++seg_idx;

            if (n_split > 1) {
                __threadfence();
                named_bar_sync(1, kDqWarps * 32);
                if (dtid == 0) {
                    int*      counter = p.counters + (size_t)blockIdx.y * p.n_col_tiles + jt;
                    const int ticket  = atomicAdd(counter, 1);
                    const int is_last = ticket == n_split - 1;
                    if (is_last) *counter = 0;
                    bars->flag = is_last;
                }
                named_bar_sync(1, kDqWarps * 32);
                if (bars->flag && !dead) {
                    __threadfence();
                    const int n_cols = min(kTileN, p.N - col0);
                    const int pairs  = n_cols / 2;
                    for (int i = dtid; i < t_rows * pairs; i += kDqWarps * 32) {
                        const int t  = i / pairs;
                        const int n  = (i - t * pairs) * 2;
                        float     v0 = 0.f, v1 = 0.f;
                        for (int cc = c_first; cc <= c_last; ++cc) {
                            const float* sl = p.workspace
                                              + ((size_t)blockIdx.y * p.slots_per_chunk + cc + jt) * (size_t)(128 * kTileN);
                            const float2 v = __ldcg(reinterpret_cast<const float2*>(sl + (size_t)t * kTileN + n));
                            v0 += v.x;
                            v1 += v.y;
                        }
                        const __half2 h = __floats2half2_rn(v0, v1);
                        if (p.fused_silu) {
                            const float2 uu   = __half22float2(h);
                            const float  silu = uu.x / (1.f + __expf(-uu.x));
                            p.C[(size_t)(t0 + t) * (p.N / 2) + (col0 + n) / 2] = __float2half_rn(silu * uu.y);
                        }
                        else {
                            *reinterpret_cast<__half2*>(p.C + (size_t)(t0 + t) * p.N + col0 + n) = h;
                        }
                    }
                }
                named_bar_sync(1, kDqWarps * 32);
            }
        }
    }

    if (p.debug != nullptr && blockIdx.x == 1 && blockIdx.y == 0 && lane == 0 && (warp <= 2 || warp == kXWarp)) {
        // developer counters of CTA 1: per role {total cycles, wait 0, wait 1, wait 2}
        const int role = warp == kXWarp ? 3 : warp;
        p.debug[role * 4 + 0] = clock64() - dbg_t0;
        p.debug[role * 4 + 1] = dbg_w0;
        p.debug[role * 4 + 2] = dbg_w1;
        p.debug[role * 4 + 3] = dbg_w2;
        if (warp == 0) p.debug[16] = n_units;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(kTmemCols) : "memory");
    }
}

}  // namespace

int gemm_tc_x_stages(int token_tile)
{
    return token_tile > 64 ? 3 : 4;
}

int gemm_tc_w_stages(int token_tile)
{
    const size_t fixed = 1024 + (size_t)kAST * kABytes + (size_t)gemm_tc_x_stages(token_tile) * 2 * token_tile * 128
                         + sizeof(Bars) + 64;
    int          n     = (int)((227 * 1024 - fixed) / (size_t)kWStage);
    return n > kWSTMax ? kWSTMax : n;
}

size_t gemm_tc_smem_bytes(int token_tile)
{
    return 1024 + (size_t)kAST * kABytes + (size_t)gemm_tc_x_stages(token_tile) * 2 * token_tile * 128
           + (size_t)gemm_tc_w_stages(token_tile) * kWStage + sizeof(Bars) + 64;
}

GemmTcPlan gemm_tc_plan(int N, int T, int K, int sm_count)
{
    GemmTcPlan pl{};
    pl.token_tile  = T >= 128 ? 128 : ((T + 15) / 16) * 16;
    pl.t_chunks    = (T + 127) / 128;
    pl.n_col_tiles = (N + kTileN - 1) / kTileN;
    const int G    = K / kGroup;
    pl.total_units = pl.n_col_tiles * G;
    int ctas       = sm_count < pl.total_units ? sm_count : pl.total_units;
    pl.units_per_cta   = (pl.total_units + ctas - 1) / ctas;
    pl.ctas            = (pl.total_units + pl.units_per_cta - 1) / pl.units_per_cta;
    pl.slots_per_chunk = pl.ctas + pl.n_col_tiles;
    pl.smem_bytes      = gemm_tc_smem_bytes(pl.token_tile);
    pl.workspace_floats = (size_t)pl.t_chunks * pl.slots_per_chunk * 128 * kTileN;
    pl.counter_ints     = (size_t)pl.t_chunks * pl.n_col_tiles;
    return pl;
}

cudaError_t gemm_tc_prepare(int max_smem)
{
    return cudaFuncSetAttribute(gemm_s4_f16_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
}

cudaError_t gemm_tc_launch(const GemmTcPlan& pl, GemmTcParams p, cudaStream_t st)
{
    p.units_per_cta   = pl.units_per_cta;
    p.total_units     = pl.total_units;
    p.slots_per_chunk = pl.slots_per_chunk;
    p.n_col_tiles     = pl.n_col_tiles;
    p.token_tile      = pl.token_tile;
    p.x_stages        = gemm_tc_x_stages(pl.token_tile);
    p.w_stages        = gemm_tc_w_stages(pl.token_tile);
    dim3 grid(pl.ctas, pl.t_chunks);
    gemm_s4_f16_tc_kernel<<<grid, kThreads, pl.smem_bytes, st>>>(p);
    return cudaGetLastError();
}

}  // namespace tmb
