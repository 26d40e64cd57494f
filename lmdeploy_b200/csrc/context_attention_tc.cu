// Prefill (context) attention on the tcgen05 tensor core: causal softmax(q k^T / sqrt(d)) v over the KV cache read in
// place, fp16 or int8 cache, head size 128.  Same interface and results as context_attention.cu (the mma.sync kernel it
// replaces as the default); what it stands in for in the reference is described there
// (LlamaContextAttentionLayer<T>::fusedMultiHeadAttention, src/turbomind/models/llama/LlamaContextAttentionLayer.cc:257-313).
//
// One CTA = 128 queries of one (sequence, head); key / value tiles of 64 rows, double-buffered in shared memory in the
// 128-byte-swizzled layout the tensor core reads (two 64-wide blocks of the 128 head dimensions per tile).
//   warps 0-3   thread = query row = TMEM lane.  They copy the tiles (cp.async for fp16; int8 rows go through registers
//               and are dequantised on the way), and per tile: read the scores S from TMEM (tcgen05.ld), mask, online
//               softmax in the log2 domain with one thread per row (no shuffles), write the probabilities as fp16 into
//               TMEM (tcgen05.st) where the second product takes them as its A operand, and rescale the output
//               accumulator only when a row's running maximum moved by more than 2^8 (the accumulator is fp32).
//   warp 4      allocates TMEM (256 columns: S 64, P 32, O 128); one lane issues S = Q K^T (both operands from shared
//               memory, M128 x N64 x K16, 8 per tile) and O += P V (A from TMEM, B = the value tile as an MN-major
//               operand, M128 x N128 x K16, 4 per tile) and commits to mbarriers.
// Two CTAs are resident per SM (97 KB of shared memory, 256 TMEM columns each), so one CTA's softmax overlaps the
// other's MMAs.  Tiles above the causal diagonal are never visited; the longest query tiles are scheduled first.
// Every barrier wait is bounded; on expiry a status bit is recorded and the CTA drains and leaves.
#include "common.cuh"
#include "context_attention.h"
#include "tm_b200.h"

namespace tmb {
namespace {

constexpr int kD        = 128;
constexpr int kBM       = 128;  // queries per CTA
constexpr int kBN       = 64;   // keys per tile
constexpr int kRowThreads = 128;
constexpr int kThreads  = 160;
constexpr int kQBytes   = kBM * kD * 2;        // 32 KB: two blocks of [128 rows][128 B]
constexpr int kQBlock   = kBM * 128;           // 16 KB
constexpr int kTileBytes = kBN * kD * 2;       // 16 KB: two blocks of [64 rows][128 B]
constexpr int kTBlock   = kBN * 128;           // 8 KB
constexpr int kTmemCols = 256;
constexpr int kColS = 0, kColP = 64, kColO = 128;

struct Bars {
    uint64_t kv_full[2];  // tile t's keys and values are in shared memory (128 arrivals)
    uint64_t s_full;      // S of tile t is in TMEM
    uint64_t p_full;      // P of tile t is in TMEM, O rescaled (128 arrivals)
    uint64_t o_full;      // every product is done
    uint32_t tmem_base;
    int      dead;
};
constexpr int kSmemBytes = 1024 + kQBytes + 4 * kTileBytes + 128;

// byte offset of 16-byte chunk `chunk` (0..15 over the 128 head dimensions) of row `row`; `block_bytes` = rows x 128
__device__ __forceinline__ uint32_t sw_off(int row, int chunk, int block_bytes)
{
    return (uint32_t)((chunk >> 3) * block_bytes + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

__device__ __forceinline__ void cp_async16z(uint32_t dst, const void* src, int bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

// K-major operand (rows of 128 B, 8-row groups 1024 B apart), 128-byte swizzle
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr)
{
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46)
           | ((uint64_t)2 << 61);
}
// MN-major operand: rows of the tile are K (keys), each row 128 B = 64 of the N (head dimension) values; groups of 8
// keys 1024 B apart, the second 64-wide block of N `block_bytes` further on
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t block_bytes)
{
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((block_bytes >> 4) & 0x3FFFu) << 16) | ((uint64_t)(1024 >> 4) << 32)
           | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc)
{
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t acc)
{
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(db), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void umma_commit_to(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// 32 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack2(float a, float b)
{
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// 4 int8 -> 4 halves, half(q * scale + zp) (llama_kernels.cu:309-316); the int -> float step through the mantissa of 2^23
__device__ __forceinline__ uint2 dequant4(uint32_t w, float scale, float zp)
{
    const uint32_t u  = w ^ 0x80808080u;
    const float    f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.f;
    const float    f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.f;
    const float    f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.f;
    const float    f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.f;
    uint2 r;
    r.x = pack2(__fmaf_rn(f0, scale, zp), __fmaf_rn(f1, scale, zp));
    r.y = pack2(__fmaf_rn(f2, scale, zp), __fmaf_rn(f3, scale, zp));
    return r;
}

template<bool INT8>
__global__ void __launch_bounds__(kThreads, 2) context_attention_tc_kernel(CtxParams p)
{
    extern __shared__ unsigned char smem_dyn[];
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5;
    const int bi = blockIdx.z, h = blockIdx.y;
    const int qt    = gridDim.x - 1 - blockIdx.x;  // the longest (latest) query tiles first
    const int tok0  = p.cu_seqlens[bi];
    const int q_len = p.cu_seqlens[bi + 1] - tok0;
    const int ctx   = p.context_length[bi];
    const int hist  = ctx - q_len;
    const int q0    = qt * kBM;
    if (q0 >= q_len) return;  // the whole CTA, before anything is set up
    // keys any query of this tile may see; never past the rows a cache head holds
    const int kv_end  = min(min(ctx, p.max_seq_len), hist + min(q0 + kBM, q_len));
    const int n_tiles = (kv_end + kBN - 1) / kBN;
    const int kvh     = h / p.n_rep;

    const uint32_t raw  = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;  // operand tiles on 1024-byte boundaries (the swizzle is a function of the address)
    unsigned char* sm   = smem_dyn + (base - raw);
    const uint32_t q_s  = base;
    const uint32_t kv_s = base + kQBytes;  // [buf][k | v]
    Bars*          bars = reinterpret_cast<Bars*>(sm + kQBytes + 4 * kTileBytes);

    if (tid == 0) {
        mbar_init(&bars->kv_full[0], kRowThreads);
        mbar_init(&bars->kv_full[1], kRowThreads);
        mbar_init(&bars->s_full, 1);
        mbar_init(&bars->p_full, kRowThreads);
        mbar_init(&bars->o_full, 1);
        bars->dead = 0;
        fence_mbar_init();
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "n"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_before();
    __syncthreads();
    tc_after();
    const uint32_t tmem = bars->tmem_base;

    if (warp < 4) {
        // ============================================================ copies, softmax, output: thread = query row
        const size_t         head_off = p.offset + (size_t)kvh * p.max_seq_len * kD;  // elements
        const unsigned char* k_base   = static_cast<const unsigned char*>(p.k_cache[bi]) + head_off * (INT8 ? 1 : 2);
        const unsigned char* v_base   = static_cast<const unsigned char*>(p.v_cache[bi]) + head_off * (INT8 ? 1 : 2);
        auto load_tile_f16 = [&](int t, int buf) {
            const int key0 = t * kBN;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const int      c = tid + r * kRowThreads, row = c >> 4, chunk = c & 15;
                const bool     ok  = key0 + row < kv_end;
                const size_t   src = ((size_t)(ok ? key0 + row : 0) * kD + chunk * 8) * 2;
                const uint32_t dst = kv_s + buf * 2 * kTileBytes + sw_off(row, chunk, kTBlock);
                cp_async16z(dst, k_base + src, ok ? 16 : 0);
                cp_async16z(dst + kTileBytes, v_base + src, ok ? 16 : 0);
            }
        };
        uint4 stage_k[4], stage_v[4];  // int8 only: the next tile on its way from global to shared memory
        auto fetch_tile_s8 = [&](int t) {
            const int key0 = t * kBN;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int  c = tid + r * kRowThreads, row = c >> 3, chunk = c & 7;
                const bool ok = key0 + row < kv_end;
                stage_k[r] = stage_v[r] = make_uint4(0, 0, 0, 0);
                if (ok) {
                    const size_t src = (size_t)(key0 + row) * kD + chunk * 16;
                    stage_k[r]       = *reinterpret_cast<const uint4*>(k_base + src);
                    stage_v[r]       = *reinterpret_cast<const uint4*>(v_base + src);
                }
            }
        };
        auto store_tile_s8 = [&](int t, int buf) {
            const int key0 = t * kBN;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int  c = tid + r * kRowThreads, row = c >> 3, chunk = c & 7;
                const bool ok = key0 + row < kv_end;  // rows past the end stay exact zeros (not the zero point)
                unsigned char* dst = sm + kQBytes + buf * 2 * kTileBytes;
                uint4 k0 = make_uint4(0, 0, 0, 0), k1 = k0, v0 = k0, v1 = k0;
                if (ok) {
                    const uint2 a = dequant4(stage_k[r].x, p.k_scale, p.k_zp), b = dequant4(stage_k[r].y, p.k_scale, p.k_zp);
                    const uint2 c2 = dequant4(stage_k[r].z, p.k_scale, p.k_zp), d = dequant4(stage_k[r].w, p.k_scale, p.k_zp);
                    k0 = make_uint4(a.x, a.y, b.x, b.y), k1 = make_uint4(c2.x, c2.y, d.x, d.y);
                    const uint2 e = dequant4(stage_v[r].x, p.v_scale, p.v_zp), f = dequant4(stage_v[r].y, p.v_scale, p.v_zp);
                    const uint2 g2 = dequant4(stage_v[r].z, p.v_scale, p.v_zp), hh = dequant4(stage_v[r].w, p.v_scale, p.v_zp);
                    v0 = make_uint4(e.x, e.y, f.x, f.y), v1 = make_uint4(g2.x, g2.y, hh.x, hh.y);
                }
                *reinterpret_cast<uint4*>(dst + sw_off(row, 2 * chunk, kTBlock))                  = k0;
                *reinterpret_cast<uint4*>(dst + sw_off(row, 2 * chunk + 1, kTBlock))              = k1;
                *reinterpret_cast<uint4*>(dst + kTileBytes + sw_off(row, 2 * chunk, kTBlock))     = v0;
                *reinterpret_cast<uint4*>(dst + kTileBytes + sw_off(row, 2 * chunk + 1, kTBlock)) = v1;
            }
        };

        // ---- prologue: the query tile and key / value tile 0
        {
            const __half* qsrc = p.q + ((size_t)bi * p.H + h) * p.max_q_len * kD;
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                const int  c = tid + r * kRowThreads, row = c >> 4, chunk = c & 15;
                const bool ok = q0 + row < q_len;
                cp_async16z(q_s + sw_off(row, chunk, kQBlock), qsrc + (size_t)(ok ? q0 + row : 0) * kD + chunk * 8, ok ? 16 : 0);
            }
        }
        if (INT8) {
            fetch_tile_s8(0);
            store_tile_s8(0, 0);
        }
        else {
            load_tile_f16(0, 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");

        const int      qi        = q0 + tid;
        const bool     row_live  = qi < q_len;
        const int      limit     = row_live ? min(hist + qi, kv_end - 1) : -1;  // last key this row may see
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        float          m_used = -INFINITY, l = 0.f;
        bool           dead = false;
        for (int t = 0; t < n_tiles; ++t) {
            const int buf = t & 1;
            if (INT8 && t > 0) store_tile_s8(t, buf);  // fetched to registers during the tile before
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            fence_async_smem();  // copies and stores of this thread become visible to the tensor core's reads
            mbar_arrive(&bars->kv_full[buf]);
            // the outcome is made uniform across the warp: the TMEM loads and stores below are warp-wide instructions
            if (!__all_sync(0xffffffffu, mbar_wait(&bars->s_full, t & 1, p.max_wait_cycles))) {
                atomicOr(p.status, kStatusGemmPipeWait);
                *(volatile int*)&bars->dead = 1;
                dead = true;
                break;
            }
            tc_after();
            // S of this tile is complete, so every product on the tile before it is too: its buffers are free
            if (t + 1 < n_tiles) {
                if (INT8) {
                    fetch_tile_s8(t + 1);
                }
                else {
                    load_tile_f16(t + 1, buf ^ 1);
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");

            uint32_t s0[32], s1[32];
            tmem_ld32(lane_base + kColS, s0);
            tmem_ld32(lane_base + kColS + 32, s1);
            const int key0 = t * kBN;
            // raw scores stay as they are; the softmax scale goes into the exponent's multiply-add.  Only tiles that
            // touch the causal diagonal or the end of the keys mask anything (the same for every row of the CTA).
            float mx = -INFINITY;
            if (key0 + kBN - 1 > hist + q0 || key0 + kBN > kv_end || !row_live) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (key0 + i > limit) s0[i] = 0xff800000u;       // -inf
                    if (key0 + 32 + i > limit) s1[i] = 0xff800000u;
                }
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(__uint_as_float(s0[i]), __uint_as_float(s1[i])));
            mx *= p.scale_log2;  // the scale is positive
            // the running maximum follows only when it is left behind by more than 2^8: p <= 256 fits fp16, the sums are
            // fp32, and the accumulator needs rescaling a few times per row instead of once per tile
            float alpha = 1.f;
            if (mx > m_used + 8.f) {
                alpha  = ex2(m_used - mx);  // 0 on the first tile
                m_used = mx;
            }
            const float nm  = m_used == -INFINITY ? 0.f : -m_used;
            float       sum = 0.f;
            uint32_t    pr[32];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float a = ex2(fmaf(__uint_as_float(s0[2 * i]), p.scale_log2, nm)), b = ex2(fmaf(__uint_as_float(s0[2 * i + 1]), p.scale_log2, nm));
                const float c = ex2(fmaf(__uint_as_float(s1[2 * i]), p.scale_log2, nm)), d = ex2(fmaf(__uint_as_float(s1[2 * i + 1]), p.scale_log2, nm));
                sum += (a + b) + (c + d);
                pr[i]      = pack2(a, b);
                pr[16 + i] = pack2(c, d);
            }
            l = l * alpha + sum;
            if (t > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t o[32];
                    tmem_ld32(lane_base + kColO + 32 * c, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(lane_base + kColO + 32 * c, o);
                }
            }
            tmem_st32(lane_base + kColP, pr);
            tmem_wait_st();
            tc_before();
            mbar_arrive(&bars->p_full);
        }
        // ---- normalise and store: out[token, h * 128 + d]
        if (!dead && !__all_sync(0xffffffffu, mbar_wait(&bars->o_full, 0, p.max_wait_cycles))) {
            atomicOr(p.status, kStatusGemmTmemWait);
            dead = true;
        }
        tc_after();
        if (!dead && *(volatile int*)&bars->dead == 0) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t o[32];
                tmem_ld32(lane_base + kColO + 32 * c, o);
                if (row_live) {
                    __half* dst = p.out + ((size_t)(tok0 + qi) * p.H + h) * kD + 32 * c;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 v;
                        v.x = pack2(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
                        v.y = pack2(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
                        v.z = pack2(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
                        v.w = pack2(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + 8 * i) = v;
                    }
                }
            }
        }
    }
    else if ((tid & 31) == 0) {
        // ============================================================ MMA issuer
        const uint32_t idesc_qk = (1u << 4) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
        const uint32_t idesc_pv = (1u << 4) | (1u << 16) | ((uint32_t)(kD >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);  // B is MN-major
        bool           ok       = true;
        for (int t = 0; t < n_tiles && ok; ++t) {
            const int buf = t & 1;
            if (!mbar_wait(&bars->kv_full[buf], (t >> 1) & 1, p.max_wait_cycles)) {
                ok = false;
                break;
            }
            tc_after();
            const uint32_t k_addr = kv_s + buf * 2 * kTileBytes, v_addr = k_addr + kTileBytes;
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
                const uint64_t dq = desc_kmajor(q_s + blk * kQBlock), dk = desc_kmajor(k_addr + blk * kTBlock);
#pragma unroll
                for (int j = 0; j < 4; ++j) umma_ss(tmem + kColS, dq + (uint64_t)(2 * j), dk + (uint64_t)(2 * j), idesc_qk, (blk | j) ? 1u : 0u);
            }
            umma_commit_to(&bars->s_full);
            if (!mbar_wait(&bars->p_full, t & 1, p.max_wait_cycles)) {
                ok = false;
                break;
            }
            tc_after();
            const uint64_t dv = desc_mnmajor(v_addr, kTBlock);
#pragma unroll
            for (int j = 0; j < 4; ++j) umma_ts(tmem + kColO, tmem + kColP + 8 * j, dv + (uint64_t)(128 * j), idesc_pv, (t | j) ? 1u : 0u);
        }
        if (!ok) {
            atomicOr(p.status, kStatusGemmPipeWait);
            *(volatile int*)&bars->dead = 1;
        }
        umma_commit_to(&bars->o_full);  // arrives when everything issued so far is complete (also on the give-up path)
    }

    tc_before();
    __syncthreads();
    if (warp == 4) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(kTmemCols) : "memory");
    }
}

}  // namespace

cudaError_t context_attention_tc_launch(const CtxParams& p, bool int8, int batch, cudaStream_t st)
{
    auto kernel = int8 ? context_attention_tc_kernel<true> : context_attention_tc_kernel<false>;
    // per call, like every attribute in this library that depends on the current device; cheap next to the kernel
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    const dim3 grid((p.max_q_len + kBM - 1) / kBM, p.H, batch);
    return launch_kernel(kernel, grid, dim3(kThreads), kSmemBytes, st, false, p);
}

}  // namespace tmb
