// Decode-step masked multi-head attention over a per-sequence KV cache (fp16 or int8), one new
// query token per sequence.  Replaces mmha::masked_multihead_attention_kernel
// (src/turbomind/kernels/decoder_masked_multihead_attention/
// decoder_masked_multihead_attention_template.cuh:1218-1913 of lmdeploy v0.0.9), which walks the
// whole sequence with one CTA per (head, sequence), three passes, no split along the sequence and
// one KV read per *query* head.
//
// Here a CTA owns (sequence, KV head, split of the sequence).  All query heads that share the KV
// head (up to 8 per CTA) ride on the same KV bytes.  Each of the 4 warps streams its own 16-token
// blocks of K and V through a private cp.async ring (XOR-swizzled 16-byte chunks, so that every
// shared-memory read below is conflict free) and keeps an online-softmax state:
//   S^T[token, head] = K . Q^T      mma.m16n8k16, A = K rows (int8 expanded to exact fp16
//                                   integers in registers), B = Q fragments held in registers
//   P^T -> fp16, transposed in registers with movmatrix to become the B operand of
//   O^T[d, head]     = V^T . P^T    A = V with token pairs interleaved by byte permutes
// RoPE on the new q/k, the KV append (with int8 quantisation) and the new token's own score are
// fused in.  Splits meet in scratch memory; the last CTA to arrive for a (sequence, KV head)
// merges them in a fixed order (no CTA waits for another).
#include "common.cuh"
#include "mmha.h"

#include <cfloat>

#ifdef TM_B200_GEMM_TRACE
// Developer build only (never defined by lmdeploy_b200/build.py): per-CTA time stamps of one launch.
__device__ unsigned long long g_mmha_trace[4096][12];
__device__ int                g_mmha_launch;
extern "C" __attribute__((visibility("default"))) int tm_dev_mmha_trace(unsigned long long* out, int want_launch)
{
    cudaMemcpyFromSymbol(out, g_mmha_trace, sizeof(unsigned long long) * 4096 * 12);
    int z = -want_launch;
    cudaMemcpyToSymbol(g_mmha_launch, &z, sizeof(z));
    return 0;
}
__device__ __forceinline__ unsigned long long mmha_globaltimer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define MMHA_TRACE(slot)                                                                                               \
    do {                                                                                                                   \
        if (trace_on && threadIdx.x == 0) g_mmha_trace[trace_id][slot] = mmha_globaltimer();                               \
    } while (0)
#else
#define MMHA_TRACE(slot) do { } while (0)
#endif

namespace tmb {
namespace {

constexpr int kD          = 128;  // head dim
constexpr int kMaxWarps   = 4;  // warps per CTA: 4, 2 or 1 (template parameter W of the kernel)
constexpr int kBlockTok   = 16;   // tokens per warp block
constexpr int kHeadsPerCta = 8;
constexpr float kLog2e    = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid)
{
    const uint32_t d = smem_u32(dst);
    const int      n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
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

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t hsub2(uint32_t a, uint32_t b)
{
    uint32_t r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a)
{
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(a));
    return r;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi)
{
    const __half2 h = __floats2half2_rn(lo, hi);
    return reinterpret_cast<const uint32_t&>(h);
}
__device__ __forceinline__ uint32_t lds32(const unsigned char* p)
{
    return *reinterpret_cast<const uint32_t*>(p);
}
__device__ __forceinline__ uint4 lds128(const unsigned char* p)
{
    return *reinterpret_cast<const uint4*>(p);
}

constexpr uint32_t kMagic64  = 0x64646464u;  // high bytes of half 1024 + x
constexpr uint32_t kBias1152 = 0x64806480u;  // half2{1152, 1152}: 1024 + 128
constexpr uint32_t kSignFlip = 0x80808080u;

// four int8 (one word, sign bits already flipped) -> two half2 holding 1152 + value (exact in
// fp16).  The constant 1152 is taken out again after the MMA, in fp32: from the scores through
// the per-head sum of q, from the outputs through the sum of the probabilities.
constexpr float kOffset = 1152.f;
__device__ __forceinline__ void s8x4_to_h2x2(uint32_t x, uint32_t& lo, uint32_t& hi)
{
    lo = prmt(x, kMagic64, 0x4140);
    hi = prmt(x, kMagic64, 0x4342);
}

// query-fragment column of lane c at MMA step j: the 4 consecutive head-dim indices d0..d0+3
// that K-slot (2c, 2c+1, 2c+8, 2c+9) stand for.  Chosen so that a lane reads whole 16-byte
// chunks of a K row: int8 row = 8 chunks, lane c owns chunks {2c, 2c+1}; fp16 row = 16 chunks,
// lane c owns {2c, 2c+1, 2c+8, 2c+9}.
template<bool INT8>
__device__ __forceinline__ int qk_d0(int c, int j)
{
    return INT8 ? 32 * c + 4 * j : 16 * c + 64 * (j >> 2) + 4 * (j & 3);
}

template<bool INT8, int W>
__global__ void __launch_bounds__(W * 32, (INT8 ? 16 : 12) / W) mmha_decode_kernel(MmhaParams p)
{
    constexpr int kWarps   = W;
    constexpr int kThreads = W * 32;
    constexpr int ROWB   = INT8 ? kD : 2 * kD;        // bytes per cached token row
    constexpr int CPR    = ROWB / 16;                 // 16-byte chunks per row
    constexpr int NSTAGE = 3;
    constexpr int TILEB  = kBlockTok * ROWB;          // one K (or V) block of a warp
    constexpr int WARPB  = NSTAGE * 2 * TILEB;        // ring of one warp

    extern __shared__ __align__(128) unsigned char smem[];
    // [warps][NSTAGE][K tile | V tile]   (reused by the merge)  | q_s[8][128] half | knew[128] half |
    // vnew[128] half | sumq[8] f32 | snew[8] f32 | flag
    unsigned char* ring   = smem;
    __half*        q_s    = reinterpret_cast<__half*>(smem + kWarps * WARPB);
    __half*        knew_s = q_s + kHeadsPerCta * kD;
    __half*        vnew_s = knew_s + kD;
    float*         sumq_s = reinterpret_cast<float*>(vnew_s + kD);
    float*         snew_s = sumq_s + kHeadsPerCta;
    int*           flag_s = reinterpret_cast<int*>(snew_s + kHeadsPerCta);

    const int tid  = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int g    = lane >> 2;
    const int c    = lane & 3;
#ifdef TM_B200_GEMM_TRACE
    const int  trace_id = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    const bool trace_on = *(volatile int*)&g_mmha_launch == 0 && trace_id < 4096;
    MMHA_TRACE(0);
#endif

    // `order`, `finished` and `lengths` are written by kernels earlier in the stream, but never by the
    // kernel directly ahead of this one (a GEMM), whose own wait has already covered them.  A CTA
    // that has nothing to do must still wait for that kernel before it exits: a grid that completes
    // without waiting would let the kernel after this one start while the one before it still runs.
    int                  bi, tlength, fin = 0;
    const unsigned char *k_base, *v_base;
    // rotation coefficients of this CTA's sequence (table in launch order): requested together with the record
    float2 rope_pre = make_float2(1.f, 0.f);
    if (p.rope_table != nullptr && 2 * (tid % 64) < p.rot_dim) rope_pre = __ldg(p.rope_table + (size_t)blockIdx.z * 64 + tid % 64);
    if (p.desc != nullptr) {
        const uint4 d0 = __ldg(reinterpret_cast<const uint4*>(p.desc + blockIdx.z));
        const uint4 d1 = __ldg(reinterpret_cast<const uint4*>(p.desc + blockIdx.z) + 1);
        k_base  = reinterpret_cast<const unsigned char*>(((unsigned long long)d0.y << 32) | d0.x);
        v_base  = reinterpret_cast<const unsigned char*>(((unsigned long long)d0.w << 32) | d0.z);
        tlength = (int)d1.x, bi = (int)d1.y, fin = (int)d1.z;
    }
    else {
        bi = p.order != nullptr ? p.order[blockIdx.z] : blockIdx.z;
        if (p.finished != nullptr) fin = p.finished[bi];
        tlength = 0;
        k_base = v_base = nullptr;
    }
    if (fin) {
        pdl_wait();
        pdl_launch_dependents();
        return;  // template.cuh:1298-1300: neither out nor the cache is touched
    }
    const int rep    = p.H / p.Hkv;
    const int n_hb   = (rep + kHeadsPerCta - 1) / kHeadsPerCta;
    const int kvh    = blockIdx.y / n_hb;
    const int hb     = blockIdx.y - kvh * n_hb;
    const int head0  = kvh * rep + hb * kHeadsPerCta;      // first query head of this CTA
    const int nheads = min(kHeadsPerCta, rep - hb * kHeadsPerCta);

    if (p.desc == nullptr) {
        tlength = p.lengths[bi];
        k_base  = reinterpret_cast<const unsigned char*>(p.k_cache[bi]);
        v_base  = reinterpret_cast<const unsigned char*>(p.v_cache[bi]);
    }
    const int first   = max(0, tlength + 1 - p.S_max);
    const int n_past  = tlength - first;
    const int n_split = max(1, (n_past + p.chunk - 1) / p.chunk);
    const int split   = blockIdx.x;
    if (split >= n_split) {
        pdl_wait();
        pdl_launch_dependents();
        return;
    }
    const bool last_split = (split == n_split - 1);
    const int  s0         = first + split * p.chunk;
    const int  s1         = min(s0 + p.chunk, tlength);
    const int  n_blocks   = (max(s1 - s0, 0) + kBlockTok - 1) / kBlockTok;

    const unsigned char* kc = k_base + (p.cache_offset + (size_t)kvh * p.S_max * kD) * (ROWB / kD);
    const unsigned char* vc = v_base + (p.cache_offset + (size_t)kvh * p.S_max * kD) * (ROWB / kD);

    // ---------------------------------------------------------------- KV ring: start the loads
    unsigned char* my_ring = ring + warp * WARPB;
    // per-lane constants of the copy pattern: lane covers chunk (lane % CPR) of token rows
    // (lane / CPR) + i * (32 / CPR)
    constexpr int kRowsPerPass = 32 / CPR;
    const int     cp_tok       = lane / CPR;
    const int     cp_ch        = lane % CPR;
    const int     slot_base    = s0 % p.S_max;  // ring slot of token s0
    auto issue_block = [&](int blk, int stage) {
        // blk: index among this warp's blocks; first token of the block relative to s0:
        const int      rel0 = (blk * kWarps + warp) * kBlockTok;
        unsigned char* ks   = my_ring + stage * 2 * TILEB;
        unsigned char* vs   = ks + TILEB;
        int            slot = slot_base + rel0 + cp_tok;  // < 3 * S_max: at most two wraps
        if (slot >= p.S_max) slot -= p.S_max;
        if (slot >= p.S_max) slot -= p.S_max;
#pragma unroll
        for (int i = 0; i < kBlockTok / kRowsPerPass; ++i) {
            const int      tok   = cp_tok + i * kRowsPerPass;
            const bool     valid = s0 + rel0 + tok < s1;
            const uint32_t src   = valid ? (uint32_t)slot * ROWB + cp_ch * 16 : 0u;
            const int      dst   = tok * ROWB + ((cp_ch ^ (tok & 7)) << 4);
            cp_async16(ks + dst, kc + src, valid);
            cp_async16(vs + dst, vc + src, valid);
            slot += kRowsPerPass;
            if (slot >= p.S_max) slot -= p.S_max;
        }
    };
    const int my_blocks = (n_blocks > warp) ? (n_blocks - warp + kWarps - 1) / kWarps : 0;
    // every stage of the ring is requested up front: nothing is being read yet
#pragma unroll
    for (int sidx = 0; sidx < NSTAGE; ++sidx) {
        if (sidx < my_blocks) {
            issue_block(sidx, sidx);
        }
        cp_async_commit();
    }

    MMHA_TRACE(1);   // first copies issued

    // ---------------------------------------------------------------- q (+k, v of the new token)
    // The rotation coefficients depend on the position only: they are taken from the table the decode driver fills
    // once per step (positions do not depend on layer or head), or worked out here, before the wait for the kernel
    // ahead of this one.  After the wait every thread requests all of its q / k / v values at once (one round trip to
    // L2, not one per row) and only then rotates and stores them.
    constexpr int kPairThreads = kThreads < 64 ? kThreads : 64;
    constexpr int kParts       = kThreads / kPairThreads;                          // 1 or 2 threads share a pair index
    constexpr int kPairIters   = 64 / kPairThreads;                                // pair indices per thread
    constexpr int kRowIters    = (kHeadsPerCta + 2 + kParts - 1) / kParts;         // rows per thread: 8 query heads, k, v
    const int     q_part       = tid / kPairThreads;                               // which rows this thread handles
    float         cs[kPairIters], sn[kPairIters];
    float         logn = 1.f;
    {
        float base = p.rope_base;
        if (p.use_dynamic_ntk) {
            // decoder_masked_multihead_attention_utils.h:862-871, seq_len = length + 1
            const float seq_len = (float)(tlength + 1);
            if (seq_len >= (float)p.max_pos) {
                const float alpha = fmaxf(exp2f(ceilf(log2f(seq_len / (float)p.max_pos) + 1.f)) - 1.f, 1.f);
                base *= powf(alpha, (float)p.rot_dim / ((float)p.rot_dim - 2.f));
            }
        }
        if (p.use_logn && (float)(tlength + 1) > (float)p.max_pos) {
            logn = log2f((float)(tlength + 1)) / log2f((float)p.max_pos);  // utils.h:854-860
        }
        const int   pad = p.padding ? p.padding[bi] : 0;
        const float pos = p.pos_from_length ? (float)tlength : (float)(p.timestep - pad);  // template.cuh:1391-1395
#pragma unroll
        for (int it = 0; it < kPairIters; ++it) {
            const int pr = tid % kPairThreads + it * kPairThreads;  // pair index: elements 2pr, 2pr+1
            cs[it] = 1.f, sn[it] = 0.f;
            if (2 * pr < p.rot_dim) {
                if (p.rope_table != nullptr) {
                    // kPairIters == 1 whenever the table is used with 64 or more threads; narrower CTAs fetch the rest here
                    const float2 t = (it == 0 && kPairThreads == 64) ? rope_pre : __ldg(p.rope_table + (size_t)blockIdx.z * 64 + pr);
                    cs[it] = t.x, sn[it] = t.y;
                }
                else {
                    const float inv_freq = pos / powf(base, (float)(2 * pr) / (float)p.rot_dim);  // utils.h:885-889
                    sincosf(inv_freq, &sn[it], &cs[it]);
                }
            }
        }
    }
    MMHA_TRACE(8);   // coefficients done

    // The cache rows requested above were written by earlier steps; q, k, v of the new token come
    // from the kernel before this one.
    pdl_wait();
    pdl_launch_dependents();
    {
        const __half* xrow = p.qkv + (size_t)bi * p.stride;
        __half2       raw[kPairIters][kRowIters];
        // rows 0..7: query heads (zero beyond nheads); row 8: k; row 9: v
        auto column_of = [&](int row) {
            return row < kHeadsPerCta ? (head0 + row) * kD : (row == kHeadsPerCta ? (p.H + kvh) * kD : (p.H + p.Hkv + kvh) * kD);
        };
        auto wanted = [&](int row) {
            return row < kHeadsPerCta + 2 && (row < kHeadsPerCta ? row < nheads : last_split);
        };
#pragma unroll
        for (int it = 0; it < kPairIters; ++it) {
            const int pr = tid % kPairThreads + it * kPairThreads;
#pragma unroll
            for (int ri = 0; ri < kRowIters; ++ri) {
                const int row = q_part + ri * kParts;
                raw[it][ri]   = __float2half2_rn(0.f);
                if (wanted(row)) {
                    const int col = column_of(row);
                    raw[it][ri]   = *reinterpret_cast<const __half2*>(xrow + col + 2 * pr);
                    if (p.bias) {
                        raw[it][ri] = __hadd2(raw[it][ri], *reinterpret_cast<const __half2*>(p.bias + col + 2 * pr));  // fp16 add, :1381-1382
                    }
                }
            }
        }
#pragma unroll
        for (int it = 0; it < kPairIters; ++it) {
            const int  pr  = tid % kPairThreads + it * kPairThreads;
            const bool rot = 2 * pr < p.rot_dim;
#pragma unroll
            for (int ri = 0; ri < kRowIters; ++ri) {
                const int  row  = q_part + ri * kParts;
                const bool is_q = row < kHeadsPerCta;
                if (row >= kHeadsPerCta + 2 || (!is_q && !last_split)) continue;
                float2 x = __half22float2(raw[it][ri]);
                if (rot && row <= kHeadsPerCta) {  // q and k only
                    x = make_float2(cs[it] * x.x - sn[it] * x.y, cs[it] * x.y + sn[it] * x.x);  // utils.h:891-897
                }
                __half2 h = __floats2half2_rn(x.x, x.y);
                if (is_q && logn != 1.f) {
                    h = __hmul2(h, __float2half2_rn(logn));
                }
                __half* dstp = is_q ? q_s + row * kD : (row == kHeadsPerCta ? knew_s : vnew_s);
                *reinterpret_cast<__half2*>(dstp + 2 * pr) = h;
            }
        }
    }
    MMHA_TRACE(9);   // q, k, v staged by this thread
    __syncthreads();
    MMHA_TRACE(10);

    // per-head sum of q (for a non-zero K zero point) and the new token's own score
    for (int h = warp; h < kHeadsPerCta; h += kWarps) {
        if (h >= nheads) {  // rows of zeros
            if (lane == 0) sumq_s[h] = snew_s[h] = 0.f;
            continue;
        }
        float sq = 0.f, dot = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float q = __half2float(q_s[h * kD + lane * 4 + i]);
            sq += q;
            if (last_split) {
                dot += q * __half2float(knew_s[lane * 4 + i]);
            }
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) {
            sq += __shfl_xor_sync(0xffffffffu, sq, m);
            dot += __shfl_xor_sync(0xffffffffu, dot, m);
        }
        if (lane == 0) {
            sumq_s[h] = sq;
            snew_s[h] = dot * p.inv_sqrt_dh * kLog2e;  // log2 units
        }
    }

    MMHA_TRACE(11);  // sums done
    __syncthreads();

    // ---------------------------------------------------------------- Q fragments, softmax state
    uint32_t qf[8][2];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int d0 = qk_d0<INT8>(c, j);
        qf[j][0]     = *reinterpret_cast<const uint32_t*>(q_s + g * kD + d0);
        qf[j][1]     = *reinterpret_cast<const uint32_t*>(q_s + g * kD + d0 + 2);
    }
    // logits in log2 units: t = S_raw * alpha + beta[head]
    const float alpha = (INT8 ? p.k_scale : 1.f) * p.inv_sqrt_dh * kLog2e;
    float       beta[2];
    // int8: S_raw = sum_d q_d (1152 + k8_d); k = k8 * k_scale + k_zp
    beta[0] = INT8 ? (p.k_zp - kOffset * p.k_scale) * sumq_s[2 * c] * p.inv_sqrt_dh * kLog2e : 0.f;
    beta[1] = INT8 ? (p.k_zp - kOffset * p.k_scale) * sumq_s[2 * c + 1] * p.inv_sqrt_dh * kLog2e : 0.f;

    float m_run[2] = {-INFINITY, -INFINITY};  // heads 2c, 2c+1
    float l_run[2] = {0.f, 0.f};              // this lane's share (token rows g, g+8)
    float acc[8][4];
#pragma unroll
    for (int a = 0; a < 8; ++a) acc[a][0] = acc[a][1] = acc[a][2] = acc[a][3] = 0.f;
    float psum[4] = {0.f, 0.f, 0.f, 0.f};  // int8: sum over tokens of the fp16 probabilities (every row alike)

    // byte offset, inside a V tile, of word g of token rows 2c, 2c+1, 2c+8, 2c+9 (swizzled)
    int v_off[4];
    {
        const int tk0[4] = {2 * c, 2 * c + 1, 2 * c + 8, 2 * c + 9};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            v_off[e] = tk0[e] * ROWB + ((((g >> 2) ^ (tk0[e] & 7)) << 4) | ((g & 3) << 2));
        }
    }

    // ---------------------------------------------------------------- main loop over this warp's blocks
    MMHA_TRACE(2);   // prologue done
    for (int blk = 0; blk < my_blocks; ++blk) {
        cp_async_wait<NSTAGE - 1>();   // block blk has landed; the NSTAGE - 1 blocks after it may still be on their way
        __syncwarp();
        if (blk == 0) MMHA_TRACE(3);   // first block landed
        const int            stage = blk % NSTAGE;
        const unsigned char* ks    = my_ring + stage * 2 * TILEB;
        const unsigned char* vs    = ks + TILEB;
        const int            tok0  = s0 + (blk * kWarps + warp) * kBlockTok;

        // ---- S^T = K . Q^T -------------------------------------------------------------
        float st[4] = {0.f, 0.f, 0.f, 0.f};
        if (INT8) {
            uint32_t kw[2][8];  // [token g / g+8][step]
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int            tok = g + 8 * hh;
                const unsigned char* row = ks + tok * ROWB;
                const uint4          a   = lds128(row + (((2 * c) ^ (tok & 7)) << 4));
                const uint4          b   = lds128(row + (((2 * c + 1) ^ (tok & 7)) << 4));
                kw[hh][0] = a.x; kw[hh][1] = a.y; kw[hh][2] = a.z; kw[hh][3] = a.w;
                kw[hh][4] = b.x; kw[hh][5] = b.y; kw[hh][6] = b.z; kw[hh][7] = b.w;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint32_t af[4];
                s8x4_to_h2x2(kw[0][j] ^ kSignFlip, af[0], af[2]);
                s8x4_to_h2x2(kw[1][j] ^ kSignFlip, af[1], af[3]);
                mma_m16n8k16(st, af, qf[j][0], qf[j][1]);
            }
        }
        else {
            uint32_t kw[2][16];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int            tok = g + 8 * hh;
                const unsigned char* row = ks + tok * ROWB;
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    const int   ch = 2 * c + (m & 1) + 8 * (m >> 1);
                    const uint4 a  = lds128(row + ((ch ^ (tok & 7)) << 4));
                    kw[hh][4 * m + 0] = a.x; kw[hh][4 * m + 1] = a.y; kw[hh][4 * m + 2] = a.z; kw[hh][4 * m + 3] = a.w;
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t af[4] = {kw[0][2 * j], kw[1][2 * j], kw[0][2 * j + 1], kw[1][2 * j + 1]};
                mma_m16n8k16(st, af, qf[j][0], qf[j][1]);
            }
        }

        // ---- online softmax (heads 2c, 2c+1; token rows g, g+8) --------------------------
        float t[4];
        {
            const bool v0 = tok0 + g < s1;
            const bool v1 = tok0 + g + 8 < s1;
            t[0]          = v0 ? fmaf(st[0], alpha, beta[0]) : -INFINITY;
            t[1]          = v0 ? fmaf(st[1], alpha, beta[1]) : -INFINITY;
            t[2]          = v1 ? fmaf(st[2], alpha, beta[0]) : -INFINITY;
            t[3]          = v1 ? fmaf(st[3], alpha, beta[1]) : -INFINITY;
        }
        float mx[2] = {fmaxf(t[0], t[2]), fmaxf(t[1], t[3])};
#pragma unroll
        for (int m = 4; m <= 16; m <<= 1) {
            mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], m));
            mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], m));
        }
        float scale[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const float m_new = fmaxf(m_run[e], mx[e]);  // finite: token tok0 of the block is valid
            scale[e]          = exp2f(m_run[e] - m_new);
            m_run[e]          = m_new;
        }
        const float p0 = exp2f(t[0] - m_run[0]);
        const float p1 = exp2f(t[1] - m_run[1]);
        const float p2 = exp2f(t[2] - m_run[0]);
        const float p3 = exp2f(t[3] - m_run[1]);
        l_run[0]       = l_run[0] * scale[0] + p0 + p2;
        l_run[1]       = l_run[1] * scale[1] + p1 + p3;
        if (__any_sync(0xffffffffu, scale[0] != 1.f || scale[1] != 1.f)) {
#pragma unroll
            for (int a = 0; a < 8; ++a) {
                acc[a][0] *= scale[0];
                acc[a][1] *= scale[1];
                acc[a][2] *= scale[0];
                acc[a][3] *= scale[1];
            }
            psum[0] *= scale[0];
            psum[1] *= scale[1];
        }
        // P^T as the B operand: (tokens 2c, 2c+1 | head g) and (tokens 2c+8, 2c+9 | head g)
        const uint32_t pb0 = movmatrix_trans(pack_half2(p0, p1));
        const uint32_t pb1 = movmatrix_trans(pack_half2(p2, p3));

        // ---- O^T += V^T . P^T ------------------------------------------------------------
        const int tk[4] = {2 * c, 2 * c + 1, 2 * c + 8, 2 * c + 9};
        if (INT8) {
            {
                const uint32_t ones[4] = {0x3c003c00u, 0x3c003c00u, 0x3c003c00u, 0x3c003c00u};
                mma_m16n8k16(psum, ones, pb0, pb1);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                // word wd = g + 8q of the row (head-dim 4wd .. 4wd+3); its swizzled address is the
                // q = 0 address with bits 5..6 flipped by q
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    w[e] = lds32(vs + (v_off[e] ^ (q << 5))) ^ kSignFlip;
                }
                // interleave token pairs: [a0 b0 a1 b1], [a2 b2 a3 b3]
                const uint32_t ab_lo = prmt(w[0], w[1], 0x5140), ab_hi = prmt(w[0], w[1], 0x7362);
                const uint32_t cd_lo = prmt(w[2], w[3], 0x5140), cd_hi = prmt(w[2], w[3], 0x7362);
                uint32_t       af[4], bfm[4];
                // rows g -> d = 4wd, rows g+8 -> d = 4wd+1
                s8x4_to_h2x2(ab_lo, af[0], af[1]);
                s8x4_to_h2x2(cd_lo, af[2], af[3]);
                mma_m16n8k16(acc[2 * q], af, pb0, pb1);
                // rows g -> d = 4wd+2, rows g+8 -> d = 4wd+3
                s8x4_to_h2x2(ab_hi, bfm[0], bfm[1]);
                s8x4_to_h2x2(cd_hi, bfm[2], bfm[3]);
                mma_m16n8k16(acc[2 * q + 1], bfm, pb0, pb1);
            }
        }
        else {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                // word wd = g + 8q of the row (head-dim 2wd, 2wd+1)
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    w[e] = lds32(vs + (v_off[e] ^ (q << 5)));
                }
                const uint32_t af[4] = {prmt(w[0], w[1], 0x5410), prmt(w[0], w[1], 0x7632), prmt(w[2], w[3], 0x5410),
                                        prmt(w[2], w[3], 0x7632)};
                mma_m16n8k16(acc[q], af, pb0, pb1);
            }
        }

        if (INT8 && (blk & 7) == 7) {
            // Take the +1152 offsets out every 128 tokens of this warp: left in, the accumulators grow to
            // 1152 x (number of tokens) and the fp32 sums lose the bits that carry sum p v.
#pragma unroll
            for (int a = 0; a < 8; ++a) {
                acc[a][0] = fmaf(-kOffset, psum[0], acc[a][0]);
                acc[a][1] = fmaf(-kOffset, psum[1], acc[a][1]);
                acc[a][2] = fmaf(-kOffset, psum[0], acc[a][2]);
                acc[a][3] = fmaf(-kOffset, psum[1], acc[a][3]);
            }
            psum[0] = psum[1] = psum[2] = psum[3] = 0.f;
        }

        // every lane is done with this stage: refill it at once (NSTAGE - 1 blocks stay in flight during the math)
        __syncwarp();
        if (blk + NSTAGE < my_blocks) {
            issue_block(blk + NSTAGE, stage);
        }
        cp_async_commit();
    }
    cp_async_wait<0>();
    MMHA_TRACE(4);   // warp 0 done with its blocks
    __syncthreads();
    MMHA_TRACE(5);   // all warps done

    // ---------------------------------------------------------------- merge the warps (ring is free now)
    // part[w]: m[8] | l[8] | o[8 heads][128]   (fp32, real units)
    float* part = reinterpret_cast<float*>(ring);
    constexpr int kPartFloats = 16 + kHeadsPerCta * kD;
    {
        float l0 = l_run[0], l1 = l_run[1];
#pragma unroll
        for (int m = 4; m <= 16; m <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, m);
            l1 += __shfl_xor_sync(0xffffffffu, l1, m);
        }
        float* mine = part + warp * kPartFloats;
        if (g == 0) {
            mine[2 * c]         = m_run[0];
            mine[2 * c + 1]     = m_run[1];
            mine[8 + 2 * c]     = l0;
            mine[8 + 2 * c + 1] = l1;
        }
        const float vs0 = INT8 ? p.v_scale : 1.f;
        const float vz  = INT8 ? p.v_zp : 0.f;
        // int8: acc = sum_t p16_t (1152 + v8); v = v8 * v_scale + v_zp.  psum (= sum_t p16_t) is the
        // same in every accumulator row; columns are heads 2c, 2c+1.
        const float off0 = INT8 ? kOffset * psum[0] : 0.f;
        const float off1 = INT8 ? kOffset * psum[1] : 0.f;
#pragma unroll
        for (int a = 0; a < 8; ++a) {
            // row mapping of accumulator a: int8: d = 4(g + 8(a/2)) + 2(a&1) + {0,1}; fp16: d = 2(g + 8a) + {0,1}
            const int d = INT8 ? 4 * (g + 8 * (a >> 1)) + 2 * (a & 1) : 2 * (g + 8 * a);
            float*    o = mine + 16;
            if (2 * c < nheads) {
                o[(2 * c) * kD + d]     = fmaf(vs0, acc[a][0] - off0, vz * l0);
                o[(2 * c) * kD + d + 1] = fmaf(vs0, acc[a][2] - off0, vz * l0);
            }
            if (2 * c + 1 < nheads) {
                o[(2 * c + 1) * kD + d]     = fmaf(vs0, acc[a][1] - off1, vz * l1);
                o[(2 * c + 1) * kD + d + 1] = fmaf(vs0, acc[a][3] - off1, vz * l1);
            }
        }
    }
    __syncthreads();

    // thread = head-dim index (a CTA of fewer than 128 threads takes several); loop over heads
    constexpr int kRec = 2 + kD;  // split record: m | l | o[128]
    for (int d = tid; d < kD; d += kThreads) {
#pragma unroll
        for (int h = 0; h < kHeadsPerCta; ++h) {
            if (h >= nheads) continue;
            float mm = last_split ? snew_s[h] : -INFINITY;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, part[w * kPartFloats + h]);
            float ll = 0.f, oo = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float f = exp2f(part[w * kPartFloats + h] - mm);  // exp2(-inf) = 0 for idle warps
                ll += part[w * kPartFloats + 8 + h] * f;
                oo += part[w * kPartFloats + 16 + h * kD + d] * f;
            }
            if (last_split) {
                const float f = exp2f(snew_s[h] - mm);
                ll += f;
                // the reference multiplies the fp16-rounded probability with the un-quantised v
                oo += f * __half2float(vnew_s[d]);
            }
            if (n_split == 1) {
                // template.cuh:1662: 1 / (sum + 1e-6)
                p.out[((size_t)bi * p.H + head0 + h) * kD + d] = __float2half_rn(oo / (ll + 1.e-6f));
            }
            else {
                float* rec = p.ws + (((size_t)bi * p.H + head0 + h) * p.max_splits + split) * kRec;
                if (d == 0) {
                    __stcg(rec, mm);
                    __stcg(rec + 1, ll);
                }
                __stcg(rec + 2 + d, oo);
            }
        }
    }
    // The new token goes into the cache (one CTA per sequence and KV head does it).  Last, off the path to the first
    // block: nothing in this launch reads the slot, and the copies in shared memory are still intact.
    if (last_split && hb == 0) {
        const size_t   slot = (size_t)(tlength % p.S_max) * ROWB;
        unsigned char* kd   = const_cast<unsigned char*>(kc) + slot;
        unsigned char* vd   = const_cast<unsigned char*>(vc) + slot;
        if (INT8) {
            for (int t2 = tid; t2 < 64; t2 += kThreads) {
                const bool          is_v = t2 >= 32;
                const int           d    = (t2 & 31) * 4;
                const __half*       src  = is_v ? vnew_s : knew_s;
                const float         sc   = is_v ? p.v_scale : p.k_scale;
                const float         zp   = is_v ? p.v_zp : p.k_zp;
                uint32_t            w    = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    // template.cuh:976-981: round(clamp((x - zp) / scale)), round = half away from zero
                    float v = __fdiv_rn(__half2float(src[d + i]) - zp, sc);
                    v       = fmaxf(-128.f, fminf(127.f, v));
                    w |= ((uint32_t)(int)roundf(v) & 0xffu) << (8 * i);
                }
                *reinterpret_cast<uint32_t*>((is_v ? vd : kd) + d) = w;
            }
        }
        else {
            if (tid < kD / 8) {
                const int d = tid * 8;  // 16 bytes of K and of V per thread
                *reinterpret_cast<uint4*>(kd + d * 2) = *reinterpret_cast<const uint4*>(knew_s + d);
                *reinterpret_cast<uint4*>(vd + d * 2) = *reinterpret_cast<const uint4*>(vnew_s + d);
            }
        }
    }
#ifdef TM_B200_GEMM_TRACE
    MMHA_TRACE(6);
    if (trace_on && tid == 0) {
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        g_mmha_trace[trace_id][7] = ((unsigned long long)smid << 32) | (unsigned)tlength;
    }
    if (tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) atomicAdd(&g_mmha_launch, 1);
#endif
    if (n_split == 1) {
        return;
    }

    // ---------------------------------------------------------------- merge the splits
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int*      counter = p.counters + (size_t)bi * gridDim.y + blockIdx.y;
        const int ticket  = atomicAdd(counter, 1);
        const int is_last = ticket == n_split - 1;
        if (is_last) {
            *counter = 0;  // self-reset for the next launch
        }
        flag_s[0] = is_last;
    }
    __syncthreads();
    if (!flag_s[0]) {
        return;
    }
    __threadfence();
    for (int d = tid; d < kD; d += kThreads) {
        for (int h = 0; h < nheads; ++h) {
            const float* rec0 = p.ws + (((size_t)bi * p.H + head0 + h) * p.max_splits) * kRec;
            float        mm   = -INFINITY;
            for (int s = 0; s < n_split; ++s) mm = fmaxf(mm, __ldcg(rec0 + (size_t)s * kRec));
            float ll = 0.f, oo = 0.f;
            for (int s = 0; s < n_split; ++s) {
                const float* rec = rec0 + (size_t)s * kRec;
                const float  f   = exp2f(__ldcg(rec) - mm);
                ll += __ldcg(rec + 1) * f;
                oo += __ldcg(rec + 2 + d) * f;
            }
            p.out[((size_t)bi * p.H + head0 + h) * kD + d] = __float2half_rn(oo / (ll + 1.e-6f));
        }
    }
}

template<bool INT8, int W>
constexpr size_t mmha_smem_bytes()
{
    constexpr int ROWB   = INT8 ? kD : 2 * kD;
    constexpr int NSTAGE = 3;
    return (size_t)W * NSTAGE * 2 * kBlockTok * ROWB + (kHeadsPerCta + 2) * kD * 2 + 2 * kHeadsPerCta * 4 + 16;
}

template<bool INT8, int W>
cudaError_t mmha_prepare_one()
{
    return cudaFuncSetAttribute(mmha_decode_kernel<INT8, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mmha_smem_bytes<INT8, W>());
}

template<bool INT8, int W>
cudaError_t mmha_launch_one(dim3 grid, const MmhaParams& p, cudaStream_t st, bool pdl)
{
    return launch_kernel(mmha_decode_kernel<INT8, W>, grid, dim3(W * 32), mmha_smem_bytes<INT8, W>(), st, pdl, p);
}

}  // namespace

cudaError_t mmha_prepare()
{
    cudaError_t e = mmha_prepare_one<true, 4>();
    if (e == cudaSuccess) e = mmha_prepare_one<true, 2>();
    if (e == cudaSuccess) e = mmha_prepare_one<true, 1>();
    if (e == cudaSuccess) e = mmha_prepare_one<false, 4>();
    if (e == cudaSuccess) e = mmha_prepare_one<false, 2>();
    if (e == cudaSuccess) e = mmha_prepare_one<false, 1>();
    return e;
}

MmhaPlan mmha_plan(int B, int H, int Hkv, int max_len, int sm_count, int want_chunk, int want_warps)
{
    MmhaPlan  pl{};
    const int rep = H / Hkv;
    pl.head_blocks = (rep + kHeadsPerCta - 1) / kHeadsPerCta;
    const long long items = (long long)B * Hkv * pl.head_blocks;
    int             chunk = want_chunk;
    if (chunk <= 0) {
        // Splitting a sequence costs a partial record per split, a ticket and a merge, and every CTA
        // pays a fixed start-up (q load, RoPE, pipeline fill) worth a few hundred tokens: measured on
        // B200, one CTA per (sequence, KV head) beats any split as soon as there is about one CTA per
        // two SMs.  So: no split up to 2048 tokens when there are that many items; 2048-token splits
        // beyond (they even out the tail of long sequences); with fewer items, just enough splits of at
        // least 256 tokens to put two CTAs on every SM.
        if (items * 2 >= sm_count) {
            chunk = max_len < 2048 ? max_len : 2048;
        }
        else {
            long long splits = (2ll * sm_count + items - 1) / items;
            long long most   = (max_len + 255) / 256;
            if (splits > most) splits = most;
            if (splits < 1) splits = 1;
            chunk = (int)((max_len + splits - 1) / splits);
            if (chunk < 256) chunk = 256;
        }
        if (chunk < 64) chunk = 64;
    }
    chunk         = (chunk + 63) / 64 * 64;
    pl.chunk      = chunk;
    pl.max_splits = max_len > 0 ? (max_len + chunk - 1) / chunk : 1;
    if (pl.max_splits < 1) pl.max_splits = 1;
    pl.ws_floats    = (size_t)B * H * pl.max_splits * (2 + kD);
    pl.counter_ints = (size_t)B * Hkv * pl.head_blocks;
    // Warps per CTA (16 warps are resident per SM in every variant).
    const long long ctas = items * pl.max_splits;
    (void)ctas;  // measured on B200: four warps per CTA win at every batch and length tried; 2 and 1 stay available as options
    pl.warps = 4;
    if (want_warps == 1 || want_warps == 2 || want_warps == 4) pl.warps = want_warps;
    return pl;
}

cudaError_t mmha_launch(const MmhaPlan& pl, MmhaParams p, bool int8, cudaStream_t st, bool pdl)
{
    p.chunk      = pl.chunk;
    p.max_splits = pl.max_splits;
    dim3 grid(pl.max_splits, p.Hkv * pl.head_blocks, p.B);
    if (int8) {
        switch (pl.warps) {
            case 1: return mmha_launch_one<true, 1>(grid, p, st, pdl);
            case 2: return mmha_launch_one<true, 2>(grid, p, st, pdl);
            default: return mmha_launch_one<true, 4>(grid, p, st, pdl);
        }
    }
    switch (pl.warps) {
        case 1: return mmha_launch_one<false, 1>(grid, p, st, pdl);
        case 2: return mmha_launch_one<false, 2>(grid, p, st, pdl);
        default: return mmha_launch_one<false, 4>(grid, p, st, pdl);
    }
}

}  // namespace tmb
