/* Drop-in for src/turbomind/kernels/gemm_s_f16/format.h of lmdeploy v0.0.9 (:11-33): the converters that
 * turn AWQ tensors into the packed layout the W4A16 GEMM reads.  Same names, argument order and default
 * stream; header-only, forwards to the C ABI in tm_b200.h.  The callers that then work unchanged:
 *   src/turbomind/python/bind.cpp:414-465           (the `_turbomind` helpers deploy.py uses)
 *   src/turbomind/models/llama/LlamaDecoderLayerWeight.cc (nothing at load time: files are already converted)
 * Put `-I <this repo>/include/compat -I <this repo>/include` ahead of the TurboMind source root. */
#pragma once

#include "tm_b200.h"

#include <cstddef>
#include <cstdint>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

namespace turbomind {

namespace b200_compat {
inline void check(int rc, const char* what)
{
    if (rc != TM_OK) throw std::runtime_error(std::string("[TM][b200] ") + what + ": " + tm_status_string(rc));
}
}  // namespace b200_compat

/* format.cu:61-67.  Nothing in the reference calls it (the [k/8, m] layout is not the one the GEMM
 * reads), and this library has no kernel for it: asking for it is an error, not a silent no-op. */
inline void reformat_s4_k8_m(uint32_t* dst, const uint32_t* src, int m, int k, cudaStream_t st = {})
{
    (void)dst, (void)src, (void)m, (void)k, (void)st;
    throw std::runtime_error("[TM][b200] reformat_s4_k8_m: the [k/8, m] layout is not provided (no caller in TurboMind)");
}

/* format.cu:69-75 */
inline void reformat_s4_k_m8(uint32_t* dst, const uint32_t* src, int m, int k, cudaStream_t st = {})
{
    b200_compat::check(tm_reformat_s4_k_m8(dst, src, m, k, (void*)st), "reformat_s4_k_m8");
}

/* format.cu:97-113: A_src int32 [k, m/8] AWQ order, scales half [k/g, m], qzeros int32 [k/g, m/8];
 * A_dst in the GEMM's layout, Q_dst half2 {zero (offset by 64), scale}; workspace: k/g * m halves. */
inline void convert_s4_k_m8(uint32_t*       A_dst,
                            half2*          Q_dst,
                            half*           workspace,
                            const uint32_t* A_src,
                            const half*     scales,
                            const uint32_t* qzeros,
                            int             m,
                            int             k,
                            int             group_size,
                            cudaStream_t    st = {})
{
    b200_compat::check(tm_convert_s4_k_m8(A_dst, Q_dst, workspace, A_src, scales, qzeros, m, k, group_size, (void*)st),
                       "convert_s4_k_m8");
}

/* format.cu:115-122 */
inline void transpose_qk_s4_k_m8_hf(uint32_t* dst, const uint32_t* src, int m, int k, int size_per_head, cudaStream_t st = {})
{
    b200_compat::check(tm_transpose_qk_s4_k_m8_hf(dst, src, m, k, size_per_head, (void*)st), "transpose_qk_s4_k_m8_hf");
}

/* format.cu:124-131 */
inline void fuse_w1_w3_s4_k_m8(uint32_t* dst, const uint32_t* src, int m, int k, cudaStream_t st = {})
{
    b200_compat::check(tm_fuse_w1_w3_s4_k_m8(dst, src, m, k, (void*)st), "fuse_w1_w3_s4_k_m8");
}

/* format.cu:139-142: eight halves per packed word */
inline void dequantize_s4(uint4* dst, const uint32_t* src, size_t count, cudaStream_t st = {})
{
    b200_compat::check(tm_dequantize_s4(dst, src, count, (void*)st), "dequantize_s4");
}

}  // namespace turbomind
