/* Drop-in for src/turbomind/kernels/gemm_s_f16/gemm_s4_f16.h of lmdeploy v0.0.9 (class at :15-57).
 *
 * Put `-I <this repo>/include/compat -I <this repo>/include` AHEAD of the TurboMind source root on the
 * compiler command line and link libtm_b200.so: the include line
 *     #include "src/turbomind/kernels/gemm_s_f16/gemm_s4_f16.h"
 * of src/turbomind/models/llama/LlamaLinear.h:5 then finds this file, and LlamaLinear<half>::forwardInt4
 * (LlamaLinear.h:62-81) compiles and runs unchanged on the sm_100a kernels of this library.  The reference's
 * gemm_s4_f16.cu / gemm_template.h are then not compiled at all.
 *
 * Same class name, enum and member signatures; header-only, forwards to the C ABI in tm_b200.h.
 * Differences, all on the error path: the reference aborts through its kernel-selection asserts, this
 * shim reports through std::runtime_error (which FT's callers already let propagate). */
#pragma once

#include "tm_b200.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>
#include <vector>

namespace turbomind {

struct Metric;  // src/turbomind/kernels/gemm_s_f16/metric.h; only named by Measure below

class GemmS4F16 {
public:
    GemmS4F16()  = default;
    ~GemmS4F16() = default;

    enum Type
    {
        kGemm,
        kFusedSiluFfn
    };

    /* The reference times every tile configuration here and remembers the best (gemm_s4_f16.cu:237-293).
     * This library plans each launch from (m, n, k) alone, so there is nothing to measure: the call runs
     * the GEMM once, which leaves C as the reference's last measured launch does, and adds no metrics. */
    void Measure(half*                C,
                 const unsigned int*  A,
                 const half*          B,
                 const half2*         Q,
                 int                  m,
                 int                  n,
                 int                  k,
                 int                  group_size,
                 Type                 type,
                 std::vector<Metric>& metrics,
                 cudaStream_t         st)
    {
        (void)metrics;
        Run(C, A, B, Q, m, n, k, group_size, type, -1, st);
    }

    /* C[n, m] = B[n, k] . dequant(A, Q)^T; m = output features, n = tokens, as gemm_s4_f16.cu:208-234.
     * algo_id is accepted and ignored (there is one plan per shape). */
    void Run(half*               C,
             const unsigned int* A,
             const half*         B,
             const half2*        Q,
             int                 m,
             int                 n,
             int                 k,
             int                 group_size,
             Type                type,
             int                 algo_id,
             cudaStream_t        st)
    {
        (void)algo_id;
        tm_handle* h = tm_handle_of_current_device();
        if (!h) throw std::runtime_error("[TM][b200] no handle for the current CUDA device");
        const int rc = tm_gemm_s4_f16(h, C, A, B, Q, m, n, k, group_size, type == kFusedSiluFfn ? 1 : 0, nullptr, 0, (void*)st);
        if (rc != TM_OK) throw std::runtime_error(std::string("[TM][b200] tm_gemm_s4_f16: ") + tm_status_string(rc));
    }
};

}  // namespace turbomind
