// Thin C entry points around the reference's own vendored MLAS, compiled in
// place from the reference checkout (see the Makefile beside this file).
//
// TEST INFRASTRUCTURE ONLY: the resulting library validates the C restatement
// in oracle.c and serves as the timed CPU baseline.  The shipped CUDA library
// never links or loads it.
//
// What runs here is what the reference's CPU code generation emits for the
// dequantised linear graph (pipeline src/nnfusion/engine/device/cpu.cpp:40-87):
//   Convert   cpu_reference_convert            core/kernels/cpu/reference/kernels.cpp:711-719
//   Subtract  _mm256_sub_ps over 8-lane blocks core/kernels/cpu/simd/elementwise.hpp:60-127
//   Multiply  _mm256_mul_ps                    (same file; op table cpu_kernelops.hpp:183-190,344-351)
//   Dot       MlasGemm(NoTrans, Trans, ...)    core/kernels/cpu/mlas/dot.cpp:89-100
// The three elementwise loops are restated here (they are a few lines each in
// the reference's generated code); the GEMM is the reference's MLAS itself,
// called with ThreadPool = nullptr so that it uses its OpenMP loop
// (thirdparty/mlas/lib/threading.cpp:36-62).
#include <immintrin.h>
#include <omp.h>
#include <cstddef>
#include <cstdint>
#include <cstdlib>

#include "mlas.h"

extern "C" {

__attribute__((visibility("default"))) void ref_mlas_sgemm(int trans_a, int trans_b, size_t M,
                                                           size_t N, size_t K, float alpha,
                                                           const float* A, size_t lda,
                                                           const float* B, size_t ldb, float beta,
                                                           float* C, size_t ldc)
{
    MlasGemm(trans_a ? CblasTrans : CblasNoTrans, trans_b ? CblasTrans : CblasNoTrans, M, N, K,
             alpha, A, lda, B, ldb, beta, C, ldc, nullptr);
}

__attribute__((visibility("default"))) int ref_num_threads(void)
{
    return omp_get_max_threads();
}

// Dequantise [N,K] uint8 weights (one byte per element; uint4 already unpacked)
// with per-(row, group) zero-point and scale into fp32, with the reference's
// kernel sequence: Convert, then Subtract, then Multiply, each writing a full
// fp32 [N,K] tensor exactly like the separately emitted kernels do.
__attribute__((visibility("default"))) void ref_dequant_graph(const uint8_t* q, const float* scale,
                                                              const uint8_t* zp, size_t N, size_t K,
                                                              size_t group, float* wf, float* wdq)
{
    size_t G = K / group;
#pragma omp parallel for
    for (size_t n = 0; n < N; n++)
        for (size_t k = 0; k < K; k++)
            wf[n * K + k] = static_cast<float>(q[n * K + k]);
#pragma omp parallel for
    for (size_t n = 0; n < N; n++)
        for (size_t g = 0; g < G; g++)
        {
            __m256 z = _mm256_set1_ps(static_cast<float>(zp[n * G + g]));
            for (size_t j = 0; j < group; j += 8)
            {
                float* p = wf + n * K + g * group + j;
                _mm256_storeu_ps(p, _mm256_sub_ps(_mm256_loadu_ps(p), z));
            }
        }
#pragma omp parallel for
    for (size_t n = 0; n < N; n++)
        for (size_t g = 0; g < G; g++)
        {
            __m256 s = _mm256_set1_ps(scale[n * G + g]);
            for (size_t j = 0; j < group; j += 8)
            {
                const float* p = wf + n * K + g * group + j;
                _mm256_storeu_ps(wdq + n * K + g * group + j, _mm256_mul_ps(_mm256_loadu_ps(p), s));
            }
        }
}

// One call of the whole CPU graph: dequantise, then Y = X . Wdq^T through MLAS.
// `wf` and `wdq` are caller-provided fp32 [N,K] scratch tensors (the generated
// runtime plans them in its static memory pool).  group must be a multiple of 8.
__attribute__((visibility("default"))) void ref_linear_graph(const float* x, size_t M, size_t N,
                                                             size_t K, size_t group,
                                                             const uint8_t* q, const float* scale,
                                                             const uint8_t* zp, float* wf,
                                                             float* wdq, float* y)
{
    ref_dequant_graph(q, scale, zp, N, K, group, wf, wdq);
    MlasGemm(CblasNoTrans, CblasTrans, M, N, K, 1.0f, x, K, wdq, K, 0.0f, y, N, nullptr);
}
}
