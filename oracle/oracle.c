/*
 * CPU oracle for the dequantize-fused low-bit linear path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic the
 * reference compiler's CPU code generation executes for the graph
 *
 *     Y = Dot(X, Multiply(Subtract(Convert(W), Broadcast(zp)), Broadcast(scale)), transB)
 *
 * so that the CUDA kernels can be checked against it.  Nothing in the shipped
 * library links, imports or calls it; only the test-suite, the smoke check and
 * the CPU-baseline leg of the benchmark do.
 *
 * Every function names the reference source it follows (paths are relative to
 * the reference project root).  Where the reference has no encoding (packed
 * uint4, group-wise scales, RMSNorm, SiLU*mul) the function says so and the
 * definition is this project's own: for those, parity is unpinned by the
 * reference and rests on this file alone.
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC oracle.c -o liboracle.so -lm
 * (-ffp-contract=off keeps a*b+c as two rounded operations wherever the
 * reference performs two separate elementwise kernels.)
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* Element-type conversion                                                    */
/* ------------------------------------------------------------------------- */

/* op::Convert on the CPU is `out[i] = static_cast<TO>(arg[i])`
 * (src/nnfusion/core/kernels/cpu/reference/kernels.cpp:711-719, emitter
 * ConvertRef :2515-2555).  uint8 -> float is exact. */
ORC_API void orc_convert_u8_f32(const uint8_t* arg, float* out, size_t count)
{
    for (size_t i = 0; i < count; i++)
        out[i] = (float)arg[i];
}

/* half -> float Convert: same static_cast, exact.  The half is carried as its
 * IEEE-754 binary16 bit pattern. */
ORC_API void orc_convert_f16_f32(const uint16_t* arg, float* out, size_t count)
{
    for (size_t i = 0; i < count; i++)
    {
        _Float16 h;
        memcpy(&h, &arg[i], 2);
        out[i] = (float)h;
    }
}

/* float -> half Convert: static_cast, round-to-nearest-even. */
ORC_API void orc_convert_f32_f16(const float* arg, uint16_t* out, size_t count)
{
    for (size_t i = 0; i < count; i++)
    {
        _Float16 h = (_Float16)arg[i];
        memcpy(&out[i], &h, 2);
    }
}

/* ------------------------------------------------------------------------- */
/* Elementwise arithmetic                                                     */
/* ------------------------------------------------------------------------- */

/* Subtract / Multiply / Add on the CPU are 8-lane AVX kernels
 * (_mm256_sub_ps / _mm256_mul_ps / _mm256_add_ps:
 * src/nnfusion/core/kernels/cpu/simd/elementwise.hpp:60-127, op table
 * src/nnfusion/core/kernels/cpu/cpu_kernelops.hpp:183-190,344-351).  They are
 * IEEE fp32 lane-wise operations, so scalar loops give identical bits. */
ORC_API void orc_subtract_f32(const float* a, const float* b, float* out, size_t n)
{
    for (size_t i = 0; i < n; i++)
        out[i] = a[i] - b[i];
}

ORC_API void orc_multiply_f32(const float* a, const float* b, float* out, size_t n)
{
    for (size_t i = 0; i < n; i++)
        out[i] = a[i] * b[i];
}

ORC_API void orc_add_f32(const float* a, const float* b, float* out, size_t n)
{
    for (size_t i = 0; i < n; i++)
        out[i] = a[i] + b[i];
}

/* Sigmoid: `1 / (1 + expf(-x0))`
 * (src/nnfusion/core/kernels/cuda_gpu/cuda_common_ops.hpp:96; the CPU side only
 * has an Eigen kernel with the same formula). */
ORC_API void orc_sigmoid_f32(const float* a, float* out, size_t n)
{
    for (size_t i = 0; i < n; i++)
        out[i] = 1.0f / (1.0f + expf(-a[i]));
}

/* op::Broadcast classified as "inner" broadcast: every input element is
 * repeated `inner` times, out[i * inner + j] = in[i]
 * (src/nnfusion/core/operators/op_define/broadcast.cpp:71-117; the fused CUDA
 * kernel reads it as in[tid / inner],
 * src/nnfusion/core/kernels/cuda_gpu/kernels/elementwise_fused.cpp:88-107). */
ORC_API void orc_broadcast_inner_f32(const float* in, float* out, size_t outer, size_t inner)
{
    for (size_t i = 0; i < outer; i++)
        for (size_t j = 0; j < inner; j++)
            out[i * inner + j] = in[i];
}

/* ------------------------------------------------------------------------- */
/* Packed uint4 (this project's definition; no reference encoding exists:     */
/* src/nnfusion/common/type/element_type.hpp:41-55 stops at u8)               */
/* ------------------------------------------------------------------------- */

/* byte i holds element 2i in bits 0-3 and element 2i+1 in bits 4-7. */
ORC_API void orc_unpack_u4(const uint8_t* packed, uint8_t* out, size_t n_elems)
{
    for (size_t i = 0; i < n_elems; i++)
    {
        uint8_t b = packed[i >> 1];
        out[i] = (i & 1) ? (uint8_t)(b >> 4) : (uint8_t)(b & 0x0F);
    }
}

ORC_API void orc_pack_u4(const uint8_t* in, uint8_t* packed, size_t n_elems)
{
    for (size_t i = 0; i < (n_elems + 1) / 2; i++)
    {
        uint8_t lo = in[2 * i] & 0x0F;
        uint8_t hi = (2 * i + 1 < n_elems) ? (in[2 * i + 1] & 0x0F) : 0;
        packed[i] = (uint8_t)(lo | (hi << 4));
    }
}

/* ------------------------------------------------------------------------- */
/* Dot                                                                        */
/* ------------------------------------------------------------------------- */

/* Naive Dot, one sequential fp32 sum per output element in increasing k:
 * `sum += arg0[...] * arg1[...]`
 * (src/nnfusion/core/kernels/cpu/reference/kernels.cpp:1532-1617).  A is
 * [M,K] row-major; B is [K,N] (trans_b = 0) or [N,K] (trans_b = 1). */
ORC_API void orc_dot_naive(const float* a, const float* b, float* c, size_t M, size_t N, size_t K,
                           int trans_b)
{
#pragma omp parallel for
    for (size_t m = 0; m < M; m++)
        for (size_t n = 0; n < N; n++)
        {
            float sum = 0;
            for (size_t k = 0; k < K; k++)
            {
                float bv = trans_b ? b[n * K + k] : b[k * N + n];
                sum += a[m * K + k] * bv;
            }
            c[m * N + n] = sum;
        }
}

/* SGEMM restated after the structure of the vendored MLAS routine the CPU code
 * generation calls, MlasGemm(CblasNoTrans, CblasTrans, M, N, K, 1.0, A, K, B, K,
 * 0.0, C, N) (call site src/nnfusion/core/kernels/cpu/mlas/dot.cpp:89-100;
 * algorithm thirdparty/mlas/lib/sgemm.cpp:766-1000): K is walked in panels of
 * 128 (MLAS_SGEMM_STRIDEK), each panel's products are accumulated with fused
 * multiply-adds starting from zero, and the panel sum is then added to C (the
 * first panel stores, later panels accumulate).  The exact lane order inside
 * the assembly micro-kernel is not reproduced; the compiled MLAS itself
 * (oracle/_ref) is used to bound the difference. */
ORC_API void orc_sgemm_nt(const float* a, const float* b, float* c, size_t M, size_t N, size_t K)
{
    const size_t stride_k = 128;
#pragma omp parallel for collapse(2)
    for (size_t m = 0; m < M; m++)
        for (size_t n = 0; n < N; n++)
        {
            float total = 0;
            for (size_t k0 = 0; k0 < K; k0 += stride_k)
            {
                size_t k1 = k0 + stride_k < K ? k0 + stride_k : K;
                float acc = 0;
                for (size_t k = k0; k < k1; k++)
                    acc = fmaf(a[m * K + k], b[n * K + k], acc);
                total = (k0 == 0) ? acc : total + acc;
            }
            c[m * N + n] = total;
        }
}

/* ------------------------------------------------------------------------- */
/* The dequantisation sub-graph                                               */
/* ------------------------------------------------------------------------- */

/* W (one uint8 per element, [N,K]) -> fp32 [N,K], as the chain the ONNX
 * importer produces for Cast -> Sub(zero-point) -> Mul(scale) with the
 * quantisation parameters declared [N, K/group, 1]:
 *   Reshape([N, K/group, group]) -> Convert(f32)
 *   zp  -> Convert(f32) -> Broadcast(inner = group)
 *   s   ->                 Broadcast(inner = group)
 *   Subtract, Multiply, Reshape([N,K])
 * (importer: src/nnfusion/frontend/onnx_import/op/cast.hpp:35-51,
 * op/binaryop.hpp:89-107; broadcasting plan
 * src/nnfusion/core/graph/util/autobroadcast.cpp:83-151).  Order of operations
 * is (float(q) - float(zp)) * scale with each step rounded to fp32.
 * group == K is the per-output-channel case of the first benchmark graph. */
ORC_API void orc_dequant(const uint8_t* q, const float* scale, const uint8_t* zp, size_t N, size_t K,
                         size_t group, float* wdq)
{
    size_t G = K / group;
#pragma omp parallel for
    for (size_t n = 0; n < N; n++)
        for (size_t g = 0; g < G; g++)
        {
            float zf = (float)zp[n * G + g];
            float sf = scale[n * G + g];
            const uint8_t* qp = q + n * K + g * group;
            float* wp = wdq + n * K + g * group;
            for (size_t j = 0; j < group; j++)
            {
                float t = (float)qp[j] - zf;
                wp[j] = t * sf;
            }
        }
}

/* ------------------------------------------------------------------------- */
/* Normalisation / activation (no RMSNorm or SiLU operator exists in the      */
/* reference; these are the formulas the primitive-op graph computes in fp32) */
/* ------------------------------------------------------------------------- */

/* y = x * rsqrt(mean(x^2) + eps) * gain, row-wise.  In the reference's op set:
 * Multiply(x,x) -> Sum (src/nnfusion/core/kernels/cuda_gpu/kernels/reduce.hpp)
 * -> Divide(K) -> Add(eps) -> Rsqrt -> Multiply -> Multiply(gain). */
ORC_API void orc_rmsnorm_f32(const float* x, const float* gain, float eps, float* out, size_t M,
                             size_t K)
{
    for (size_t m = 0; m < M; m++)
    {
        float ss = 0;
        for (size_t k = 0; k < K; k++)
            ss += x[m * K + k] * x[m * K + k];
        float r = 1.0f / sqrtf(ss / (float)K + eps);
        for (size_t k = 0; k < K; k++)
            out[m * K + k] = x[m * K + k] * r * gain[k];
    }
}

/* SiLU(g) * u = g * sigmoid(g) * u with the reference's sigmoid formula. */
ORC_API void orc_silu_mul_f32(const float* g, const float* u, float* out, size_t n)
{
    for (size_t i = 0; i < n; i++)
    {
        float s = 1.0f / (1.0f + expf(-g[i]));
        out[i] = g[i] * s * u[i];
    }
}

/* ------------------------------------------------------------------------- */
/* Whole linear: the graph of one dequantised linear layer                    */
/* ------------------------------------------------------------------------- */

/* y[M,N] = epilogue( prologue(x)[M,K] . dequant(q)[N,K]^T )
 *   x, y, bias are fp32 here (fp16 tensors are converted by the caller with the
 *   Convert functions above: fp16 inputs are upcast on entry, the result is
 *   rounded to fp16 once at the end).
 *   gain != NULL  -> RMSNorm prologue.
 *   bias != NULL  -> Add(bias broadcast over rows) epilogue (how Gemm's C term
 *                    is imported: src/nnfusion/frontend/onnx_import/op/gemm.cpp:41-96).
 *   q2 != NULL    -> second weight set; result is SiLU(x.W1^T) * (x.W2^T).
 * use_naive_dot selects the sequential reference Dot instead of the blocked
 * SGEMM.  Returns 0, or -1 when a scratch allocation fails. */
ORC_API int orc_linear(const float* x, size_t M, size_t N, size_t K, size_t group, const uint8_t* q,
                       const float* scale, const uint8_t* zp, const uint8_t* q2, const float* scale2,
                       const uint8_t* zp2, const float* gain, float eps, const float* bias,
                       int use_naive_dot, float* y)
{
    float* wdq = (float*)malloc(sizeof(float) * N * K);
    float* xn = NULL;
    float* y2 = NULL;
    if (!wdq)
        return -1;
    const float* xin = x;
    if (gain)
    {
        xn = (float*)malloc(sizeof(float) * M * K);
        if (!xn)
        {
            free(wdq);
            return -1;
        }
        orc_rmsnorm_f32(x, gain, eps, xn, M, K);
        xin = xn;
    }
    orc_dequant(q, scale, zp, N, K, group, wdq);
    if (use_naive_dot)
        orc_dot_naive(xin, wdq, y, M, N, K, 1);
    else
        orc_sgemm_nt(xin, wdq, y, M, N, K);
    if (q2)
    {
        y2 = (float*)malloc(sizeof(float) * M * N);
        if (!y2)
        {
            free(wdq);
            free(xn);
            return -1;
        }
        orc_dequant(q2, scale2, zp2, N, K, group, wdq);
        if (use_naive_dot)
            orc_dot_naive(xin, wdq, y2, M, N, K, 1);
        else
            orc_sgemm_nt(xin, wdq, y2, M, N, K);
        orc_silu_mul_f32(y, y2, y, M * N);
    }
    if (bias)
        for (size_t m = 0; m < M; m++)
            for (size_t n = 0; n < N; n++)
                y[m * N + n] = y[m * N + n] + bias[n];
    free(wdq);
    free(xn);
    free(y2);
    return 0;
}
