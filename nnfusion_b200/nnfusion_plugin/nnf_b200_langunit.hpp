// Declarations of the language units the B200 emitters require in the generated project.
// Goes next to src/nnfusion/core/kernels/cuda_gpu/cuda_langunit.hpp (which declares header::cuda,
// macro::CUDA_SAFE_CALL, declaration::global_cublas_handle ... with the same macro, :7-59) and
// src/nnfusion/engine/pass/codegen/codegen_langunit.hpp (cmake::superscaler_cuda ..., :7-30); the definitions are in
// codegen_units.cpp.
#pragma once
#include "nnfusion/core/kernels/common_langunit.hpp"

namespace nnfusion
{
    namespace kernels
    {
        namespace header
        {
            LU_DECLARE(nnf_b200);
        }
        namespace macro
        {
            LU_DECLARE(NNF_B200_SAFE_CALL);
        }
        namespace declaration
        {
            LU_DECLARE(nnf_b200_ctx);
        }
    } // namespace kernels
    namespace codegen
    {
        namespace cmake
        {
            LU_DECLARE(nnf_b200);
        }
    } // namespace codegen
} // namespace nnfusion
