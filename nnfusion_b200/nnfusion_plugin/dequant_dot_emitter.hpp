// cuda::DequantDot -- kernel emitter that serves the DequantDot operator with one call into libnnf_b200.so.
// Goes to src/nnfusion/core/kernels/cuda_gpu/kernels/; emitter contract: src/nnfusion/core/kernels/kernel_emitter.hpp:18-160,
// CudaLibEmitter: src/nnfusion/core/kernels/cuda_gpu/cuda_emitter.hpp:190-199 (same family as cuda::Dot, kernels/dot.cpp).
#pragma once
#include "../cuda_emitter.hpp"
#include "../cuda_langunit.hpp"
#include "nnf_b200_langunit.hpp"

namespace nnfusion
{
    namespace kernels
    {
        namespace cuda
        {
            class DequantDot : public CudaLibEmitter
            {
            public:
                DequantDot(shared_ptr<KernelContext> ctx);
                LanguageUnit_p emit_function_body() override;
                LanguageUnit_p emit_dependency() override;
                LanguageUnit_p emit_function_signature() override;

            private:
                shared_ptr<op::GenericOp> generic_op;
                size_t M, N, K;
                int w_bits, group_size;
                std::string prologue, epilogue;
                float rms_eps;
                size_t workspace_bytes;
                std::shared_ptr<nnfusion::descriptor::Tensor> workspace; // planned into the static pool
            };
        } // namespace cuda
    }     // namespace kernels
} // namespace nnfusion
