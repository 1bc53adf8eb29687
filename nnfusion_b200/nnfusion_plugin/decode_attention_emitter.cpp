// Kernel emitter of the DecodeAttention node: a host-side library call, like cuda::BatchMatMul's cuBLAS call
// (src/nnfusion/core/kernels/cuda_gpu/kernels/batch_matmul.cpp:49-144), to nnf_b200_decode_attention.
// Goes to src/nnfusion/core/kernels/cuda_gpu/kernels/decode_attention.cpp.
#include "../cuda_emitter.hpp"
#include "../cuda_langunit.hpp"
#include "nnf_b200_langunit.hpp"
#include "nnf_b200.h" // host functions only: workspace sizing at code-generation time
#include "nnfusion/core/operators/generic_op/generic_op.hpp"

namespace nnfusion
{
    namespace kernels
    {
        namespace cuda
        {
            class DecodeAttention : public CudaLibEmitter
            {
                shared_ptr<nnfusion::op::GenericOp> generic_op;
                nnf_b200_attn_desc desc;
                size_t workspace_bytes = 0;

            public:
                DecodeAttention(shared_ptr<KernelContext> ctx)
                    : CudaLibEmitter(ctx)
                    , generic_op(static_pointer_cast<nnfusion::op::GenericOp>(ctx->gnode->get_op_ptr()))
                {
                    auto& cfg = generic_op->localOpConfig.getRoot();
                    desc = {};
                    desc.heads = cfg["heads"], desc.kv_heads = cfg["kv_heads"], desc.head_dim = cfg["head_dim"];
                    desc.capacity = (int32_t)ctx->inputs[3]->get_shape()[1];
                    desc.position = cfg["position"];
                    desc.rotary = (bool)cfg["rotary"] ? 1 : 0;
                    desc.rotary_base = cfg["rotary_base"], desc.softmax_scale = cfg["softmax_scale"];
                    desc.dtype = NNF_B200_F16;
                    // sized for the longest sequence the caches hold, planned into the pool like any temp tensor
                    // (KernelEmitter::allocate_tensor, src/nnfusion/core/kernels/kernel_emitter.cpp:282-319)
                    nnf_b200_attn_desc full = desc;
                    full.position = desc.capacity - 1;
                    workspace_bytes = nnf_b200_decode_attention_workspace_bytes(nullptr, &full);
                    if (workspace_bytes > 0)
                        allocate_tensor(Shape{workspace_bytes + 256}, element::character);
                    std::stringstream tag;
                    tag << "b200_decode_attention_" << desc.heads << "_" << desc.kv_heads << "_" << desc.capacity;
                    custom_tag = tag.str();
                }

                LanguageUnit_p emit_function_body() override
                {
                    if (desc.head_dim != 128)
                        return nullptr; // not served: the selector tries the next emitter
                    LanguageUnit_p _lu(new LanguageUnit(get_function_name()));
                    auto& lu = *_lu;
                    lu << "static const nnf_b200_attn_desc desc = {" << desc.heads << ", " << desc.kv_heads << ", "
                       << desc.head_dim << ", " << desc.capacity << ", " << desc.position << ", " << desc.rotary
                       << ", " << desc.rotary_base << "f, " << desc.softmax_scale
                       << "f, 0, NNF_B200_F16, {0, 0, 0, 0}};\n";
                    lu << "NNF_B200_SAFE_CALL(nnf_b200_decode_attention(nnf_b200_ctx_0, stream, &desc, input0, input1, "
                          "input2, input3, input4, output0, "
                       << (workspace_bytes ? "(char*)(((uintptr_t)temp0 + 255) & ~(uintptr_t)255), " : "nullptr, ")
                       << workspace_bytes << "));\n";
                    return _lu;
                }

                LanguageUnit_p emit_dependency() override
                {
                    LanguageUnit_p _lu(new LanguageUnit(get_function_name() + "_dep"));
                    _lu->require(header::cuda);
                    _lu->require(header::stdexcept);
                    _lu->require(header::sstream);
                    _lu->require(header::nnf_b200); // codegen_units.cpp
                    _lu->require(declaration::nnf_b200_ctx);
                    _lu->require(macro::NNF_B200_SAFE_CALL);
                    return _lu;
                }

                LanguageUnit_p emit_function_signature() override
                {
                    // "cudaStream_t" in the text makes the call site pass the stream
                    // (src/nnfusion/core/kernels/kernel_emitter.cpp:160-181)
                    LanguageUnit_p _lu(new LanguageUnit(this->m_kernel_name + "_sig"));
                    auto& lu = *_lu;
                    lu << "void (cudaStream_t stream, half* input0, half* input1, half* input2, half* input3, "
                          "half* input4, half* output0"
                       << (workspace_bytes ? ", char* temp0)" : ")");
                    return _lu;
                }
            };
        } // namespace cuda
    }     // namespace kernels
} // namespace nnfusion

using namespace nnfusion;
using namespace nnfusion::kernels;

// f32 constraint: every kernel lookup passes f32 whatever the tensors hold
// (src/nnfusion/engine/pass/graph/kernel_selection.cpp:185-187)
REGISTER_KERNEL_EMITTER("DecodeAttention",
                        Device(CUDA_GPU).TypeConstraint(element::f32).Tag("b200").Priority(4),
                        cuda::DecodeAttention)
