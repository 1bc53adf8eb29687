// See dequant_dot_emitter.hpp.  The generated function takes the stream (the call site prepends it when the
// signature contains "cudaStream_t": src/nnfusion/core/kernels/kernel_emitter.cpp:160-181), the inputs, the output
// and the workspace tensor, and makes one nnf_b200_linear call.
#include "dequant_dot_emitter.hpp"
#include "nnf_b200.h" // linked into the compiler only for nnf_b200_linear_plan / _workspace_bytes (host functions)

using namespace nnfusion;
using namespace nnfusion::kernels;

namespace
{
    const char* dtype_enum(const element::Type& t)
    {
        return t == element::f16 ? "NNF_B200_F16" : "NNF_B200_F32";
    }
    int dtype_value(const element::Type& t) { return t == element::f16 ? NNF_B200_F16 : NNF_B200_F32; }
    int epilogue_value(const std::string& e)
    {
        return e == "bias" ? NNF_B200_EPILOGUE_BIAS
                           : e == "silu_mul" ? NNF_B200_EPILOGUE_SILU_MUL
                                             : e == "add" ? NNF_B200_EPILOGUE_ADD : NNF_B200_EPILOGUE_NONE;
    }
    const char* epilogue_enum(const std::string& e)
    {
        return e == "bias" ? "NNF_B200_EPILOGUE_BIAS"
                           : e == "silu_mul" ? "NNF_B200_EPILOGUE_SILU_MUL"
                                             : e == "add" ? "NNF_B200_EPILOGUE_ADD" : "NNF_B200_EPILOGUE_NONE";
    }
}

cuda::DequantDot::DequantDot(shared_ptr<KernelContext> ctx)
    : CudaLibEmitter(ctx)
{
    generic_op = static_pointer_cast<op::GenericOp>(ctx->gnode->get_op_ptr());
    auto& cfg = generic_op->localOpConfig.getRoot();
    w_bits = cfg["w_bits"];
    group_size = cfg["group_size"];
    prologue = cfg["prologue"];
    epilogue = cfg["epilogue"];
    rms_eps = cfg["rms_eps"];
    const auto& x_shape = ctx->inputs[0]->get_shape();
    const auto& w_shape = ctx->inputs[1]->get_shape();
    M = x_shape[0], K = x_shape[1], N = w_shape[0];

    // Workspace: sized at code-generation time for a 148-SM device, planned like any temp tensor
    // (KernelEmitter::allocate_tensor, kernel_emitter.cpp:282-319).
    nnf_b200_linear_desc d = {};
    d.M = (int32_t)M, d.N = (int32_t)N, d.K = (int32_t)K;
    d.w_bits = w_bits, d.group_size = group_size;
    d.x_dtype = dtype_value(ctx->inputs[0]->get_element_type());
    d.y_dtype = dtype_value(ctx->outputs[0]->get_element_type());
    d.scale_dtype = dtype_value(ctx->inputs[2]->get_element_type());
    d.prologue = prologue == "rmsnorm" ? NNF_B200_PROLOGUE_RMSNORM : NNF_B200_PROLOGUE_NONE;
    d.epilogue = epilogue_value(epilogue);
    workspace_bytes = nnf_b200_linear_workspace_bytes(nullptr, &d);
    if (workspace_bytes > 0)
        workspace = allocate_tensor(Shape{workspace_bytes + 256}, element::character);

    std::stringstream tag;
    tag << "b200_dqdot_" << M << "_" << N << "_" << K << "_w" << w_bits << "_g" << group_size << "_" << prologue << "_"
        << epilogue;
    custom_tag = tag.str();
}

LanguageUnit_p cuda::DequantDot::emit_function_body()
{
    int32_t plan[8];
    nnf_b200_linear_desc probe = {};
    probe.M = (int32_t)M, probe.N = (int32_t)N, probe.K = (int32_t)K, probe.w_bits = w_bits, probe.group_size = group_size;
    probe.x_dtype = dtype_value(m_context->inputs[0]->get_element_type());
    probe.y_dtype = dtype_value(m_context->outputs[0]->get_element_type());
    probe.scale_dtype = dtype_value(m_context->inputs[2]->get_element_type());
    probe.epilogue = epilogue_value(epilogue);
    if (nnf_b200_linear_plan(nullptr, &probe, plan) != NNF_B200_OK && M <= 16)
        return nullptr; // shape not served: the selector falls through to the next emitter (kernel_selection.cpp:262-267)

    LanguageUnit_p _lu(new LanguageUnit(get_function_name()));
    auto& lu = *_lu;
    size_t next = 4; // first optional input
    std::string gain = "nullptr", bias = "nullptr", w2 = "nullptr";
    if (prologue == "rmsnorm")
        gain = "input" + std::to_string(next++);
    if (epilogue == "bias" || epilogue == "add") // the [M,N] addend travels in the bias argument
        bias = "input" + std::to_string(next++);
    lu << "static const nnf_b200_linear_desc desc = {" << M << ", " << N << ", " << K << ", " << w_bits << ", "
       << group_size << ", " << dtype_enum(m_context->inputs[0]->get_element_type()) << ", "
       << dtype_enum(m_context->outputs[0]->get_element_type()) << ", "
       << dtype_enum(m_context->inputs[2]->get_element_type()) << ", "
       << (prologue == "rmsnorm" ? "NNF_B200_PROLOGUE_RMSNORM" : "NNF_B200_PROLOGUE_NONE") << ", "
       << epilogue_enum(epilogue) << ", " << rms_eps << "f, NNF_B200_KERNEL_AUTO, 0, 0, {0, 0}};\n";
    lu << "const nnf_b200_qweight w = {input1, input2, input3};\n";
    if (epilogue == "silu_mul")
    {
        lu << "const nnf_b200_qweight w_up = {input" << next << ", input" << next + 1 << ", input" << next + 2 << "};\n";
        w2 = "&w_up";
    }
    if (workspace_bytes > 0)
        lu << "char* ws = (char*)(((uintptr_t)temp0 + 255) & ~(uintptr_t)255);\n";
    lu << "NNF_B200_SAFE_CALL(nnf_b200_linear(nnf_b200_ctx_0, stream, &desc, input0, &w, " << w2 << ", " << gain << ", "
       << bias << ", output0, " << (workspace_bytes > 0 ? "ws" : "nullptr") << ", " << workspace_bytes << "));\n";
    return _lu;
}

LanguageUnit_p cuda::DequantDot::emit_function_signature()
{
    LanguageUnit_p _lu(new LanguageUnit(this->m_kernel_name + "_sig"));
    auto& lu = *_lu;
    vector<string> params;
    for (size_t i = 0; i < m_context->inputs.size(); i++)
        params.push_back(m_context->inputs[i]->get_element_type().c_type_string() + "* input" + to_string(i));
    for (size_t i = 0; i < m_context->outputs.size(); i++)
        params.push_back(m_context->outputs[i]->get_element_type().c_type_string() + "* output" + to_string(i));
    for (size_t i = 0; i < m_context->tensors.size(); i++)
        params.push_back(m_context->tensors[i]->get_element_type().c_type_string() + "* temp" + to_string(i));
    lu << "void (cudaStream_t stream, " << join(params, ", ") << ")";
    return _lu;
}

LanguageUnit_p cuda::DequantDot::emit_dependency()
{
    LanguageUnit_p _lu(new LanguageUnit(get_function_name() + "_dep"));
    _lu->require(header::cuda);
    _lu->require(header::stdexcept);
    _lu->require(header::sstream);
    _lu->require(header::nnf_b200);
    _lu->require(declaration::nnf_b200_ctx);
    _lu->require(macro::NNF_B200_SAFE_CALL);
    return _lu;
}

// Lookups always pass f32 whatever the tensor types are (engine/pass/graph/kernel_selection.cpp:185-187).
// Priority 4 is above the cuBLAS emitters (2) and below Antares (9) and custom ops (10).
REGISTER_KERNEL_EMITTER("DequantDot",
                        Device(CUDA_GPU).TypeConstraint(element::f32).Tag("b200").Priority(4),
                        cuda::DequantDot)
