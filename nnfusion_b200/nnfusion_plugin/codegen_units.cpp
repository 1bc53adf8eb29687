// Language units the DequantDot / DecodeAttention emitters require in the generated project (declared in
// nnf_b200_langunit.hpp; LU_DEFINE: src/nnfusion/core/kernels/common_langunit.hpp:11-14).
//   header::nnf_b200, macro::NNF_B200_SAFE_CALL  -> next to the units of
//       src/nnfusion/core/kernels/cuda_gpu/cuda_langunit.cpp (CUDA_SAFE_CALL: :47-62)
//   cmake::nnf_b200                               -> next to cmake::superscaler_cuda,
//       src/nnfusion/engine/pass/codegen/codegen_langunit.cpp:44-51; cuda_codegen_pass adds it when the header
//       unit is present (pattern: cuda_codegen_pass.cpp:62,100-104,1420-1424) and extends CUDA_ARCH (:1374).
#include "nnf_b200_langunit.hpp"

LU_DEFINE(nnfusion::kernels::header::nnf_b200, "#include \"nnf_b200.h\"\n");

LU_DEFINE(nnfusion::kernels::declaration::nnf_b200_ctx, "nnf_b200_ctx* nnf_b200_ctx_0 = nullptr;\n");

LU_DEFINE(nnfusion::kernels::macro::NNF_B200_SAFE_CALL,
          R"(#define NNF_B200_SAFE_CALL(func)                                                              \
    do                                                                                            \
    {                                                                                             \
        int nnf_status_ = (func);                                                                 \
        if (nnf_status_ != NNF_B200_OK)                                                           \
        {                                                                                         \
            std::stringstream safe_call_ss;                                                       \
            safe_call_ss << "\nerror: " #func " failed with error"                                \
                         << "\nfile: " << __FILE__ << "\nline: " << __LINE__                      \
                         << "\nmsg: " << nnf_b200_strerror(nnf_status_) << ": "                   \
                         << nnf_b200_last_error(nnf_b200_ctx_0);                                  \
            throw std::runtime_error(safe_call_ss.str());                                         \
        }                                                                                         \
    } while (0)
)");

LU_DEFINE(nnfusion::codegen::cmake::nnf_b200,
          R"(
if (NOT DEFINED ENV{NNF_B200_LIB})
message(FATAL_ERROR "NNF_B200_LIB must point at libnnf_b200.so: this graph has no other kernel for DequantDot")
endif()
include_directories($ENV{NNF_B200_INCLUDE})
target_link_libraries(${TARGET_NAME} $ENV{NNF_B200_LIB})
set(CUDA_NVCC_FLAGS "${CUDA_NVCC_FLAGS} -gencode arch=compute_100a,code=sm_100a")
)");
