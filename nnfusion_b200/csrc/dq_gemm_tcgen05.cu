// placeholder until the tcgen05 kernel lands
#include "nnf_internal.h"
namespace nnf
{
size_t gemm_workspace_bytes(const nnf_b200_ctx*, const nnf_b200_linear_desc&) { return 0; }
int gemm_supported(const nnf_b200_ctx*, const nnf_b200_linear_desc&, std::string* why)
{
    *why = "large-M kernel not built";
    return NNF_B200_ENOTSUP;
}
int gemm_launch(nnf_b200_ctx* ctx, cudaStream_t, const nnf_b200_linear_desc&, const void*, const nnf_b200_qweight*,
                const nnf_b200_qweight*, const void*, const void*, void*, void*, size_t)
{
    return set_error(ctx, NNF_B200_ENOTSUP, "large-M kernel not built");
}
int gemm_configure(nnf_b200_ctx*) { return NNF_B200_OK; }
} // namespace nnf
