// C ABI of the library (declarations and reference citations: include/nnf_b200.h).
#include <cuda_runtime.h>
#include <cstring>
#include <new>

#include "nnf_internal.h"
#include "sm100_ptx.cuh"

namespace nnf
{
int set_error(nnf_b200_ctx* ctx, int status, const std::string& msg)
{
    if (ctx)
        ctx->last_error = msg;
    return status;
}

void* load_encode_tiled()
{
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
        return nullptr;
    return fn;
}

bool encode_tensor_map_2d(void* encode_fn, CUtensorMap* map, CUtensorMapDataType dtype, size_t elem_bytes,
                          const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                          uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle)
{
    using Fn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                            const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                            CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    if (!encode_fn)
        return false;
    (void)elem_bytes;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {row_stride_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = reinterpret_cast<Fn>(encode_fn)(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                                                 CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

void overlap_attribute(cudaLaunchAttribute* attr, unsigned* count)
{
    attr->id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr->val.programmaticStreamSerializationAllowed = 1;
    *count = 1;
}

const CUtensorMap* weight_tensor_map(nnf_b200_ctx* ctx, const void* base, int rows, int row_bytes, int box_bytes,
                                     int box_rows)
{
    const int swz = box_bytes == 128 ? 1 : 0;
    auto key = std::make_tuple(base, rows, row_bytes, box_bytes, box_rows, swz);
    auto it = ctx->tensor_maps.find(key);
    if (it != ctx->tensor_maps.end())
        return &it->second;
    alignas(64) CUtensorMap map;
    if (!encode_tensor_map_2d(ctx->encode_tiled, &map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, base, (uint64_t)row_bytes,
                              (uint64_t)rows, (uint64_t)row_bytes, (uint32_t)box_bytes, (uint32_t)box_rows,
                              swz ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE))
        return nullptr;
    if (ctx->tensor_maps.size() > 4096) // callers that churn through weight buffers: start over
        ctx->tensor_maps.clear();
    return &(ctx->tensor_maps[key] = map);
}
} // namespace nnf

namespace
{
bool aligned16(const void* p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

} // namespace

namespace nnf
{
// Everything about a linear call that can be checked without a context: the descriptor's fields, and that the
// operands match it.  Shared by nnf_b200_linear (and its variants) and the entry point that has no context.
int check_linear_call(const nnf_b200_linear_desc* d, const void* x, const nnf_b200_qweight* w,
                      const nnf_b200_qweight* w2, const void* gain, const void* bias, const void* y,
                      const void* workspace, std::string* why)
{
    auto fail = [&](int status, const char* msg) {
        *why = msg;
        return status;
    };
    if (!d)
        return fail(NNF_B200_EINVAL, "null descriptor");
    if (d->M < 1 || d->N < 1 || d->K < 1)
        return fail(NNF_B200_EINVAL, "M, N and K must be positive");
    if (d->w_bits != 4 && d->w_bits != 8)
        return fail(NNF_B200_EINVAL, "w_bits must be 4 or 8");
    if (d->group_size < 0)
        return fail(NNF_B200_EINVAL, "group_size must be >= 0");
    for (int v : {d->x_dtype, d->y_dtype, d->scale_dtype})
        if (v != NNF_B200_F32 && v != NNF_B200_F16)
            return fail(NNF_B200_EINVAL, "dtype fields must be NNF_B200_F32 or NNF_B200_F16");
    if (d->prologue != NNF_B200_PROLOGUE_NONE && d->prologue != NNF_B200_PROLOGUE_RMSNORM)
        return fail(NNF_B200_EINVAL, "unknown prologue");
    if (d->epilogue < NNF_B200_EPILOGUE_NONE || d->epilogue > NNF_B200_EPILOGUE_ADD)
        return fail(NNF_B200_EINVAL, "unknown epilogue");
    if (d->kernel < NNF_B200_KERNEL_AUTO || d->kernel > NNF_B200_KERNEL_GEMM)
        return fail(NNF_B200_EINVAL, "unknown kernel selector");
    if (d->reserved[0] || d->reserved[1] || d->split_k < 0 || (d->flags & ~NNF_B200_FLAG_EXACT_ZP))
        return fail(NNF_B200_EINVAL, "reserved fields must be zero, split_k >= 0, flags known");
    if (!x || !y || !w || !w->wq || !w->scale || !w->zp)
        return fail(NNF_B200_EINVAL, "x, y and the weight set must be non-null");
    const bool dual = d->epilogue == NNF_B200_EPILOGUE_SILU_MUL;
    if (dual && (!w2 || !w2->wq || !w2->scale || !w2->zp))
        return fail(NNF_B200_EINVAL, "SiLU*mul epilogue needs the second weight set");
    if (!dual && w2)
        return fail(NNF_B200_EINVAL, "second weight set given without the SiLU*mul epilogue");
    if (d->prologue == NNF_B200_PROLOGUE_RMSNORM && !gain)
        return fail(NNF_B200_EINVAL, "RMSNorm prologue needs gain");
    if (d->prologue != NNF_B200_PROLOGUE_RMSNORM && gain)
        return fail(NNF_B200_EINVAL, "gain given without the RMSNorm prologue");
    const bool takes_bias = d->epilogue == NNF_B200_EPILOGUE_BIAS || d->epilogue == NNF_B200_EPILOGUE_ADD;
    if (takes_bias && !bias)
        return fail(NNF_B200_EINVAL, "bias / add epilogue needs the bias argument");
    if (!takes_bias && bias)
        return fail(NNF_B200_EINVAL, "bias given without a bias or add epilogue");
    if (!aligned16(x) || !aligned16(w->wq) || (dual && !aligned16(w2->wq)) || (gain && !aligned16(gain)))
        return fail(NNF_B200_EALIGN, "x, wq and gain must be 16-byte aligned");
    if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return fail(NNF_B200_EALIGN, "workspace must be 256-byte aligned");
    return NNF_B200_OK;
}
} // namespace nnf

namespace
{
// Which kernel serves a descriptor: the HBM-bound small-M kernel up to 16 rows, the tensor-core kernel above.
int pick_kernel(const nnf_b200_linear_desc& d)
{
    if (d.kernel != NNF_B200_KERNEL_AUTO)
        return d.kernel;
    return d.M <= 16 ? NNF_B200_KERNEL_GEMV : NNF_B200_KERNEL_GEMM;
}
} // namespace

extern "C" {

int nnf_b200_init(int device, nnf_b200_ctx** out)
{
    if (!out)
        return NNF_B200_EINVAL;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count)
        return NNF_B200_ECUDA;
    if (cudaSetDevice(device) != cudaSuccess)
        return NNF_B200_ECUDA;
    nnf_b200_ctx* ctx = new (std::nothrow) nnf_b200_ctx();
    if (!ctx)
        return NNF_B200_ECUDA;
    ctx->device = device;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess)
    {
        delete ctx;
        return NNF_B200_ECUDA;
    }
    ctx->sm_count = prop.multiProcessorCount;
    ctx->smem_optin = (int)prop.sharedMemPerBlockOptin;
    ctx->cc_major = prop.major;
    ctx->cc_minor = prop.minor;
    if (prop.major != 10)
    {
        // Built for sm_100a only: there is no fallback path.
        delete ctx;
        return NNF_B200_ENOTSUP;
    }
    ctx->encode_tiled = nnf::load_encode_tiled();
    if (!ctx->encode_tiled || cudaMalloc(&ctx->dev_status, 256) != cudaSuccess ||
        cudaMemset(ctx->dev_status, 0, 256) != cudaSuccess)
    {
        delete ctx;
        return NNF_B200_ECUDA;
    }
    int rc = nnf::gemv_configure(ctx);
    if (rc == NNF_B200_OK)
        rc = nnf::gemm_configure(ctx);
    if (rc != NNF_B200_OK)
    {
        delete ctx;
        return rc;
    }
    *out = ctx;
    return NNF_B200_OK;
}

int nnf_b200_free(nnf_b200_ctx* ctx)
{
    if (ctx && ctx->dev_status)
        cudaFree(ctx->dev_status);
    delete ctx;
    return NNF_B200_OK;
}

const char* nnf_b200_strerror(int status)
{
    switch (status)
    {
    case NNF_B200_OK: return "ok";
    case NNF_B200_EINVAL: return "invalid argument";
    case NNF_B200_ENOTSUP: return "not supported";
    case NNF_B200_ECUDA: return "CUDA call failed";
    case NNF_B200_EWORKSPACE: return "workspace missing or too small";
    case NNF_B200_ETIMEDOUT: return "device-side wait timed out";
    case NNF_B200_EALIGN: return "misaligned pointer";
    default: return "unknown status";
    }
}

const char* nnf_b200_last_error(const nnf_b200_ctx* ctx)
{
    return ctx ? ctx->last_error.c_str() : "";
}

int nnf_b200_sm_count(const nnf_b200_ctx* ctx)
{
    return ctx ? ctx->sm_count : 0;
}

size_t nnf_b200_linear_workspace_bytes(const nnf_b200_ctx* ctx, const nnf_b200_linear_desc* desc)
{
    if (!desc) // ctx may be NULL: a 148-SM device is assumed (sizing at code-generation time)
        return 0;
    if (pick_kernel(*desc) == NNF_B200_KERNEL_GEMV)
    {
        // The larger of what the two small-M kernels ask for (the ring kernel serves NNF_B200_FLAG_EXACT_ZP).
        nnf::GemvPlan plan, ring;
        std::string why;
        if (nnf::gemv_plan(ctx, *desc, &plan, &why) != NNF_B200_OK)
            return 0;
        if (nnf::gemv_plan(ctx, *desc, &ring, &why, false) != NNF_B200_OK)
            return plan.workspace_bytes;
        return plan.workspace_bytes > ring.workspace_bytes ? plan.workspace_bytes : ring.workspace_bytes;
    }
    return nnf::gemm_workspace_bytes(ctx, *desc);
}

size_t nnf_b200_allreduce_flag_bytes(size_t count)
{
    return nnf::allreduce_flag_bytes(count);
}

int nnf_b200_allreduce_oneshot(nnf_b200_ctx* ctx, void* stream, int rank, int world, const void* const* bufs,
                               void* const* flags, size_t count, size_t half_stride_bytes, void* out, uint32_t epoch)
{
    if (!ctx)
        return NNF_B200_EINVAL;
    if (world < 1 || world > 8 || rank < 0 || rank >= world || !bufs || !flags || !out || count == 0)
        return nnf::set_error(ctx, NNF_B200_EINVAL, "1 <= world <= 8, 0 <= rank < world, non-null arrays, count > 0");
    if (half_stride_bytes < count * 2 || half_stride_bytes % 16 != 0)
        return nnf::set_error(ctx, NNF_B200_EINVAL, "half_stride_bytes must hold the tensor and be a multiple of 16");
    if (count % 8 != 0 || count > (size_t)1 << 24)
        return nnf::set_error(ctx, NNF_B200_ENOTSUP, "count must be a multiple of 8 fp16 elements, at most 2^24");
    for (int r = 0; r < world; r++)
    {
        if (!bufs[r] || !flags[r])
            return nnf::set_error(ctx, NNF_B200_EINVAL, "null buffer or flag pointer");
        if (!aligned16(bufs[r]) || (reinterpret_cast<uintptr_t>(flags[r]) & 3u))
            return nnf::set_error(ctx, NNF_B200_EALIGN, "buffers must be 16-byte aligned, flags 4-byte aligned");
    }
    if (!aligned16(out))
        return nnf::set_error(ctx, NNF_B200_EALIGN, "out must be 16-byte aligned");
    return nnf::allreduce_launch(ctx, static_cast<cudaStream_t>(stream), rank, world, bufs, flags, count,
                                 half_stride_bytes, out, epoch);
}

size_t nnf_b200_decode_attention_workspace_bytes(const nnf_b200_ctx* ctx, const nnf_b200_attn_desc* desc)
{
    std::string why;
    if (!desc || nnf::attn_check(*desc, &why) != NNF_B200_OK)
        return 0;
    return nnf::attn_workspace_bytes(ctx, *desc);
}

int nnf_b200_decode_attention(nnf_b200_ctx* ctx, void* stream, const nnf_b200_attn_desc* desc, const void* q,
                              const void* k_new, const void* v_new, void* k_cache, void* v_cache, void* out,
                              void* workspace, size_t workspace_bytes)
{
    if (!ctx)
        return NNF_B200_EINVAL;
    if (!desc)
        return nnf::set_error(ctx, NNF_B200_EINVAL, "null descriptor");
    std::string why;
    int rc = nnf::attn_check(*desc, &why);
    if (rc != NNF_B200_OK)
        return nnf::set_error(ctx, rc, why);
    if (!q || !k_new || !v_new || !k_cache || !v_cache || !out)
        return nnf::set_error(ctx, NNF_B200_EINVAL, "q, k_new, v_new, the caches and out must be non-null");
    if (!aligned16(q) || !aligned16(k_new) || !aligned16(v_new) || !aligned16(k_cache) || !aligned16(v_cache) ||
        !aligned16(out))
        return nnf::set_error(ctx, NNF_B200_EALIGN, "attention operands must be 16-byte aligned");
    const size_t need = nnf::attn_workspace_bytes(ctx, *desc);
    if (need > 0 && (!workspace || workspace_bytes < need))
        return nnf::set_error(ctx, NNF_B200_EWORKSPACE,
                              "decode attention needs " + std::to_string(need) + " bytes of workspace");
    if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return nnf::set_error(ctx, NNF_B200_EALIGN, "workspace must be 256-byte aligned");
    return nnf::attn_launch(ctx, static_cast<cudaStream_t>(stream), *desc, q, k_new, v_new, k_cache, v_cache, out,
                            workspace);
}

int nnf_b200_linear_plan(const nnf_b200_ctx* ctx, const nnf_b200_linear_desc* desc, int32_t out[8])
{
    if (!desc || !out)
        return NNF_B200_EINVAL;
    for (int i = 0; i < 8; i++)
        out[i] = 0;
    out[0] = pick_kernel(*desc);
    if (out[0] == NNF_B200_KERNEL_GEMV)
    {
        nnf::GemvPlan plan;
        std::string why;
        int rc = nnf::gemv_plan(ctx, *desc, &plan, &why);
        if (rc != NNF_B200_OK)
            return rc;
        out[1] = plan.warps, out[2] = plan.splits, out[3] = plan.depth, out[4] = plan.splits * plan.ctas_per_split;
        out[5] = (int32_t)plan.smem_bytes;
        out[6] = plan.batch;
        out[7] = (plan.cluster ? 1 : 0) | (plan.l1_lines ? 2 : 0) | (plan.range_layout ? 4 : 0) |
                 (plan.direct && plan.param_bufs == 1 ? 8 : 0);
    }
    return NNF_B200_OK;
}

int nnf_b200_workspace_reset(nnf_b200_ctx* ctx, void* stream, void* workspace, size_t bytes)
{
    if (!ctx)
        return NNF_B200_EINVAL;
    if (bytes == 0)
        return NNF_B200_OK;
    if (!workspace)
        return nnf::set_error(ctx, NNF_B200_EINVAL, "null workspace");
    cudaError_t e = cudaMemsetAsync(workspace, 0, bytes, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess)
        return nnf::set_error(ctx, NNF_B200_ECUDA, std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));
    return NNF_B200_OK;
}

size_t nnf_b200_linear_allreduce_flag_bytes(const nnf_b200_linear_desc* desc)
{
    if (!desc || desc->N < 1)
        return 0;
    return (size_t)((desc->N + 15) / 16) * 9 * sizeof(uint32_t); // [row tile][8 senders], then [row tile] counters
}

static int linear_impl(nnf_b200_ctx* ctx, void* stream, const nnf_b200_linear_desc* desc, const void* x,
                       const nnf_b200_qweight* w, const nnf_b200_qweight* w2, const void* gain, const void* bias,
                       void* y, void* workspace, size_t workspace_bytes, const nnf_b200_peers* peers);

int nnf_b200_linear(nnf_b200_ctx* ctx, void* stream, const nnf_b200_linear_desc* desc, const void* x,
                    const nnf_b200_qweight* w, const nnf_b200_qweight* w2, const void* gain, const void* bias,
                    void* y, void* workspace, size_t workspace_bytes)
{
    return linear_impl(ctx, stream, desc, x, w, w2, gain, bias, y, workspace, workspace_bytes, nullptr);
}

int nnf_b200_linear_allreduce(nnf_b200_ctx* ctx, void* stream, const nnf_b200_linear_desc* desc, const void* x,
                              const nnf_b200_qweight* w, const void* bias, void* y, void* workspace,
                              size_t workspace_bytes, const nnf_b200_peers* peers)
{
    if (!ctx)
        return NNF_B200_EINVAL;
    if (!peers || !desc)
        return nnf::set_error(ctx, NNF_B200_EINVAL, "null descriptor or peer description");
    if (peers->world < 1 || peers->world > 8 || peers->rank < 0 || peers->rank >= peers->world || !peers->bufs ||
        !peers->flags)
        return nnf::set_error(ctx, NNF_B200_EINVAL, "1 <= world <= 8, 0 <= rank < world, non-null pointer arrays");
    if (desc->M > 16 || desc->kernel == NNF_B200_KERNEL_GEMM || desc->prologue != NNF_B200_PROLOGUE_NONE ||
        desc->epilogue == NNF_B200_EPILOGUE_SILU_MUL || desc->y_dtype != NNF_B200_F16)
        return nnf::set_error(ctx, NNF_B200_ENOTSUP,
                              "the fused sum over ranks serves the small-M kernel (M <= 16), fp16 output, no RMSNorm "
                              "prologue and no SiLU*mul epilogue");
    if (peers->half_stride_bytes < (size_t)peers->world * desc->M * desc->N * sizeof(float) ||
        peers->half_stride_bytes % 16 != 0)
        return nnf::set_error(ctx, NNF_B200_EINVAL,
                              "half_stride_bytes must hold world * M * N floats and be a multiple of 16");
    for (int r = 0; r < peers->world; r++)
    {
        if (!peers->bufs[r] || !peers->flags[r])
            return nnf::set_error(ctx, NNF_B200_EINVAL, "null peer buffer or flag pointer");
        if (!aligned16(peers->bufs[r]) || (reinterpret_cast<uintptr_t>(peers->flags[r]) & 3u))
            return nnf::set_error(ctx, NNF_B200_EALIGN, "peer buffers 16-byte aligned, flags 4-byte aligned");
    }
    return linear_impl(ctx, stream, desc, x, w, nullptr, nullptr, bias, y, workspace, workspace_bytes, peers);
}

static int linear_impl(nnf_b200_ctx* ctx, void* stream, const nnf_b200_linear_desc* desc, const void* x,
                       const nnf_b200_qweight* w, const nnf_b200_qweight* w2, const void* gain, const void* bias,
                       void* y, void* workspace, size_t workspace_bytes, const nnf_b200_peers* peers)
{
    if (!ctx)
        return NNF_B200_EINVAL;
    std::string bad;
    int rc = nnf::check_linear_call(desc, x, w, w2, gain, bias, y, workspace, &bad);
    if (rc != NNF_B200_OK)
        return nnf::set_error(ctx, rc, bad);
    const nnf_b200_linear_desc& d = *desc;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (pick_kernel(d) == NNF_B200_KERNEL_GEMV)
    {
        nnf::GemvPlan plan;
        std::string why;
        rc = nnf::gemv_plan(ctx, d, &plan, &why);
        if (rc != NNF_B200_OK)
            return nnf::set_error(ctx, rc, why);
        if (plan.workspace_bytes > 0 && (!workspace || workspace_bytes < plan.workspace_bytes))
            return nnf::set_error(ctx, NNF_B200_EWORKSPACE,
                                  "workspace of " + std::to_string(plan.workspace_bytes) + " bytes required");
        return nnf::gemv_launch(ctx, s, d, plan, x, w, w2, gain, bias, y, workspace, peers);
    }
    if (peers)
        return nnf::set_error(ctx, NNF_B200_ENOTSUP, "the fused sum over ranks needs the small-M kernel");
    std::string why;
    rc = nnf::gemm_supported(ctx, d, &why);
    if (rc != NNF_B200_OK)
        return nnf::set_error(ctx, rc, why);
    return nnf::gemm_launch(ctx, s, d, x, w, w2, gain, bias, y, workspace, workspace_bytes);
}

int nnf_b200_device_status(nnf_b200_ctx* ctx, void* stream)
{
    if (!ctx)
        return NNF_B200_EINVAL;
    int host = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(&host, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaMemsetAsync(ctx->dev_status, 0, sizeof(int), s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess)
        return nnf::set_error(ctx, NNF_B200_ECUDA, "reading the device status word failed");
    if (host != 0)
        return nnf::set_error(ctx, NNF_B200_ETIMEDOUT, "a bounded device-side wait gave up");
    return NNF_B200_OK;
}

uint64_t nnf_b200_launch_count(nnf_b200_ctx* ctx, int reset)
{
    if (!ctx)
        return 0;
    uint64_t v = ctx->launches;
    if (reset)
        ctx->launches = 0;
    return v;
}

int nnf_b200_pack_u4(const uint8_t* vals, size_t rows, size_t cols, uint8_t* out)
{
    if (!vals || !out)
        return NNF_B200_EINVAL;
    const size_t ob = (cols + 1) / 2;
    for (size_t r = 0; r < rows; r++)
        for (size_t b = 0; b < ob; b++)
        {
            const uint8_t lo = vals[r * cols + 2 * b];
            const uint8_t hi = (2 * b + 1 < cols) ? vals[r * cols + 2 * b + 1] : 0;
            if (lo > 15 || hi > 15)
                return NNF_B200_EINVAL;
            out[r * ob + b] = (uint8_t)(lo | (hi << 4));
        }
    return NNF_B200_OK;
}
}
