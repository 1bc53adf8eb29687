// Single-token (decode) attention over a key/value cache for sm_100a, with the rotary embedding of q and of the new
// key and the append of the new key/value row fused in:
//     out[h] = softmax(rot(q[h]) . K[kv(h)]^T * scale) . V[kv(h)],   K/V rows 0 .. position (the new row included).
//
// In the reference this is a chain of separate kernels: Slice / Negative / Concat / Multiply / Add for the rotary
// embedding (element-wise emitters, src/nnfusion/core/kernels/cuda_gpu/kernels/elementwise.hpp:33-157), a strided-batched
// cuBLAS GEMM for q.K^T (src/nnfusion/core/kernels/cuda_gpu/kernels/batch_matmul.cpp:49-144, adj_y), Softmax
// (src/nnfusion/core/kernels/cuda_gpu/kernels/softmax.cpp:78-122) and a second batched GEMM for P.V; the BERT-style
// fused Attention op (src/nnfusion/core/kernels/cuda_gpu/kernels/attention.cpp:13-152) stops at 1024 positions.
//
// The kernel is HBM-bound: every cache row is read once (16-byte loads into two register buffers of 32 rows each:
// 32 KB in flight per CTA, four CTAs per SM).  The positions of a head are cut into `splits` contiguous ranges, one CTA each; a CTA keeps a running
// maximum / sum / weighted value sum (fp32) over its range, stores them, takes a ticket, and the CTA that arrives last
// for a head combines the ranges in a fixed order, so results are bitwise repeatable and nothing ever waits.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <algorithm>
#include <cmath>
#include <string>

#include "nnf_internal.h"

namespace
{
constexpr int kD = 128;        // head dimension
constexpr int kThreads = 128;  // 4 warps; 16 lanes x 16 bytes cover one row, so a warp load covers 2 rows
constexpr int kRounds = 4;     // rows per thread in flight: 4 rounds x 8 rows = 32 rows per pass
constexpr int kRowsPerPass = 8 * kRounds;
constexpr int kSlot = kD + 2;  // floats per (head, split): weighted value sum, maximum, sum

struct AttnParams
{
    const __half* q;     // [heads][128], before the rotary embedding
    const __half* k_new; // [kv_heads][128], before the rotary embedding
    const __half* v_new; // [kv_heads][128]
    __half* k_cache;     // [kv_heads][capacity][128]
    __half* v_cache;
    __half* out;         // [heads][128]
    float* ws_part;      // [heads][splits][kSlot]
    unsigned* ws_count;  // [heads]
    int heads, kv_heads, capacity, position, splits, chunk, rotary;
    float scale, log2_base;
};

// Rotary embedding of element d of a 128-vector held in shared memory (fp32): pairs (i, i + 64) are rotated by
// position * base^(-2i/128); the "rotate half" form, x*cos + concat(-x[64:], x[:64])*sin.
__device__ __forceinline__ float rotate(const float* x, int d, int position, float log2_base)
{
    const int i = d & 63;
    const float inv_freq = exp2f(-(float)(2 * i) / (float)kD * log2_base);
    float sn, cs;
    sincosf((float)position * inv_freq, &sn, &cs);
    return d < 64 ? x[d] * cs - x[d + 64] * sn : x[d] * cs + x[d - 64] * sn;
}

__global__ void __launch_bounds__(kThreads, 4) decode_attention_kernel(const AttnParams p)
{
    __shared__ float q_s[kD];      // rotated q, already multiplied by the softmax scale
    __shared__ float raw_s[kD];    // staging for the rotary embedding
    __shared__ __half knew_s[kD];  // the new key row as it is stored in the cache (fp16)
    __shared__ float red_s[4][kD]; // per-warp weighted value sums
    __shared__ float stat_s[2][4]; // per-warp maximum / sum
    __shared__ int last_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int half = lane >> 4, dg = lane & 15; // which of the warp's two rows, which 8 dimensions
    const int head = blockIdx.y, split = blockIdx.x;
    const int kvh = head / (p.heads / p.kv_heads);
    const int n_rows = p.position + 1;
    const int begin = split * p.chunk, end = min(begin + p.chunk, n_rows);
    const bool owns_new = begin <= p.position && p.position < end;
    // Before anything else, and before the launch ahead of this one has finished: ask for the CTA's whole range of
    // both caches to be brought into L2 (two bulk requests; a prefetch hands no values to anyone, so it may run
    // ahead of the wait below).  HBM then streams from the first microsecond, and the register loads further down see
    // L2 latency.
    if (tid == 0 && end > begin)
    {
        const size_t first = ((size_t)kvh * p.capacity + begin) * kD;
        const uint32_t bytes = (uint32_t)(end - begin) * kD * (uint32_t)sizeof(__half);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.k_cache + first), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.v_cache + first), "r"(bytes) : "memory");
    }
    // The next launch on the stream may start as SMs become free; this one waits for the launch before it (which
    // produced q, k, v; the cache rows it reads were written by earlier steps, but nothing is assumed about those).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- q first (a few bytes that everything waits for), then the first two passes of cache rows: nothing below
    // depends on those until the scores
    const float q_raw = __half2float(p.q[(size_t)head * kD + tid]);
    const __half* kbase = p.k_cache + (size_t)kvh * p.capacity * kD + 8 * dg;
    const __half* vbase = p.v_cache + (size_t)kvh * p.capacity * kD + 8 * dg;
    const int my_row = warp * 2 + half; // row of this thread within a group of 8
    // Two register buffers of one pass (32 rows) each.  Rows past the end of the range read as zeros; the new row
    // is not in the cache yet and is patched in when it is used.
    uint4 kraw[2][kRounds], vraw[2][kRounds];
    auto load_pass = [&](uint4 (&kb)[kRounds], uint4 (&vb)[kRounds], int row0) {
#pragma unroll
        for (int r = 0; r < kRounds; r++)
        {
            const int row = row0 + r * 8 + my_row;
            const bool live = row < end && row != p.position;
            kb[r] = live ? __ldcs(reinterpret_cast<const uint4*>(kbase + (size_t)row * kD)) : make_uint4(0u, 0u, 0u, 0u);
            vb[r] = live ? __ldcs(reinterpret_cast<const uint4*>(vbase + (size_t)row * kD)) : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    load_pass(kraw[0], vraw[0], begin);
    load_pass(kraw[1], vraw[1], begin + kRowsPerPass);

    // ---- q (and, in the CTA whose range holds the new row, k) through the rotary embedding
    raw_s[tid] = q_raw;
    __syncthreads();
    q_s[tid] = (p.rotary ? rotate(raw_s, tid, p.position, p.log2_base) : raw_s[tid]) * p.scale;
    __syncthreads();
    if (owns_new)
    {
        raw_s[tid] = __half2float(p.k_new[(size_t)kvh * kD + tid]);
        __syncthreads();
        const __half kr = __float2half_rn(p.rotary ? rotate(raw_s, tid, p.position, p.log2_base) : raw_s[tid]);
        knew_s[tid] = kr;
        // append: every head of a group writes the same values
        p.k_cache[((size_t)kvh * p.capacity + p.position) * kD + tid] = kr;
        p.v_cache[((size_t)kvh * p.capacity + p.position) * kD + tid] = p.v_new[(size_t)kvh * kD + tid];
    }
    __syncthreads();
    float qv[8];
#pragma unroll
    for (int j = 0; j < 8; j++)
        qv[j] = q_s[8 * dg + j];

    // ---- running softmax over the range, 32 rows per pass
    float m_run = -INFINITY, l_run = 0.f, acc[8];
#pragma unroll
    for (int j = 0; j < 8; j++)
        acc[j] = 0.f;
    auto consume = [&](uint4 (&kb)[kRounds], uint4 (&vb)[kRounds], int row0) {
        float s[kRounds];
        float m_pass = -INFINITY;
#pragma unroll
        for (int r = 0; r < kRounds; r++)
        {
            const int row = row0 + r * 8 + my_row;
            if (row == p.position && row < end)
            {
                kb[r] = *reinterpret_cast<const uint4*>(knew_s + 8 * dg);
                vb[r] = *reinterpret_cast<const uint4*>(p.v_new + (size_t)kvh * kD + 8 * dg);
            }
            const __half2* kh = reinterpret_cast<const __half2*>(&kb[r]);
            float d = 0.f;
#pragma unroll
            for (int j = 0; j < 4; j++)
            {
                const float2 kf = __half22float2(kh[j]);
                d = fmaf(qv[2 * j], kf.x, d);
                d = fmaf(qv[2 * j + 1], kf.y, d);
            }
            d += __shfl_xor_sync(0xffffffffu, d, 8);
            d += __shfl_xor_sync(0xffffffffu, d, 4);
            d += __shfl_xor_sync(0xffffffffu, d, 2);
            d += __shfl_xor_sync(0xffffffffu, d, 1);
            s[r] = row < end ? d : -INFINITY;
            m_pass = fmaxf(m_pass, s[r]);
        }
        // maximum of the pass over the whole CTA (every pass has at least one row)
        m_pass = fmaxf(m_pass, __shfl_xor_sync(0xffffffffu, m_pass, 16));
        if (lane == 0)
            stat_s[0][warp] = m_pass;
        __syncthreads();
        m_pass = fmaxf(fmaxf(stat_s[0][0], stat_s[0][1]), fmaxf(stat_s[0][2], stat_s[0][3]));
        __syncthreads();
        const float m_new = fmaxf(m_run, m_pass);
        const float corr = expf(m_run - m_new); // 0 on the first pass
        l_run *= corr;
#pragma unroll
        for (int j = 0; j < 8; j++)
            acc[j] *= corr;
#pragma unroll
        for (int r = 0; r < kRounds; r++)
        {
            const float w = expf(s[r] - m_new); // 0 for rows past the end
            l_run += w;
            const __half2* vh = reinterpret_cast<const __half2*>(&vb[r]);
#pragma unroll
            for (int j = 0; j < 4; j++)
            {
                const float2 vf = __half22float2(vh[j]);
                acc[2 * j] = fmaf(w, vf.x, acc[2 * j]);
                acc[2 * j + 1] = fmaf(w, vf.y, acc[2 * j + 1]);
            }
        }
        m_run = m_new;
    };
    // two passes per trip: while one buffer is consumed the other one's rows are on their way, and a buffer is
    // asked to be refilled as soon as it has been consumed
    for (int row0 = begin; row0 < end; row0 += 2 * kRowsPerPass)
    {
        consume(kraw[0], vraw[0], row0);
        if (row0 + 2 * kRowsPerPass < end)
            load_pass(kraw[0], vraw[0], row0 + 2 * kRowsPerPass);
        if (row0 + kRowsPerPass < end)
        {
            consume(kraw[1], vraw[1], row0 + kRowsPerPass);
            if (row0 + 3 * kRowsPerPass < end)
                load_pass(kraw[1], vraw[1], row0 + 3 * kRowsPerPass);
        }
    }

    // ---- sums over the CTA: the two rows of a warp, then the four warps (fixed order)
#pragma unroll
    for (int j = 0; j < 8; j++)
        acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 16);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 16); // every lane of a 16-lane group carries the same sum
    if (half == 0)
    {
#pragma unroll
        for (int j = 0; j < 8; j++)
            red_s[warp][8 * dg + j] = acc[j];
    }
    if (lane == 0)
        stat_s[1][warp] = l_run;
    __syncthreads();
    const float acc_d = (red_s[0][tid] + red_s[1][tid]) + (red_s[2][tid] + red_s[3][tid]);
    const float l_cta = (stat_s[1][0] + stat_s[1][1]) + (stat_s[1][2] + stat_s[1][3]);

    float* mine = p.ws_part + ((size_t)head * p.splits + split) * kSlot;
    if (p.splits == 1)
    {
        p.out[(size_t)head * kD + tid] = __float2half_rn(acc_d / l_cta);
        return;
    }
    __stcg(mine + tid, acc_d);
    if (tid == 0)
    {
        __stcg(mine + kD, m_run);
        __stcg(mine + kD + 1, l_cta);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0)
    {
        const unsigned old = atomicAdd(p.ws_count + head, 1u);
        last_s = old == (unsigned)(p.splits - 1);
        if (last_s)
            p.ws_count[head] = 0u; // leave the counter zeroed for the next call
    }
    __syncthreads();
    if (!last_s)
        return;
    __threadfence();
    const float* parts = p.ws_part + (size_t)head * p.splits * kSlot;
    float m_all = -INFINITY;
    for (int s = 0; s < p.splits; s++)
        m_all = fmaxf(m_all, __ldcg(parts + s * kSlot + kD));
    float l_all = 0.f, o = 0.f;
    for (int s = 0; s < p.splits; s++)
    {
        const float l_s = __ldcg(parts + s * kSlot + kD + 1);
        if (l_s == 0.f)
            continue; // an empty range
        const float w = expf(__ldcg(parts + s * kSlot + kD) - m_all);
        l_all = fmaf(l_s, w, l_all);
        o = fmaf(__ldcg(parts + s * kSlot + tid), w, o);
    }
    p.out[(size_t)head * kD + tid] = __float2half_rn(o / l_all);
}

// Ranges per head: as many CTAs as the machine holds at once (four per SM), at least 16 rows each.
int pick_splits(const nnf_b200_ctx* ctx, const nnf_b200_attn_desc& d)
{
    const int sms = ctx ? ctx->sm_count : 148;
    const int rows = d.position + 1;
    if (d.splits > 0)
        return std::min(std::min(d.splits, std::max(1, rows / 16)), 1024);
    // ranges of whole passes (32 rows), as many as fill the machine once
    const int target = std::max(1, (sms * 4) / d.heads); // four CTAs of this kernel fit on an SM
    const int passes = std::max(1, (rows + target * kRowsPerPass / 2) / (target * kRowsPerPass));
    const int chunk = passes * kRowsPerPass;
    return std::min((rows + chunk - 1) / chunk, 1024);
}
} // namespace

namespace nnf
{
int attn_check(const nnf_b200_attn_desc& d, std::string* why)
{
    if (d.heads < 1 || d.kv_heads < 1 || d.heads % d.kv_heads != 0 || d.position < 0 || d.capacity <= d.position ||
        d.splits < 0 || d.reserved[0] || d.reserved[1] || d.reserved[2] || d.reserved[3])
    {
        *why = "heads must be a positive multiple of kv_heads, 0 <= position < capacity, splits >= 0, reserved zero";
        return NNF_B200_EINVAL;
    }
    if (d.head_dim != kD || d.dtype != NNF_B200_F16)
    {
        *why = "decode attention is built for head_dim 128 and fp16 tensors";
        return NNF_B200_ENOTSUP;
    }
    return NNF_B200_OK;
}

size_t attn_workspace_bytes(const nnf_b200_ctx* ctx, const nnf_b200_attn_desc& d)
{
    const int splits = pick_splits(ctx, d);
    if (splits == 1)
        return 0;
    const size_t cnt = ((size_t)d.heads * sizeof(unsigned) + 255) / 256 * 256;
    return cnt + (size_t)d.heads * splits * kSlot * sizeof(float);
}

int attn_launch(nnf_b200_ctx* ctx, cudaStream_t stream, const nnf_b200_attn_desc& d, const void* q, const void* k_new,
                const void* v_new, void* k_cache, void* v_cache, void* out, void* workspace)
{
    AttnParams p{};
    p.q = static_cast<const __half*>(q);
    p.k_new = static_cast<const __half*>(k_new);
    p.v_new = static_cast<const __half*>(v_new);
    p.k_cache = static_cast<__half*>(k_cache);
    p.v_cache = static_cast<__half*>(v_cache);
    p.out = static_cast<__half*>(out);
    p.heads = d.heads, p.kv_heads = d.kv_heads, p.capacity = d.capacity, p.position = d.position;
    p.rotary = d.rotary != 0;
    p.scale = d.softmax_scale > 0.f ? d.softmax_scale : 1.0f / sqrtf((float)kD);
    p.log2_base = log2f(d.rotary_base > 0.f ? d.rotary_base : 10000.f);
    p.splits = pick_splits(ctx, d);
    const int rows = d.position + 1;
    // whole passes per range; ranges left without rows store an empty partial result that the combine skips
    p.chunk = ((rows + p.splits - 1) / p.splits + kRowsPerPass - 1) / kRowsPerPass * kRowsPerPass;
    if (p.splits > 1)
    {
        const size_t cnt = ((size_t)d.heads * sizeof(unsigned) + 255) / 256 * 256;
        p.ws_count = static_cast<unsigned*>(workspace);
        p.ws_part = reinterpret_cast<float*>(static_cast<char*>(workspace) + cnt);
    }
    (void)cudaGetLastError();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.splits, d.heads);
    cfg.blockDim = dim3(kThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    overlap_attribute(attr, &cfg.numAttrs);
    cfg.attrs = attr;
    cudaError_t e = cudaLaunchKernelEx(&cfg, decode_attention_kernel, p);
    if (e != cudaSuccess)
        return set_error(ctx, NNF_B200_ECUDA, std::string("decode_attention launch: ") + cudaGetErrorString(e));
    ctx->launches++;
    return NNF_B200_OK;
}
} // namespace nnf
