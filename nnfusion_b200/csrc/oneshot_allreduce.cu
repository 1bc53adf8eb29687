// One-shot sum all-reduce of a small fp16 tensor over peer memory (NVLink / NVSwitch), for the shard boundary of a
// tensor-parallel layer at decode sizes (a few KB to a few hundred KB per rank).
//
// Stands in for the NCCL call behind the reference's only collective, cuda::SuperScalerAllReduce
// (src/nnfusion/core/kernels/cuda_gpu/kernels/allreduce.cpp:18-98; the call itself in
// src/tools/nnfusion/templates/super_scaler/super_scaler.cu:244-277), where a ring over a few kilobytes is all
// latency.  Every rank keeps its addend in a buffer that all ranks have mapped (plain peer pointers,
// plain loads and stores): a CTA tells every peer "my buffer holds call number `epoch`" with one flag store per peer, waits until every
// peer has said the same to it, then reads its slice of all buffers with 16-byte peer loads, adds them in rank
// order in fp32 (so every rank gets the same bits) and writes the sum to local memory.
//
// Flags are never reset: they only grow (one 32-bit word per CTA and sender on the receiving rank), a wait is
// "flag >= epoch".  Calls alternate between the two halves of every rank's buffer (half = epoch & 1): a rank may run
// one call ahead of a peer that is still reading, never two (its next wait needs that peer's next flag).  The call
// number comes from the host, or (epoch argument 0) from ONE counter per flag area, which makes a captured sequence
// of calls replayable: every CTA of a launch reads it, the CTA that finishes last (a ticket word beside it) writes
// the new value, and the next launch reads it only after this one has completed.  The layout of a flag area does
// not depend on the size of the tensor of a particular call -- 16 header words (counter, ticket), then the flag
// words [CTA][sender] -- so calls of different sizes may share one area.  Every wait is bounded; a wait that gives up
// raises the context's device status word and the CTA writes nothing.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <string>

#include "nnf_internal.h"

namespace
{
constexpr int kMaxRanks = 8;
constexpr int kArThreads = 256;
constexpr uint32_t kArSpin = 1u << 19; // polls of just under a microsecond each: gives up after roughly 0.4 s
constexpr int kArHeaderWords = 16;     // call counter, ticket, padding to 64 bytes; the flags follow

struct ArParams
{
    const char* bufs[kMaxRanks]; // buffer (both halves) of every rank, own included, as mapped on this rank
    uint32_t* flags[kMaxRanks];  // flag words of every rank: [CTA][sender] (behind the header words)
    uint32_t* header;            // this rank's call counter [0] and ticket [1]
    size_t half_stride;          // bytes between the two halves of a buffer
    uint4* out;
    int* status;
    int rank, world;
    uint32_t vecs; // 16-byte pieces (8 fp16) in the tensor
    uint32_t epoch;
};

__device__ __forceinline__ void store_release_sys(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kArThreads) oneshot_allreduce_kernel(const ArParams p)
{
    __shared__ int ok_s;
    __shared__ uint32_t epoch_s;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory"); // the addend comes from the launch before this one
    const int tid = threadIdx.x;
    if (tid == 0)
    {
        ok_s = 1;
        uint32_t e = p.epoch;
        if (e == 0)
        {
            // the launch before this one has completed (griddepcontrol.wait above), and nobody of this launch
            // writes the word before every CTA has read it (see the ticket below)
            e = __ldcg(p.header) + 1;
            if (e == 0)
                e = 2; // skip 0 ("take the counter") at the wrap, keeping the parity
        }
        epoch_s = e;
    }
    __syncthreads();
    const uint32_t epoch = epoch_s;
    // thread r talks to rank r: announce, then wait for its announcement
    if (tid < p.world && tid != p.rank)
    {
        store_release_sys(p.flags[tid] + blockIdx.x * kMaxRanks + p.rank, epoch);
        const uint32_t* mine = p.flags[p.rank] + blockIdx.x * kMaxRanks + tid;
        bool seen = false;
        for (uint32_t i = 0; i < kArSpin && !seen; i++)
        {
            seen = (int32_t)(load_acquire_sys(mine) - epoch) >= 0;
            if (!seen)
                __nanosleep(40);
        }
        if (!seen)
        {
            ok_s = 0;
            atomicExch(p.status, 1);
        }
    }
    __syncthreads();
    const uint32_t v = blockIdx.x * kArThreads + tid;
    if (ok_s && v < p.vecs)
    {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; j++)
            acc[j] = 0.f;
        uint4 part[kMaxRanks];
#pragma unroll
        for (int r = 0; r < kMaxRanks; r++)
            if (r < p.world) // never served from a stale line
                part[r] = __ldcv(reinterpret_cast<const uint4*>(p.bufs[r] + (epoch & 1u) * p.half_stride) + v);
#pragma unroll
        for (int r = 0; r < kMaxRanks; r++)
            if (r < p.world)
            {
                const __half2* h = reinterpret_cast<const __half2*>(&part[r]);
#pragma unroll
                for (int j = 0; j < 4; j++)
                {
                    const float2 f = __half22float2(h[j]);
                    acc[2 * j] += f.x, acc[2 * j + 1] += f.y;
                }
            }
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int j = 0; j < 4; j++)
            oh[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
        p.out[v] = o;
    }
    // device-counted calls: the CTA that arrives last moves the counter on (whatever happened above: a call that
    // gave up still counts, so that the ranks stay in step once their peers are back)
    if (p.epoch == 0 && tid == 0)
    {
        const uint32_t old = atomicAdd(p.header + 1, 1u);
        if (old == gridDim.x - 1)
        {
            __stcg(p.header + 1, 0u);
            __stcg(p.header, epoch);
        }
    }
}
} // namespace

namespace nnf
{
size_t allreduce_flag_bytes(size_t count)
{
    const size_t vecs = (count + 7) / 8;
    const size_t ctas = (vecs + kArThreads - 1) / kArThreads;
    return (kArHeaderWords + ctas * kMaxRanks) * sizeof(uint32_t); // header, then flags [CTA][sender]
}

int allreduce_launch(nnf_b200_ctx* ctx, cudaStream_t stream, int rank, int world, const void* const* bufs,
                     void* const* flags, size_t count, size_t half_stride, void* out, uint32_t epoch)
{
    ArParams p{};
    for (int r = 0; r < world; r++)
    {
        p.bufs[r] = static_cast<const char*>(bufs[r]);
        p.flags[r] = static_cast<uint32_t*>(flags[r]) + kArHeaderWords;
    }
    p.header = static_cast<uint32_t*>(flags[rank]);
    p.out = static_cast<uint4*>(out);
    p.status = ctx->dev_status;
    p.rank = rank, p.world = world;
    p.vecs = (uint32_t)(count / 8);
    p.epoch = epoch;
    p.half_stride = half_stride;
    const unsigned ctas = (p.vecs + kArThreads - 1) / kArThreads;
    (void)cudaGetLastError();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(kArThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    overlap_attribute(attr, &cfg.numAttrs);
    cfg.attrs = attr;
    cudaError_t e = cudaLaunchKernelEx(&cfg, oneshot_allreduce_kernel, p);
    if (e != cudaSuccess)
        return set_error(ctx, NNF_B200_ECUDA, std::string("oneshot_allreduce launch: ") + cudaGetErrorString(e));
    ctx->launches++;
    return NNF_B200_OK;
}
} // namespace nnf
