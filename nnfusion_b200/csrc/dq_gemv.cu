// Small-M (decode) dequantize-fused linear for sm_100a:  y[M,N] = epi(pro(x)[M,K] . dequant(W)[N,K]^T), M <= 16.
//
// Fused replacement of the reference's Convert -> Subtract -> Multiply element-wise kernels
// (src/nnfusion/core/kernels/cuda_gpu/kernels/elementwise.hpp:33-157, elementwise_fused.cpp:42-189)
// followed by the cuBLAS Dot (src/nnfusion/core/kernels/cuda_gpu/kernels/dot.cpp:27-372): the
// weights are read once, at their packed size, and never materialised in fp32.
//
// The kernel is HBM-bound.  Work decomposition:
//   * a weight row is cut into 128-byte "slices" (256 uint4 / 128 uint8 elements); warp w of a CTA owns
//     slice (split * warps + w) for the whole launch, so the activations it needs are loaded once and
//     live in registers as mma B-fragments;
//   * a CTA walks over 16-row tiles of W (persistent, round-robin); per tile every lane issues four
//     128-bit loads (rows g and g+8, two 64-byte halves of the slice), so each row is touched in
//     128 contiguous bytes per warp and 128*warps contiguous bytes per CTA.  The loads are cp.async copies
//     into a shared-memory ring several tiles deep; every thread later reads back exactly the 16-byte
//     chunks it copied itself, so the ring needs no barrier and holds the bytes in flight that an
//     HBM-bound kernel needs without spending registers on them;
//   * nibbles/bytes are turned into exact fp16 integers with one LOP3/PRMT each (the 0x6400 / 0x5400
//     exponent trick), the zero-point is removed exactly in fp16, and the products are accumulated in
//     fp32 by mma.sync.m16n8k16 with W as the 16-row operand and up to 8 batch rows as the 8-column
//     operand (the contraction index is permuted identically on both sides, so no data shuffling is
//     needed).  The group scale multiplies the fp32 partial sum once per 64-byte half, which keeps the
//     arithmetic equal to (q - zp) * scale accumulated in fp32;
//   * the partial sums of the CTA's warps are added in shared memory; with split-K each split stores
//     its tile sums into its own workspace slot and the split that arrives last (a counter per tile)
//     adds the slots in a fixed order, so results do not depend on timing.  No thread ever waits on
//     another CTA.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdio>

#include "nnf_internal.h"

namespace
{
constexpr int kMaxWarps = 8;
constexpr int kBatch = 8;    // row tiles whose results are kept in shared memory between flushes
constexpr int kMaxDepth = 8; // deepest load ring

struct GemvParams
{
    const uint8_t* wq[2];
    const void* scale[2];
    const uint8_t* zp[2];
    const void* x;
    const float* gain;
    const float* bias;
    void* y;
    float* ws_slots;
    unsigned* ws_count;
    int M, N, K;
    int group, G, zp_row_bytes, row_bytes;
    int units;  // 64-byte units per weight row
    int slices; // ceil(units / 2)
    int row_tiles, splits, ctas_per_split;
    int slices_base, slices_rem; // split s owns slices_base + (s < slices_rem) consecutive slices
    int x_f32, y_f32, scale_f32, rmsnorm, has_bias;
    int fast_params; // scale / zero-point tensors may be read as aligned 32-bit words
    int depth;       // ring depth (tiles in flight + 1)
    float eps;
    int slot_floats;
};

__device__ __forceinline__ void cp_async16(uint32_t smem, const void* g)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t smem, const void* g)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async_commit()
{
    asm volatile("cp.async.commit_group;" ::: "memory");
}
// Wait until at most `pending` of this thread's committed groups are still in flight.
__device__ __forceinline__ void cp_async_wait(int pending)
{
    switch (pending)
    {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
    }
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <uint32_t MASK, uint32_t ORV>
__device__ __forceinline__ uint32_t and_or(uint32_t w)
{
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(w), "n"(MASK), "n"(ORV)); // (a & b) | c
    return r;
}

__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b)
{
    uint32_t r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

__device__ __forceinline__ uint32_t pack_h2(__half a, __half b)
{
    return (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16);
}

template <int WBITS>
struct Fmt
{
    static constexpr int UE = (WBITS == 4) ? 128 : 64; // elements per 64-byte unit
    static constexpr int LE = UE / 4;                  // elements per lane per 16-byte load
    static constexpr int NF = LE / 2;                  // half2 fragments per load
};

// Shared-memory footprint, shared by host and device.
template <int MB, bool DUAL>
struct Smem
{
    static constexpr int SETS = DUAL ? 2 : 1;
    static constexpr int TILE_F = SETS * MB * 128; // floats of one tile result: [set][mb][lane][4]
    static constexpr int MPAD = 8 * MB;
    // per thread and ring slot: SETS * 4 weight chunks of 16 bytes + SETS * 2 (scale word, zp word) pairs
    static constexpr int SLOT_BYTES_PER_THREAD = SETS * (4 * 16 + 2 * 8);
    __host__ __device__ static size_t ring_bytes(int threads, int depth)
    {
        return (size_t)depth * threads * SLOT_BYTES_PER_THREAD;
    }
    __host__ __device__ static size_t total_bytes(int warps, int depth)
    {
        return ring_bytes(warps * 32, depth) +
               sizeof(float) * ((size_t)2 * warps * 2 * TILE_F + kBatch * TILE_F + warps * MPAD + MPAD) +
               sizeof(int) * kBatch;
    }
};

template <int WBITS, int MB, bool XSPLIT, bool DUAL>
__global__ void __launch_bounds__(kMaxWarps * 32, (MB == 1) ? 2 : 1) dq_gemv_kernel(const GemvParams p)
{
    using F = Fmt<WBITS>;
    using S = Smem<MB, DUAL>;
    constexpr int SETS = S::SETS;
    constexpr int XS = XSPLIT ? 2 : 1;
    constexpr int NF = F::NF;
    constexpr int TILE_F = S::TILE_F;
    constexpr int MPAD = S::MPAD;

    extern __shared__ uint4 smem_u4[];
    const int nthreads = blockDim.x;
    const int nwarps = nthreads >> 5;
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    // ring: [depth][SETS*4][nthreads] uint4 weights, then [depth][SETS*2][nthreads] uint2 {scale word, zp word}
    uint4* wring = smem_u4;
    uint2* pring = reinterpret_cast<uint2*>(wring + (size_t)p.depth * SETS * 4 * nthreads);
    float* red = reinterpret_cast<float*>(pring + (size_t)p.depth * SETS * 2 * nthreads); // [2][nwarps][2*TILE_F]
    float* res = red + 2 * nwarps * 2 * TILE_F;                                           // [kBatch][TILE_F]
    float* ss_w = res + kBatch * TILE_F;                                                  // [nwarps][MPAD]
    float* ss_cta = ss_w + nwarps * MPAD;                                                 // [MPAD]
    int* last_flag = reinterpret_cast<int*>(ss_cta + MPAD);                               // [kBatch]
    const uint32_t wring_s = (uint32_t)__cvta_generic_to_shared(wring);
    const uint32_t pring_s = (uint32_t)__cvta_generic_to_shared(pring);

    const int split = blockIdx.x / p.ctas_per_split;
    const int cta_in_split = blockIdx.x - split * p.ctas_per_split;
    const int my_slices = p.slices_base + (split < p.slices_rem ? 1 : 0);
    const int slice = split * p.slices_base + min(split, p.slices_rem) + warp;
    const bool has_slice = warp < my_slices;

    int unit_of[2], grp_of[2];
    bool unit_ok[2];
#pragma unroll
    for (int l = 0; l < 2; l++)
    {
        int u = 2 * slice + l;
        unit_ok[l] = has_slice && u < p.units;
        if (!unit_ok[l])
            u = 0;
        unit_of[l] = u;
        grp_of[l] = (u * F::UE) / p.group;
    }
    // Can the (scale, zero-point) of both halves of the slice be taken from one aligned 32-bit word per row?
    bool fast = p.fast_params != 0;
    {
        const int g0 = grp_of[0], g1 = grp_of[1];
        const bool same = g1 == g0, pair = (g1 == g0 + 1) && !(g0 & 1);
        const bool sc_ok = p.scale_f32 ? same : (same || (pair && !(p.G & 1)));
        const bool zp_ok = (WBITS == 4) ? (same || pair) : (same || (pair && !(p.G & 3)));
        fast = fast && sc_ok && zp_ok;
    }

    const int nsteps = (cta_in_split < p.row_tiles)
                           ? (p.row_tiles - cta_in_split + p.ctas_per_split - 1) / p.ctas_per_split
                           : 0;

    // ---------------------------------------------------------------- asynchronous loads of one row tile
    auto issue = [&](int step) {
        if (has_slice && step < nsteps)
        {
            const int slot = step % p.depth;
            const int rt = cta_in_split + step * p.ctas_per_split;
            int row[2];
            row[0] = min(rt * 16 + g, p.N - 1);
            row[1] = min(rt * 16 + g + 8, p.N - 1);
#pragma unroll
            for (int s = 0; s < SETS; s++)
#pragma unroll
                for (int h = 0; h < 2; h++)
                {
                    const uint8_t* wrow = p.wq[s] + (size_t)row[h] * p.row_bytes + t * 16;
#pragma unroll
                    for (int l = 0; l < 2; l++)
                        cp_async16(wring_s + (uint32_t)(((slot * SETS + s) * 4 + h * 2 + l) * nthreads + tid) * 16u,
                                   wrow + unit_of[l] * 64);
                    if (fast)
                    {
                        const uint32_t dst = pring_s + (uint32_t)(((slot * SETS + s) * 2 + h) * nthreads + tid) * 8u;
                        const size_t sidx = (size_t)row[h] * p.G + grp_of[0];
                        const char* sp = static_cast<const char*>(p.scale[s]);
                        cp_async4(dst, p.scale_f32 ? sp + sidx * 4 : sp + ((sidx * 2) & ~(size_t)3));
                        const size_t zoff = (WBITS == 4) ? (size_t)row[h] * p.zp_row_bytes + (grp_of[0] >> 1) : sidx;
                        cp_async4(dst + 4, p.zp[s] + (zoff & ~(size_t)3));
                    }
                }
        }
        cp_async_commit();
    };

    // Weights do not depend on the activations: start streaming before touching x.
    for (int j = 0; j < p.depth - 1; j++)
        issue(j);

    // ---------------------------------------------------------------- activations -> B fragments
    uint32_t xf[2][MB][XS][NF];
    float ss_local[MB];
#pragma unroll
    for (int mb = 0; mb < MB; mb++)
        ss_local[mb] = 0.f;
#pragma unroll
    for (int l = 0; l < 2; l++)
    {
        const int k0 = unit_of[l] * F::UE + t * F::LE;
#pragma unroll
        for (int mb = 0; mb < MB; mb++)
        {
            const int m = g + 8 * mb;
            float xv[F::LE];
            if (unit_ok[l] && m < p.M)
            {
                if (p.x_f32)
                {
                    const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(p.x) +
                                                                       (size_t)m * p.K + k0);
#pragma unroll
                    for (int j = 0; j < F::LE / 4; j++)
                    {
                        float4 v = __ldg(src + j);
                        xv[4 * j + 0] = v.x, xv[4 * j + 1] = v.y, xv[4 * j + 2] = v.z, xv[4 * j + 3] = v.w;
                    }
                }
                else
                {
                    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __half*>(p.x) +
                                                                     (size_t)m * p.K + k0);
#pragma unroll
                    for (int j = 0; j < F::LE / 8; j++)
                    {
                        uint4 v = __ldg(src + j);
                        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
                        for (int q = 0; q < 4; q++)
                        {
                            float2 f = __half22float2(h[q]);
                            xv[8 * j + 2 * q] = f.x, xv[8 * j + 2 * q + 1] = f.y;
                        }
                    }
                }
                if (p.rmsnorm)
                {
                    const float4* gsrc = reinterpret_cast<const float4*>(p.gain + k0);
#pragma unroll
                    for (int j = 0; j < F::LE / 4; j++)
                    {
                        float4 gv = __ldg(gsrc + j);
                        float* e = xv + 4 * j;
                        ss_local[mb] += e[0] * e[0] + e[1] * e[1] + e[2] * e[2] + e[3] * e[3];
                        e[0] *= gv.x, e[1] *= gv.y, e[2] *= gv.z, e[3] *= gv.w;
                    }
                }
            }
            else
            {
#pragma unroll
                for (int j = 0; j < F::LE; j++)
                    xv[j] = 0.f;
            }
            __half hi[F::LE], lo[F::LE];
#pragma unroll
            for (int j = 0; j < F::LE; j++)
            {
                hi[j] = __float2half_rn(xv[j]);
                lo[j] = XSPLIT ? __float2half_rn(xv[j] - __half2float(hi[j])) : __half();
            }
#pragma unroll
            for (int f = 0; f < NF; f++)
            {
                // Element order inside a fragment mirrors the order the weight unpacking produces:
                // uint4 word i yields pairs (n0,n4) (n1,n5) (n2,n6) (n3,n7); uint8 word i yields (b0,b1) (b2,b3).
                int e0, e1;
                if (WBITS == 4)
                {
                    e0 = 8 * (f >> 2) + (f & 3);
                    e1 = e0 + 4;
                }
                else
                {
                    e0 = 2 * f;
                    e1 = e0 + 1;
                }
                xf[l][mb][0][f] = pack_h2(hi[e0], hi[e1]);
                if (XSPLIT)
                    xf[l][mb][XS - 1][f] = pack_h2(lo[e0], lo[e1]);
            }
        }
    }

    // Sum of squares of this CTA's K range (RMSNorm prologue), reduced over the 4 lanes of a row and
    // over the warps.  Applied to the final sums as rsqrt(mean + eps).
    if (p.rmsnorm)
    {
#pragma unroll
        for (int mb = 0; mb < MB; mb++)
        {
            float v = ss_local[mb];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if (t == 0)
                ss_w[warp * MPAD + g + 8 * mb] = v;
        }
        __syncthreads();
        if (tid < MPAD)
        {
            float v = 0.f;
            for (int w = 0; w < nwarps; w++)
                v += ss_w[w * MPAD + tid];
            ss_cta[tid] = v;
        }
        __syncthreads();
    }

    // ---------------------------------------------------------------- arithmetic on one landed row tile
    float tot[SETS][MB][4];
    auto compute = [&](int step) {
        const int slot = step % p.depth;
#pragma unroll
        for (int s = 0; s < SETS; s++)
#pragma unroll
            for (int mb = 0; mb < MB; mb++)
#pragma unroll
                for (int c = 0; c < 4; c++)
                    tot[s][mb][c] = 0.f;
#pragma unroll
        for (int s = 0; s < SETS; s++)
        {
            // (scale, zero-point) of rows g / g+8 for both halves of the slice
            float sc[2][2];
            uint32_t zq[2][2];
            if (fast)
            {
#pragma unroll
                for (int h = 0; h < 2; h++)
                {
                    const uint2 pw = pring[((slot * SETS + s) * 2 + h) * nthreads + tid];
                    const int row = min((cta_in_split + step * p.ctas_per_split) * 16 + g + 8 * h, p.N - 1);
                    const size_t sidx = (size_t)row * p.G + grp_of[0];
                    const size_t zoff = (WBITS == 4) ? (size_t)row * p.zp_row_bytes + (grp_of[0] >> 1) : sidx;
#pragma unroll
                    for (int l = 0; l < 2; l++)
                    {
                        const int dg = grp_of[l] - grp_of[0];
                        if (p.scale_f32)
                            sc[l][h] = __uint_as_float(pw.x);
                        else
                            sc[l][h] = __half2float(
                                __ushort_as_half((unsigned short)(pw.x >> (16 * (int)((sidx + dg) & 1)))));
                        if (WBITS == 4)
                            zq[l][h] = (pw.y >> (8 * (int)(zoff & 3) + 4 * (grp_of[l] & 1))) & 0xF;
                        else
                            zq[l][h] = (pw.y >> (8 * (int)((zoff + dg) & 3))) & 0xFF;
                    }
                }
            }
            else
            {
#pragma unroll
                for (int h = 0; h < 2; h++)
                {
                    const int row = min((cta_in_split + step * p.ctas_per_split) * 16 + g + 8 * h, p.N - 1);
#pragma unroll
                    for (int l = 0; l < 2; l++)
                    {
                        const size_t sidx = (size_t)row * p.G + grp_of[l];
                        sc[l][h] = p.scale_f32 ? __ldg(static_cast<const float*>(p.scale[s]) + sidx)
                                               : __half2float(__ldg(static_cast<const __half*>(p.scale[s]) + sidx));
                        if (WBITS == 4)
                            zq[l][h] = (__ldg(p.zp[s] + (size_t)row * p.zp_row_bytes + (grp_of[l] >> 1)) >>
                                        (4 * (grp_of[l] & 1))) &
                                       0xF;
                        else
                            zq[l][h] = __ldg(p.zp[s] + sidx);
                    }
                }
            }
#pragma unroll
            for (int l = 0; l < 2; l++)
            {
                float acc[MB][4];
#pragma unroll
                for (int mb = 0; mb < MB; mb++)
#pragma unroll
                    for (int c = 0; c < 4; c++)
                        acc[mb][c] = 0.f;
                uint32_t zA[2], zB[2]; // fp16x2 constants holding (offset + zero-point)
#pragma unroll
                for (int h = 0; h < 2; h++)
                {
                    zA[h] = (0x6400u | zq[l][h]) * 0x00010001u; // 1024 + zp
                    zB[h] = (WBITS == 4) ? (0x5400u | (zq[l][h] << 4)) * 0x00010001u : zA[h]; // 64 + zp
                }
                const uint4 w_lo = wring[((slot * SETS + s) * 4 + 0 * 2 + l) * nthreads + tid];
                const uint4 w_hi = wring[((slot * SETS + s) * 4 + 1 * 2 + l) * nthreads + tid];
                const uint32_t wl[4] = {w_lo.x, w_lo.y, w_lo.z, w_lo.w};
                const uint32_t wh[4] = {w_hi.x, w_hi.y, w_hi.z, w_hi.w};
#pragma unroll
                for (int i = 0; i < 4; i++)
                {
                    uint32_t a[2][4]; // [row half][pair]
#pragma unroll
                    for (int h = 0; h < 2; h++)
                    {
                        const uint32_t w = h ? wh[i] : wl[i];
                        if (WBITS == 4)
                        {
                            const uint32_t w8 = w >> 8;
                            a[h][0] = hsub2_u32(and_or<0x000F000Fu, 0x64006400u>(w), zA[h]);  // n0, n4
                            a[h][1] = hsub2_u32(and_or<0x00F000F0u, 0x54005400u>(w), zB[h]);  // n1, n5
                            a[h][2] = hsub2_u32(and_or<0x000F000Fu, 0x64006400u>(w8), zA[h]); // n2, n6
                            a[h][3] = hsub2_u32(and_or<0x00F000F0u, 0x54005400u>(w8), zB[h]); // n3, n7
                        }
                        else
                        {
                            a[h][0] = hsub2_u32(__byte_perm(w, 0x64646464u, 0x4140), zA[h]); // b0, b1
                            a[h][1] = hsub2_u32(__byte_perm(w, 0x64646464u, 0x4342), zA[h]); // b2, b3
                        }
                    }
                    constexpr int PAIRS = (WBITS == 4) ? 4 : 2; // half2 pairs per word
#pragma unroll
                    for (int q = 0; q < PAIRS; q += 2)
                    {
                        const int f = i * PAIRS + q;
#pragma unroll
                        for (int mb = 0; mb < MB; mb++)
#pragma unroll
                            for (int xs = 0; xs < XS; xs++)
                                mma16816(acc[mb], a[0][q], a[1][q], a[0][q + 1], a[1][q + 1], xf[l][mb][xs][f],
                                         xf[l][mb][xs][f + 1]);
                    }
                }
#pragma unroll
                for (int mb = 0; mb < MB; mb++)
                {
                    tot[s][mb][0] = fmaf(sc[l][0], acc[mb][0], tot[s][mb][0]);
                    tot[s][mb][1] = fmaf(sc[l][0], acc[mb][1], tot[s][mb][1]);
                    tot[s][mb][2] = fmaf(sc[l][1], acc[mb][2], tot[s][mb][2]);
                    tot[s][mb][3] = fmaf(sc[l][1], acc[mb][3], tot[s][mb][3]);
                }
            }
        }
    };

    // Final value of one output element from its summed parts.
    auto finish = [&](float a0, float a1, float ssum, int n) -> float {
        float r = 1.f;
        if (p.rmsnorm)
            r = 1.0f / sqrtf(ssum / (float)p.K + p.eps);
        float v = a0 * r;
        if (DUAL)
        {
            const float u = a1 * r;
            const float sg = 1.0f / (1.0f + expf(-v));
            v = v * sg * u;
        }
        if (p.has_bias)
            v += __ldg(p.bias + n);
        return v;
    };
    auto store_y = [&](int m, int n, float v) {
        if (p.y_f32)
            static_cast<float*>(p.y)[(size_t)m * p.N + n] = v;
        else
            static_cast<__half*>(p.y)[(size_t)m * p.N + n] = __float2half_rn(v);
    };
    // Index o in [0, MB*128) of a tile result <-> (row in tile, batch row m).
    auto decode = [&](int o, int& row, int& m) {
        const int mb = o >> 7, ln = (o >> 2) & 31, c = o & 3;
        row = (ln >> 2) + 8 * (c >> 1);
        m = 8 * mb + 2 * (ln & 3) + (c & 1);
    };

    // Flush the tile results held in shared memory for steps [first, first + count).
    auto flush = [&](int first, int count) {
        __syncthreads();
        if (p.splits == 1)
        {
            for (int idx = tid; idx < count * MB * 128; idx += nthreads)
            {
                const int j = idx / (MB * 128), o = idx - j * (MB * 128);
                int row, m;
                decode(o, row, m);
                const int n = (cta_in_split + (first + j) * p.ctas_per_split) * 16 + row;
                if (m < p.M && n < p.N)
                {
                    const float* r = res + j * TILE_F;
                    store_y(m, n, finish(r[o], DUAL ? r[MB * 128 + o] : 0.f, p.rmsnorm ? ss_cta[m] : 0.f, n));
                }
            }
        }
        else
        {
            // 1. publish this split's partial sums (and its share of the sum of squares)
            for (int idx = tid; idx < count * p.slot_floats; idx += nthreads)
            {
                const int j = idx / p.slot_floats, o = idx - j * p.slot_floats;
                const int rt = cta_in_split + (first + j) * p.ctas_per_split;
                const float v = (o < TILE_F) ? res[j * TILE_F + o] : (p.rmsnorm ? ss_cta[o - TILE_F] : 0.f);
                __stcg(p.ws_slots + ((size_t)split * p.row_tiles + rt) * p.slot_floats + o, v);
            }
            __threadfence();
            __syncthreads();
            // 2. one arrival per tile; the last split to arrive owns the tile's final sum
            if (tid < count)
            {
                const int rt = cta_in_split + (first + tid) * p.ctas_per_split;
                const unsigned old = atomicAdd(p.ws_count + rt, 1u);
                last_flag[tid] = (old == (unsigned)(p.splits - 1));
                if (last_flag[tid])
                    p.ws_count[rt] = 0u; // leave the counter zeroed for the next call
            }
            __syncthreads();
            __threadfence();
            // 3. fixed-order sum over the splits
            for (int idx = tid; idx < count * MB * 128; idx += nthreads)
            {
                const int j = idx / (MB * 128), o = idx - j * (MB * 128);
                if (!last_flag[j])
                    continue;
                int row, m;
                decode(o, row, m);
                const int rt = cta_in_split + (first + j) * p.ctas_per_split;
                const int n = rt * 16 + row;
                if (m < p.M && n < p.N)
                {
                    float a0 = 0.f, a1 = 0.f, ssum = 0.f;
                    for (int s = 0; s < p.splits; s++)
                    {
                        const float* slot = p.ws_slots + ((size_t)s * p.row_tiles + rt) * p.slot_floats;
                        a0 += __ldcg(slot + o);
                        if (DUAL)
                            a1 += __ldcg(slot + MB * 128 + o);
                        if (p.rmsnorm)
                            ssum += __ldcg(slot + TILE_F + m);
                    }
                    store_y(m, n, finish(a0, a1, ssum, n));
                }
            }
        }
        __syncthreads();
    };

    // ---------------------------------------------------------------- main loop: two row tiles per barrier
    for (int step = 0; step < nsteps; step += 2)
    {
        const int pair_n = min(2, nsteps - step);
        float* my = red + (((step >> 1) & 1) * nwarps + warp) * 2 * TILE_F;
        for (int j = 0; j < pair_n; j++)
        {
            issue(step + j + p.depth - 1);
            cp_async_wait(p.depth - 1);
            if (has_slice)
            {
                compute(step + j);
#pragma unroll
                for (int s = 0; s < SETS; s++)
#pragma unroll
                    for (int mb = 0; mb < MB; mb++)
                        reinterpret_cast<float4*>(my + j * TILE_F)[(s * MB + mb) * 32 + lane] =
                            make_float4(tot[s][mb][0], tot[s][mb][1], tot[s][mb][2], tot[s][mb][3]);
            }
            else
            {
#pragma unroll
                for (int q = 0; q < SETS * MB; q++)
                    reinterpret_cast<float4*>(my + j * TILE_F)[q * 32 + lane] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        __syncthreads();
        const float* rb = red + ((step >> 1) & 1) * nwarps * 2 * TILE_F;
        for (int o = tid; o < pair_n * TILE_F; o += nthreads)
        {
            const int j = o / TILE_F, oo = o - j * TILE_F;
            float v = 0.f;
            for (int w = 0; w < nwarps; w++)
                v += rb[w * 2 * TILE_F + j * TILE_F + oo];
            res[((step + j) % kBatch) * TILE_F + oo] = v;
        }
        const int last = step + pair_n - 1;
        if ((last % kBatch) == kBatch - 1 || last == nsteps - 1)
            flush(last - (last % kBatch), (last % kBatch) + 1);
    }
    cp_async_wait(0);
}

// Raise the kernel's dynamic shared-memory limit (monotonically: the attribute is a plain setter).
template <int WBITS, int MB, bool XSPLIT, bool DUAL>
cudaError_t ensure_smem(size_t smem)
{
    static size_t configured = 48 * 1024;
    if (smem <= configured)
        return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(dq_gemv_kernel<WBITS, MB, XSPLIT, DUAL>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
        configured = smem;
    return e;
}

template <int WBITS, int MB, bool XSPLIT, bool DUAL>
cudaError_t launch(const GemvParams& p, int warps, int grid, cudaStream_t stream)
{
    const size_t smem = Smem<MB, DUAL>::total_bytes(warps, p.depth);
    cudaError_t e = ensure_smem<WBITS, MB, XSPLIT, DUAL>(smem);
    if (e != cudaSuccess)
        return e;
    (void)cudaGetLastError(); // do not inherit a stale error left behind by an unrelated earlier call
    dq_gemv_kernel<WBITS, MB, XSPLIT, DUAL><<<grid, warps * 32, smem, stream>>>(p);
    return cudaGetLastError();
}

template <int WBITS, int MB, bool XSPLIT, bool DUAL>
int occupancy(int warps, int depth)
{
    static int cache[kMaxWarps + 1][kMaxDepth + 1]; // 0 = not queried yet
    if (cache[warps][depth] > 0)
        return cache[warps][depth];
    const size_t smem = Smem<MB, DUAL>::total_bytes(warps, depth);
    if (ensure_smem<WBITS, MB, XSPLIT, DUAL>(smem) != cudaSuccess)
        return 0;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, dq_gemv_kernel<WBITS, MB, XSPLIT, DUAL>, warps * 32,
                                                      smem) != cudaSuccess)
        return 0;
    cache[warps][depth] = n;
    return n;
}

#define NNF_GEMV_FOR_EACH_VARIANT(X)                                                                              \
    X(4, 1, false, false)                                                                                         \
    X(4, 1, false, true)                                                                                          \
    X(4, 1, true, false)                                                                                          \
    X(4, 1, true, true)                                                                                           \
    X(4, 2, false, false)                                                                                         \
    X(4, 2, false, true)                                                                                          \
    X(8, 1, false, false)                                                                                         \
    X(8, 1, false, true)                                                                                          \
    X(8, 1, true, false)                                                                                          \
    X(8, 1, true, true)                                                                                           \
    X(8, 2, false, false)                                                                                         \
    X(8, 2, false, true)                                                                                          \
    X(8, 2, true, false)                                                                                          \
    X(8, 2, true, true)

cudaError_t dispatch(int wbits, const nnf::GemvPlan& plan, const GemvParams& p, int grid, cudaStream_t stream)
{
#define NNF_X(WB, MBV, XSP, DU)                                                                                   \
    if (wbits == WB && plan.mb == MBV && plan.xsplit == XSP && plan.dual == DU)                                   \
        return launch<WB, MBV, XSP, DU>(p, plan.warps, grid, stream);
    NNF_GEMV_FOR_EACH_VARIANT(NNF_X)
#undef NNF_X
    return cudaErrorInvalidValue;
}

// Resident CTAs per SM of the variant a plan selects (0 when it cannot be queried, e.g. without a device).
int query_occupancy(int wbits, const nnf::GemvPlan& plan)
{
#define NNF_X(WB, MBV, XSP, DU)                                                                                   \
    if (wbits == WB && plan.mb == MBV && plan.xsplit == XSP && plan.dual == DU)                                   \
        return occupancy<WB, MBV, XSP, DU>(plan.warps, plan.depth);
    NNF_GEMV_FOR_EACH_VARIANT(NNF_X)
#undef NNF_X
    return 0;
}

size_t smem_for(const nnf::GemvPlan& plan)
{
    if (plan.mb == 1)
        return plan.dual ? Smem<1, true>::total_bytes(plan.warps, plan.depth)
                         : Smem<1, false>::total_bytes(plan.warps, plan.depth);
    return plan.dual ? Smem<2, true>::total_bytes(plan.warps, plan.depth)
                     : Smem<2, false>::total_bytes(plan.warps, plan.depth);
}
} // namespace

namespace nnf
{
int gemv_configure(nnf_b200_ctx*)
{
    return NNF_B200_OK;
}

int gemv_plan(const nnf_b200_ctx* ctx, const nnf_b200_linear_desc& d, GemvPlan* plan, std::string* why)
{
    const int ue = (d.w_bits == 4) ? 128 : 64;
    const int group = d.group_size > 0 ? d.group_size : d.K;
    if (d.M < 1 || d.M > 16)
    {
        *why = "small-M kernel handles 1 <= M <= 16";
        return NNF_B200_ENOTSUP;
    }
    if (d.K % ue != 0 || group % ue != 0 || d.K % group != 0)
    {
        *why = "K and group_size must be multiples of " + std::to_string(ue) + " and K a multiple of group_size";
        return NNF_B200_ENOTSUP;
    }
    GemvPlan pl;
    pl.mb = d.M > 8 ? 2 : 1;
    pl.dual = d.epilogue == NNF_B200_EPILOGUE_SILU_MUL;
    // fp32 activations are carried as fp16 hi + lo where the register budget allows it
    pl.xsplit = d.x_dtype == NNF_B200_F32 && !(d.w_bits == 4 && pl.mb == 2);
    pl.row_tiles = (d.N + 15) / 16;
    const int units = d.K / ue;
    pl.slices = (units + 1) / 2;
    // Split K so that every CTA has at most kMaxWarps slices, spread evenly (sizes differ by at most one).
    pl.splits = (pl.slices + kMaxWarps - 1) / kMaxWarps;
    if (d.split_k > 0)
    {
        if ((pl.slices + d.split_k - 1) / d.split_k > kMaxWarps)
        {
            *why = "split_k too small: more than " + std::to_string(kMaxWarps) + " slices of 128 bytes per split";
            return NNF_B200_EINVAL;
        }
        pl.splits = std::min(d.split_k, pl.slices);
    }
    pl.warps = (pl.slices + pl.splits - 1) / pl.splits;
    // Ring depth: as deep as lets two CTAs share an SM's shared memory (one for the 16-row-batch variants).
    const int smem_cap = ctx ? ctx->smem_optin : 227 * 1024;
    const int want_ctas = pl.mb == 1 ? 2 : 1;
    pl.depth = 2;
    for (int depth = kMaxDepth; depth >= 2; depth--)
    {
        pl.depth = depth;
        if ((int)smem_for(pl) + 1024 <= smem_cap / want_ctas)
            break;
    }
    const int sms = ctx ? ctx->sm_count : 148;
    int resident = ctx ? query_occupancy(d.w_bits, pl) : 0;
    if (resident <= 0)
        resident = 1;
    int per_split = std::max(1, (sms * resident) / pl.splits);
    per_split = std::min(per_split, pl.row_tiles);
    pl.ctas_per_split = per_split;
    const int sets = pl.dual ? 2 : 1;
    pl.slot_floats = (size_t)sets * pl.mb * 128 + 8 * pl.mb;
    pl.workspace_bytes = 0;
    if (pl.splits > 1)
    {
        const size_t cnt = ((size_t)pl.row_tiles * sizeof(unsigned) + 255) / 256 * 256;
        pl.workspace_bytes = cnt + (size_t)pl.splits * pl.row_tiles * pl.slot_floats * sizeof(float);
    }
    *plan = pl;
    return NNF_B200_OK;
}

int gemv_launch(nnf_b200_ctx* ctx, cudaStream_t stream, const nnf_b200_linear_desc& d, const GemvPlan& plan,
                const void* x, const nnf_b200_qweight* w, const nnf_b200_qweight* w2, const void* gain,
                const void* bias, void* y, void* workspace)
{
    GemvParams p{};
    const int ue = (d.w_bits == 4) ? 128 : 64;
    p.wq[0] = static_cast<const uint8_t*>(w->wq);
    p.scale[0] = w->scale;
    p.zp[0] = static_cast<const uint8_t*>(w->zp);
    if (plan.dual)
    {
        p.wq[1] = static_cast<const uint8_t*>(w2->wq);
        p.scale[1] = w2->scale;
        p.zp[1] = static_cast<const uint8_t*>(w2->zp);
    }
    p.x = x;
    p.gain = static_cast<const float*>(gain);
    p.bias = static_cast<const float*>(bias);
    p.y = y;
    p.M = d.M, p.N = d.N, p.K = d.K;
    p.group = d.group_size > 0 ? d.group_size : d.K;
    p.G = d.K / p.group;
    p.zp_row_bytes = (d.w_bits == 4) ? (p.G + 1) / 2 : p.G;
    p.row_bytes = (d.w_bits == 4) ? d.K / 2 : d.K;
    p.units = d.K / ue;
    p.slices = plan.slices;
    p.row_tiles = plan.row_tiles;
    p.splits = plan.splits;
    p.ctas_per_split = plan.ctas_per_split;
    p.slices_base = plan.slices / plan.splits;
    p.slices_rem = plan.slices % plan.splits;
    p.x_f32 = d.x_dtype == NNF_B200_F32;
    p.y_f32 = d.y_dtype == NNF_B200_F32;
    p.scale_f32 = d.scale_dtype == NNF_B200_F32;
    p.rmsnorm = d.prologue == NNF_B200_PROLOGUE_RMSNORM;
    p.has_bias = bias != nullptr;
    p.eps = d.rms_eps;
    p.depth = plan.depth;
    p.slot_floats = (int)plan.slot_floats;
    // Reading the quantisation parameters as aligned 32-bit words must stay inside the tensors.
    const size_t scale_bytes = (size_t)d.N * p.G * (p.scale_f32 ? 4 : 2);
    const size_t zp_bytes = (size_t)d.N * p.zp_row_bytes;
    auto word_ok = [](const void* ptr, size_t bytes) {
        return (reinterpret_cast<uintptr_t>(ptr) & 3u) == 0 && (bytes & 3u) == 0;
    };
    p.fast_params = word_ok(w->scale, scale_bytes) && word_ok(w->zp, zp_bytes) &&
                    (!plan.dual || (word_ok(w2->scale, scale_bytes) && word_ok(w2->zp, zp_bytes)));
    if (plan.splits > 1)
    {
        const size_t cnt = ((size_t)plan.row_tiles * sizeof(unsigned) + 255) / 256 * 256;
        p.ws_count = static_cast<unsigned*>(workspace);
        p.ws_slots = reinterpret_cast<float*>(static_cast<char*>(workspace) + cnt);
    }
    const int grid = plan.splits * plan.ctas_per_split;
    cudaError_t e = dispatch(d.w_bits, plan, p, grid, stream);
    if (e != cudaSuccess)
        return set_error(ctx, NNF_B200_ECUDA,
                         std::string("dq_gemv launch: ") + cudaGetErrorString(e) + " (grid " + std::to_string(grid) +
                             ", warps " + std::to_string(plan.warps) + ", depth " + std::to_string(plan.depth) +
                             ", smem " + std::to_string(smem_for(plan)) + ")");
    ctx->launches++;
    return NNF_B200_OK;
}
} // namespace nnf
