// Small-M (decode) dequantize-fused linear for sm_100a:  y[M,N] = epi(pro(x)[M,K] . dequant(W)[N,K]^T), M <= 16.
//
// Fused replacement of the reference's Convert -> Subtract -> Multiply element-wise kernels
// (src/nnfusion/core/kernels/cuda_gpu/kernels/elementwise.hpp:33-157, elementwise_fused.cpp:42-189)
// followed by the cuBLAS Dot (src/nnfusion/core/kernels/cuda_gpu/kernels/dot.cpp:27-372): the
// weights are read once, at their packed size, and never materialised in fp32.
//
// The kernel is HBM-bound and, next to that, bound by instruction issue; its shape follows from both:
//   * a weight row is cut into 128-byte "slices" (256 uint4 / 128 uint8 elements).  Warp w of a CTA owns slice
//     (first slice of the CTA's K range + w) for the whole launch, so the activations it needs are loaded and
//     converted once and live in registers as mma B fragments;
//   * CTAs are persistent: CTA c of a K split walks over the 16-row tiles c, c + P, c + 2P ...  The weight tiles
//     arrive by TMA (one thread issues a 16-row x 128-byte box per warp and tile, 128-byte swizzle, completion
//     counted on an mbarrier per ring slot) into a shared-memory ring several tiles deep, which holds the bytes in
//     flight that an HBM-bound kernel needs without spending registers or load instructions on them; scales and
//     zero-points are prefetched two tiles ahead in registers;
//   * nibbles/bytes become exact fp16 integers with one LOP3/PRMT per pair (the 0x6400 / 0x5400 exponent trick)
//     and feed mma.sync.m16n8k16 with W as the 16-row operand and up to 8 batch rows as the 8-column operand (the
//     contraction index is permuted identically on both sides, so nothing is shuffled); accumulation is fp32 and
//     the group scale multiplies the fp32 sum of each 64-byte unit, i.e. sum((q - zp) * x) * scale;
//   * the partial sums of the CTA's warps are added in shared memory in a fixed order, once per two tiles; with
//     split-K each split stores its tile sums into its own workspace slot and the split that arrives last (a
//     counter per tile) adds the slots in a fixed order, so results are bitwise repeatable.  Nothing ever waits on
//     another CTA, and every mbarrier wait is bounded.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdio>

#include "nnf_internal.h"
#include "sm100_ptx.cuh"

namespace
{
using namespace nnf::ptx;

constexpr int kMaxWarps = 16;
constexpr int kBatch = 8;            // row tiles whose results are kept in shared memory between flushes
constexpr int kMaxDepth = 8;         // deepest load ring
constexpr int kTileBytes = 16 * 128; // one warp's weight tile: 16 rows x 128 bytes

struct GemvParams
{
    const void* scale[2];
    const uint8_t* zp[2];
    const void* x;
    const float* gain;
    const float* bias;
    void* y;
    float* ws_slots;
    unsigned* ws_count;
    int* status; // device status word: set to 1 when a bounded wait gave up
    int M, N, K;
    int group, G, zp_row_bytes;
    int units;  // 64-byte units per weight row
    int slices; // ceil(units / 2)
    int row_tiles, splits, ctas_per_split;
    int x_f32, y_f32, scale_f32, rmsnorm, has_bias;
    int fast_params; // scale / zero-point tensors may be read as aligned 32-bit words
    int depth;       // ring depth in row tiles
    float eps;
    int slot_floats;
};

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
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
    static constexpr int LE = UE / 4;                  // elements per lane per 16-byte chunk
    static constexpr int NF = LE / 2;                  // half2 fragments per chunk
};

// Shared-memory footprint, shared by host and device.
template <int MB, bool DUAL>
struct Smem
{
    static constexpr int SETS = DUAL ? 2 : 1;
    static constexpr int TILE_F = SETS * MB * 128; // floats of one tile result: [set][mb][lane][4]
    static constexpr int MPAD = 8 * MB;
    __host__ __device__ static size_t ring_bytes(int warps, int depth)
    {
        return (size_t)depth * SETS * warps * kTileBytes;
    }
    __host__ __device__ static size_t total_bytes(int warps, int depth)
    {
        return 1024 /* alignment slack */ + ring_bytes(warps, depth) + 8 * kMaxDepth +
               sizeof(float) * ((size_t)2 * warps * 2 * TILE_F + kBatch * TILE_F + warps * MPAD + MPAD) +
               sizeof(int) * kBatch;
    }
};

// EXACT = true : zero-points are removed from the fp16 integers before the multiply (bit-exact integers into the
//                tensor core).
// EXACT = false: the tensor core multiplies x by (offset + q) and the offset and zero-point are taken out of the
//                fp32 sum afterwards, acc - (C1 + zp * C2), with C1 = sum(offset_k * x_k), C2 = sum(x_k) over the
//                64-byte unit.  Same fp32 accumulation, about 40 % fewer unpack instructions.
template <int WBITS, int MB, bool XSPLIT, bool DUAL, bool EXACT>
__global__ void __launch_bounds__(kMaxWarps * 32, 1)
    dq_gemv_kernel(const GemvParams p, const __grid_constant__ CUtensorMap tmap0,
                   const __grid_constant__ CUtensorMap tmap1)
{
    using F = Fmt<WBITS>;
    using S = Smem<MB, DUAL>;
    constexpr int SETS = S::SETS;
    constexpr int XS = XSPLIT ? 2 : 1;
    constexpr int NF = F::NF;
    constexpr int TILE_F = S::TILE_F;
    constexpr int MPAD = S::MPAD;

    extern __shared__ uint8_t smem_raw[];
    const int nthreads = blockDim.x;
    const int nwarps = nthreads >> 5;
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    // ring (1024-byte aligned: the TMA 128-byte swizzle is a function of the shared-memory address):
    //   [depth][SETS][nwarps] tiles of 16 rows x 128 bytes
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(ring + S::ring_bytes(nwarps, p.depth)); // [kMaxDepth]
    float* red = reinterpret_cast<float*>(full_bar + kMaxDepth);                             // [2][nwarps][2*TILE_F]
    float* res = red + 2 * nwarps * 2 * TILE_F;                                              // [kBatch][TILE_F]
    float* ss_w = res + kBatch * TILE_F;                                                     // [nwarps][MPAD]
    float* ss_cta = ss_w + nwarps * MPAD;                                                    // [MPAD]
    int* last_flag = reinterpret_cast<int*>(ss_cta + MPAD);                                  // [kBatch]
    const uint32_t ring_s = smem_u32(ring);
    const uint32_t bar_s = smem_u32(full_bar);

    const int split = blockIdx.x / p.ctas_per_split;
    const int cta_in_split = blockIdx.x - split * p.ctas_per_split;
    const int sb = p.slices / p.splits, sr = p.slices % p.splits; // K ranges differ by at most one slice
    const int my_slices = sb + (split < sr ? 1 : 0);
    const int slice0 = split * sb + min(split, sr);
    const int slice = slice0 + warp;
    const bool has_slice = warp < my_slices;
    const int nsteps = (cta_in_split < p.row_tiles)
                           ? (p.row_tiles - cta_in_split + p.ctas_per_split - 1) / p.ctas_per_split
                           : 0;

    // ---------------------------------------------------------------- TMA producer (thread 0)
    // One 16-row x 128-byte box per (weight set, slice) and row tile, all counted on the slot's barrier.
    auto produce = [&](int step) {
        if (step < nsteps)
        {
            const int slot = step % p.depth;
            const uint32_t bar = bar_s + 8 * slot;
            const int row0 = (cta_in_split + step * p.ctas_per_split) * 16;
            mbar_arrive_expect_tx(bar, (uint32_t)(SETS * my_slices * kTileBytes));
            for (int w = 0; w < my_slices; w++)
            {
                tma_load_2d(ring_s + (uint32_t)(((slot * SETS + 0) * nwarps + w) * kTileBytes), &tmap0, bar,
                            (slice0 + w) * 128, row0);
                if (DUAL)
                    tma_load_2d(ring_s + (uint32_t)(((slot * SETS + 1) * nwarps + w) * kTileBytes), &tmap1, bar,
                                (slice0 + w) * 128, row0);
            }
        }
    };
    if (tid == 0)
    {
        for (int i = 0; i < p.depth; i++)
            mbar_init(bar_s + 8 * i, 1);
        fence_barrier_init();
        // Weights do not depend on the activations: start streaming before anybody touches x.  (The arrive on
        // the barrier waits for this thread's earlier loads, so nothing is loaded ahead of it.)
        for (int i = 0; i < p.depth; i++)
            produce(i);
    }

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

    // ---------------------------------------------------------------- quantisation parameters of one row tile
    struct PReg
    {
        uint32_t sw[SETS][2]; // word holding the scale(s) of row g / g+8
        uint32_t zw[SETS][2]; // word holding the zero-point(s)
    };
    auto row_of = [&](int step, int h) { return min((cta_in_split + step * p.ctas_per_split) * 16 + g + 8 * h, p.N - 1); };
    auto load_params = [&](PReg& r, int step) {
        if (fast && has_slice && step < nsteps)
        {
#pragma unroll
            for (int h = 0; h < 2; h++)
            {
                const int row = row_of(step, h);
                const size_t sidx = (size_t)row * p.G + grp_of[0];
                const size_t zoff = (WBITS == 4) ? (size_t)row * p.zp_row_bytes + (grp_of[0] >> 1) : sidx;
#pragma unroll
                for (int s = 0; s < SETS; s++)
                {
                    const char* sp = static_cast<const char*>(p.scale[s]);
                    r.sw[s][h] = __ldg(reinterpret_cast<const uint32_t*>(
                        p.scale_f32 ? sp + sidx * 4 : sp + ((sidx * 2) & ~(size_t)3)));
                    r.zw[s][h] = __ldg(reinterpret_cast<const uint32_t*>(p.zp[s] + (zoff & ~(size_t)3)));
                }
            }
        }
    };
    PReg pr[3]; // tiles step, step + 1, step + 2
    load_params(pr[0], 0);
    load_params(pr[1], 1);

    // ---------------------------------------------------------------- activations -> B fragments in registers
    uint32_t xf[2][MB][XS][NF];
    float c1[2][MB][2], c2[2][MB][2]; // offset / zero-point corrections for accumulator columns 2t, 2t+1
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
            float se = 0.f, so = 0.f; // sums of what the tensor core will see, even / odd element positions
#pragma unroll
            for (int j = 0; j < F::LE; j++)
            {
                hi[j] = __float2half_rn(xv[j]);
                float seen = __half2float(hi[j]);
                if (XSPLIT)
                {
                    lo[j] = __float2half_rn(xv[j] - seen);
                    seen += __half2float(lo[j]);
                }
                if (j & 1)
                    so += seen;
                else
                    se += seen;
            }
#pragma unroll
            for (int f = 0; f < NF; f++)
            {
                // Element order inside a fragment mirrors the order the weight unpacking produces:
                // uint4 word i yields pairs (n0,n4) (n1,n5) (n2,n6) (n3,n7); uint8 word i yields (b0,b1) (b2,b3).
                const int e0 = (WBITS == 4) ? 8 * (f >> 2) + (f & 3) : 2 * f;
                const int e1 = (WBITS == 4) ? e0 + 4 : e0 + 1;
                xf[l][mb][0][f] = pack_h2(hi[e0], hi[e1]);
                if (XSPLIT)
                    xf[l][mb][XS - 1][f] = pack_h2(lo[e0], lo[e1]);
            }
            if (!EXACT)
            {
                // uint4: even positions carry offset 1024 (bits 0-3 of a half), odd positions 64 (bits 4-7);
                // uint8: every position carries 1024.
                float a1 = (WBITS == 4) ? 1024.f * se + 64.f * so : 1024.f * (se + so);
                float a2 = se + so;
                a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
                a2 += __shfl_xor_sync(0xffffffffu, a2, 1);
                a1 += __shfl_xor_sync(0xffffffffu, a1, 2);
                a2 += __shfl_xor_sync(0xffffffffu, a2, 2);
                // every lane of quad g now holds the unit sums of batch row g; fetch those of rows 2t, 2t+1
                c1[l][mb][0] = __shfl_sync(0xffffffffu, a1, (2 * t) * 4);
                c1[l][mb][1] = __shfl_sync(0xffffffffu, a1, (2 * t + 1) * 4);
                c2[l][mb][0] = __shfl_sync(0xffffffffu, a2, (2 * t) * 4);
                c2[l][mb][1] = __shfl_sync(0xffffffffu, a2, (2 * t + 1) * 4);
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
    }
    __syncthreads(); // barrier initialisation and ss_w visible to everybody
    if (p.rmsnorm)
    {
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
    auto compute = [&](int step, int slot, const PReg& prm) {
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
                    const int row = row_of(step, h);
                    const uint32_t sidx_lo = (uint32_t)row * (uint32_t)p.G + (uint32_t)grp_of[0];
                    const uint32_t zoff_lo =
                        (WBITS == 4) ? (uint32_t)row * (uint32_t)p.zp_row_bytes + (uint32_t)(grp_of[0] >> 1) : sidx_lo;
#pragma unroll
                    for (int l = 0; l < 2; l++)
                    {
                        const int dg = grp_of[l] - grp_of[0];
                        if (p.scale_f32)
                            sc[l][h] = __uint_as_float(prm.sw[s][h]);
                        else
                            sc[l][h] = __half2float(
                                __ushort_as_half((unsigned short)(prm.sw[s][h] >> (16 * ((sidx_lo + dg) & 1)))));
                        if (WBITS == 4)
                            zq[l][h] = (prm.zw[s][h] >> (8 * (zoff_lo & 3) + 4 * (grp_of[l] & 1))) & 0xF;
                        else
                            zq[l][h] = (prm.zw[s][h] >> (8 * ((zoff_lo + dg) & 3))) & 0xFF;
                    }
                }
            }
            else
            {
#pragma unroll
                for (int h = 0; h < 2; h++)
                {
                    const int row = row_of(step, h);
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
            // this warp's tile: row r at r*128, 16-byte chunk c stored at chunk (c ^ (r & 7))
            const uint8_t* wt = ring + (size_t)((slot * SETS + s) * nwarps + warp) * kTileBytes;
            uint32_t wq[2][2][4]; // [unit][row half][word]
#pragma unroll
            for (int l = 0; l < 2; l++)
#pragma unroll
                for (int h = 0; h < 2; h++)
                {
                    const uint4 v = *reinterpret_cast<const uint4*>(wt + (g + 8 * h) * 128 + ((4 * l + t) ^ g) * 16);
                    wq[l][h][0] = v.x, wq[l][h][1] = v.y, wq[l][h][2] = v.z, wq[l][h][3] = v.w;
                }
            uint32_t zA[2][2], zB[2][2]; // fp16x2 constants holding (offset + zero-point)
            if (EXACT)
            {
#pragma unroll
                for (int l = 0; l < 2; l++)
#pragma unroll
                    for (int h = 0; h < 2; h++)
                    {
                        zA[l][h] = (0x6400u | zq[l][h]) * 0x00010001u;                                  // 1024 + zp
                        zB[l][h] = (WBITS == 4) ? (0x5400u | (zq[l][h] << 4)) * 0x00010001u : zA[l][h]; // 64 + zp
                    }
            }
            // four independent accumulation chains: (unit, word parity)
            float acc[2][2][MB][4];
#pragma unroll
            for (int l = 0; l < 2; l++)
#pragma unroll
                for (int e = 0; e < 2; e++)
#pragma unroll
                    for (int mb = 0; mb < MB; mb++)
#pragma unroll
                        for (int c = 0; c < 4; c++)
                            acc[l][e][mb][c] = 0.f;
#pragma unroll
            for (int w4 = 0; w4 < 4; w4++)
#pragma unroll
                for (int l = 0; l < 2; l++)
                {
                    uint32_t a[2][4]; // [row half][pair]
#pragma unroll
                    for (int h = 0; h < 2; h++)
                    {
                        const uint32_t w = wq[l][h][w4];
                        if (WBITS == 4)
                        {
                            const uint32_t w8 = w >> 8;
                            a[h][0] = and_or<0x000F000Fu, 0x64006400u>(w);  // 1024 + (n0, n4)
                            a[h][1] = and_or<0x00F000F0u, 0x54005400u>(w);  //   64 + (n1, n5)
                            a[h][2] = and_or<0x000F000Fu, 0x64006400u>(w8); // 1024 + (n2, n6)
                            a[h][3] = and_or<0x00F000F0u, 0x54005400u>(w8); //   64 + (n3, n7)
                            if (EXACT)
                            {
                                a[h][0] = hsub2_u32(a[h][0], zA[l][h]);
                                a[h][1] = hsub2_u32(a[h][1], zB[l][h]);
                                a[h][2] = hsub2_u32(a[h][2], zA[l][h]);
                                a[h][3] = hsub2_u32(a[h][3], zB[l][h]);
                            }
                        }
                        else
                        {
                            a[h][0] = __byte_perm(w, 0x64646464u, 0x4140); // 1024 + (b0, b1)
                            a[h][1] = __byte_perm(w, 0x64646464u, 0x4342); // 1024 + (b2, b3)
                            if (EXACT)
                            {
                                a[h][0] = hsub2_u32(a[h][0], zA[l][h]);
                                a[h][1] = hsub2_u32(a[h][1], zA[l][h]);
                            }
                        }
                    }
                    constexpr int PAIRS = (WBITS == 4) ? 4 : 2; // half2 pairs per word
#pragma unroll
                    for (int q = 0; q < PAIRS; q += 2)
                    {
                        const int f = w4 * PAIRS + q;
#pragma unroll
                        for (int mb = 0; mb < MB; mb++)
#pragma unroll
                            for (int xsn = 0; xsn < XS; xsn++)
                                mma16816(acc[l][w4 & 1][mb], a[0][q], a[1][q], a[0][q + 1], a[1][q + 1],
                                         xf[l][mb][xsn][f], xf[l][mb][xsn][f + 1]);
                    }
                }
#pragma unroll
            for (int mb = 0; mb < MB; mb++)
#pragma unroll
                for (int c = 0; c < 4; c++)
                {
                    float v = 0.f;
#pragma unroll
                    for (int l = 0; l < 2; l++)
                    {
                        float u = acc[l][0][mb][c] + acc[l][1][mb][c];
                        if (!EXACT)
                            u -= fmaf((float)zq[l][c >> 1], c2[l][mb][c & 1], c1[l][mb][c & 1]);
                        v = fmaf(sc[l][c >> 1], u, v);
                    }
                    tot[s][mb][c] = v;
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
    int slot = 0;
    uint32_t parity = 0;
    bool timed_out = false;
    for (int step = 0; step < nsteps; step += 6)
    {
        // unrolled by 6 = lcm(2 tiles per barrier, 3 parameter registers) so that every register index is static
#pragma unroll
        for (int pair = 0; pair < 3; pair++)
        {
            const int st = step + 2 * pair;
            if (st < nsteps)
            {
                const int pair_n = min(2, nsteps - st);
                float* my = red + (((st >> 1) & 1) * nwarps + warp) * 2 * TILE_F;
#pragma unroll
                for (int j = 0; j < 2; j++)
                {
                    if (j < pair_n)
                    {
                        constexpr int kRegs = 3;
                        const int ri = (2 * pair + j) % kRegs;
                        load_params(pr[(ri + 2) % kRegs], st + j + 2); // two tiles ahead, in registers
                        if (has_slice)
                        {
                            if (!mbar_wait(bar_s + 8 * slot, parity))
                                timed_out = true;
                            compute(st + j, slot, pr[ri]);
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
                                reinterpret_cast<float4*>(my + j * TILE_F)[q * 32 + lane] =
                                    make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                        if (++slot == p.depth)
                            slot = 0, parity ^= 1;
                    }
                }
                __syncthreads(); // every warp has read its tiles of this pair: the slots may be refilled
                if (tid == 0)
                    for (int j = 0; j < pair_n; j++)
                        produce(st + j + p.depth); // lands in the slot of tile st + j
                const float* rb = red + ((st >> 1) & 1) * nwarps * 2 * TILE_F;
                for (int o = tid; o < pair_n * TILE_F; o += nthreads)
                {
                    const int j = o / TILE_F, oo = o - j * TILE_F;
                    float v = 0.f;
                    for (int w = 0; w < nwarps; w++)
                        v += rb[w * 2 * TILE_F + j * TILE_F + oo];
                    res[((st + j) % kBatch) * TILE_F + oo] = v;
                }
                const int last = st + pair_n - 1;
                if ((last % kBatch) == kBatch - 1 || last == nsteps - 1)
                    flush(last - (last % kBatch), (last % kBatch) + 1);
            }
        }
    }
    if (timed_out)
        atomicExch(p.status, 1);
}

// Raise the kernel's dynamic shared-memory limit (monotonically: the attribute is a plain setter).
template <int WBITS, int MB, bool XSPLIT, bool DUAL, bool EXACT>
cudaError_t ensure_smem(size_t smem)
{
    static size_t configured = 48 * 1024;
    if (smem <= configured)
        return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(dq_gemv_kernel<WBITS, MB, XSPLIT, DUAL, EXACT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
        configured = smem;
    return e;
}

template <int WBITS, int MB, bool XSPLIT, bool DUAL, bool EXACT>
cudaError_t launch(const GemvParams& p, const CUtensorMap& t0, const CUtensorMap& t1, int warps, int grid,
                   size_t smem, cudaStream_t stream)
{
    cudaError_t e = ensure_smem<WBITS, MB, XSPLIT, DUAL, EXACT>(smem);
    if (e != cudaSuccess)
        return e;
    (void)cudaGetLastError(); // do not inherit a stale error left behind by an unrelated earlier call
    dq_gemv_kernel<WBITS, MB, XSPLIT, DUAL, EXACT><<<grid, warps * 32, smem, stream>>>(p, t0, t1);
    return cudaGetLastError();
}

size_t smem_for(int mb, bool dual, int warps, int depth)
{
    if (mb == 1)
        return dual ? Smem<1, true>::total_bytes(warps, depth) : Smem<1, false>::total_bytes(warps, depth);
    return dual ? Smem<2, true>::total_bytes(warps, depth) : Smem<2, false>::total_bytes(warps, depth);
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

cudaError_t dispatch(int wbits, const nnf::GemvPlan& plan, const GemvParams& p, const CUtensorMap& t0,
                     const CUtensorMap& t1, int grid, cudaStream_t stream)
{
#define NNF_X(WB, MBV, XSP, DU)                                                                                   \
    if (wbits == WB && plan.mb == MBV && plan.xsplit == XSP && plan.dual == DU)                                   \
        return plan.exact                                                                                         \
                   ? launch<WB, MBV, XSP, DU, true>(p, t0, t1, plan.warps, grid, plan.smem_bytes, stream)         \
                   : launch<WB, MBV, XSP, DU, false>(p, t0, t1, plan.warps, grid, plan.smem_bytes, stream);
    NNF_GEMV_FOR_EACH_VARIANT(NNF_X)
#undef NNF_X
    return cudaErrorInvalidValue;
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
    pl.exact = (d.flags & NNF_B200_FLAG_EXACT_ZP) != 0;
    // fp32 activations are carried as fp16 hi + lo where the register budget allows it
    pl.xsplit = d.x_dtype == NNF_B200_F32 && !(d.w_bits == 4 && pl.mb == 2);
    pl.row_tiles = (d.N + 15) / 16;
    const int units = d.K / ue;
    pl.slices = (units + 1) / 2;
    const int sms = ctx ? ctx->sm_count : 148;
    const int smem_cap = ctx ? ctx->smem_optin : 227 * 1024;
    const int sets = pl.dual ? 2 : 1;
    // Warps per CTA: one per slice of the CTA's K range; split K when a row has more slices than that.  The
    // widest CTA whose reduction buffers and a ring of at least two tiles fit in shared memory is taken.
    int resident = 1;
    bool fits = false;
    for (int max_warps : {16, 12, 8, 6, 4, 2, 1})
    {
        pl.splits = (pl.slices + max_warps - 1) / max_warps;
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
        // CTAs per SM by registers (the kernel is compiled for at most 128 per thread: 512 threads per SM), then
        // the deepest ring that lets that many CTAs share the SM's shared memory.
        resident = std::max(1, 512 / (pl.warps * 32));
        for (int depth = kMaxDepth; depth >= 2 && !fits; depth--)
        {
            pl.depth = depth;
            fits = (int)smem_for(pl.mb, pl.dual, pl.warps, depth) + 1024 <= smem_cap / resident;
        }
        if (!fits && resident > 1)
        {
            resident = 1;
            pl.depth = 2;
            fits = (int)smem_for(pl.mb, pl.dual, pl.warps, 2) + 1024 <= smem_cap;
        }
        if (fits || d.split_k > 0)
            break;
    }
    pl.smem_bytes = smem_for(pl.mb, pl.dual, pl.warps, pl.depth);
    if (!fits || (int)pl.smem_bytes > smem_cap)
    {
        *why = "shared memory: the launch shape does not fit";
        return NNF_B200_ENOTSUP;
    }
    int per_split = std::max(1, (sms * resident) / pl.splits);
    per_split = std::min(per_split, pl.row_tiles);
    pl.ctas_per_split = per_split;
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
    const int row_bytes = (d.w_bits == 4) ? d.K / 2 : d.K;
    p.scale[0] = w->scale;
    p.zp[0] = static_cast<const uint8_t*>(w->zp);
    if (plan.dual)
    {
        p.scale[1] = w2->scale;
        p.zp[1] = static_cast<const uint8_t*>(w2->zp);
    }
    // Weight tensor maps: bytes [N][row_bytes], boxes of 16 rows x 128 bytes, 128-byte swizzle.
    const CUtensorMap* t0 = weight_tensor_map(ctx, w->wq, d.N, row_bytes, 128, 16);
    const CUtensorMap* t1 = plan.dual ? weight_tensor_map(ctx, w2->wq, d.N, row_bytes, 128, 16) : t0;
    if (!t0 || !t1)
        return set_error(ctx, NNF_B200_ECUDA, "cuTensorMapEncodeTiled failed for the weight tensor");
    p.x = x;
    p.gain = static_cast<const float*>(gain);
    p.bias = static_cast<const float*>(bias);
    p.y = y;
    p.status = ctx->dev_status;
    p.M = d.M, p.N = d.N, p.K = d.K;
    p.group = d.group_size > 0 ? d.group_size : d.K;
    p.G = d.K / p.group;
    p.zp_row_bytes = (d.w_bits == 4) ? (p.G + 1) / 2 : p.G;
    p.units = d.K / ue;
    p.slices = plan.slices;
    p.row_tiles = plan.row_tiles;
    p.splits = plan.splits;
    p.ctas_per_split = plan.ctas_per_split;
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
    cudaError_t e = dispatch(d.w_bits, plan, p, *t0, *t1, grid, stream);
    if (e != cudaSuccess)
        return set_error(ctx, NNF_B200_ECUDA,
                         std::string("dq_gemv launch: ") + cudaGetErrorString(e) + " (grid " + std::to_string(grid) +
                             ", warps " + std::to_string(plan.warps) + ", smem " + std::to_string(plan.smem_bytes) + ")");
    ctx->launches++;
    return NNF_B200_OK;
}
} // namespace nnf

// ------------------------------------------------------------------------------------------------------------------
// Allocation-free variant of the split-K small-M linear.
//
// Who needs it: code that runs where device memory can no longer be requested -- in a real-time or
// safety-certified loop whose memory budget is frozen after start-up,
// or in a process that shares the GPU under a hard quota and must not grow.  Such a caller cannot obtain the split-K
// workspace that nnf_b200_linear expects from it.  Here the workspace is a fixed array that lives in the library's
// own device image, so every GPU that loads the library carries NNF_B200_STATIC_SCRATCH_BYTES of it until the process
// exits, and nothing is ever allocated or freed.
//
// The array's name is only a host-side handle in host code; the device address is fetched with
// cudaGetSymbolAddress once per device, by the first call made while that device is current.  That first call also
// raises the kernel's shared-memory limit and looks up the driver's tensor-map encoder, so it should be made
// outside of any stream capture.  All calls share the one array (and it keeps what the previous call left): calls
// that overlap on the GPU race on it; the tile counters are cleared on the stream at the start of every call.
namespace
{
static __device__ __align__(256) unsigned char g_static_scratch[NNF_B200_STATIC_SCRATCH_BYTES];
static __device__ int g_static_status;

struct StaticDeviceState
{
    bool ready = false;
    void* scratch = nullptr;
    int* status = nullptr;
    void* encode_tiled = nullptr;
    int sm_count = 0;
    int smem_optin = 0;
};
StaticDeviceState g_static_state[64];

void put_message(char* buf, size_t len, const char* msg)
{
    if (buf && len)
        snprintf(buf, len, "%s", msg);
}
} // namespace

extern "C" __attribute__((visibility("default"))) int
nnf_b200_linear_static_scratch(void* stream, const nnf_b200_linear_desc* desc, const void* x,
                               const nnf_b200_qweight* w, const nnf_b200_qweight* w2, const void* gain,
                               const void* bias, void* y, char* errbuf, size_t errbuf_len)
{
    using namespace nnf;
    put_message(errbuf, errbuf_len, "");
    if (!desc || !x || !y || !w || !w->wq || !w->scale || !w->zp)
    {
        put_message(errbuf, errbuf_len, "null descriptor, activations, output or weight set");
        return NNF_B200_EINVAL;
    }
    const nnf_b200_linear_desc& d = *desc;
    const bool dual = d.epilogue == NNF_B200_EPILOGUE_SILU_MUL;
    if (d.M < 1 || d.N < 1 || d.K < 1 || (d.w_bits != 4 && d.w_bits != 8) || d.group_size < 0 ||
        (dual && (!w2 || !w2->wq || !w2->scale || !w2->zp)) || (!dual && w2) ||
        ((d.prologue == NNF_B200_PROLOGUE_RMSNORM) != (gain != nullptr)) ||
        ((d.epilogue == NNF_B200_EPILOGUE_BIAS) != (bias != nullptr)))
    {
        put_message(errbuf, errbuf_len, "malformed descriptor or operands that do not match it");
        return NNF_B200_EINVAL;
    }
    if ((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(w->wq) & 15u) ||
        (dual && (reinterpret_cast<uintptr_t>(w2->wq) & 15u)) || (gain && (reinterpret_cast<uintptr_t>(gain) & 15u)))
    {
        put_message(errbuf, errbuf_len, "x, wq and gain must be 16-byte aligned");
        return NNF_B200_EALIGN;
    }

    // ---- once per device, with that device current
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    {
        put_message(errbuf, errbuf_len, "no current CUDA device");
        return NNF_B200_ECUDA;
    }
    StaticDeviceState& st = g_static_state[dev];
    if (!st.ready)
    {
        void* sp = nullptr;
        void* tp = nullptr;
        if (cudaGetSymbolAddress(&sp, g_static_scratch) != cudaSuccess || !sp ||
            cudaGetSymbolAddress(&tp, g_static_status) != cudaSuccess || !tp)
        {
            put_message(errbuf, errbuf_len, "cudaGetSymbolAddress failed for the built-in scratch array");
            return NNF_B200_ECUDA;
        }
        int major = 0;
        if (cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&st.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess || major != 10)
        {
            put_message(errbuf, errbuf_len, "device attributes unavailable, or not an sm_100 device");
            return NNF_B200_ENOTSUP;
        }
        st.encode_tiled = load_encode_tiled();
        if (!st.encode_tiled)
        {
            put_message(errbuf, errbuf_len, "cuTensorMapEncodeTiled entry point not found");
            return NNF_B200_ECUDA;
        }
        st.scratch = sp;
        st.status = static_cast<int*>(tp);
        st.ready = true;
    }

    // ---- launch shape; the only kernel served here is the small-M one, which is the one that needs scratch
    nnf_b200_ctx shape_ctx; // plain host struct, used only to carry the device's SM count and shared-memory limit
    shape_ctx.device = dev;
    shape_ctx.sm_count = st.sm_count;
    shape_ctx.smem_optin = st.smem_optin;
    GemvPlan plan;
    std::string why;
    int rc = gemv_plan(&shape_ctx, d, &plan, &why);
    if (rc != NNF_B200_OK)
    {
        put_message(errbuf, errbuf_len, why.c_str());
        return rc;
    }
    if (plan.workspace_bytes > (size_t)NNF_B200_STATIC_SCRATCH_BYTES)
    {
        char msg[160];
        snprintf(msg, sizeof msg, "this shape needs %zu bytes of scratch; the built-in array holds %d",
                 plan.workspace_bytes, (int)NNF_B200_STATIC_SCRATCH_BYTES);
        put_message(errbuf, errbuf_len, msg);
        return NNF_B200_EWORKSPACE;
    }

    const int ue = (d.w_bits == 4) ? 128 : 64;
    const int row_bytes = (d.w_bits == 4) ? d.K / 2 : d.K;
    alignas(64) CUtensorMap t0, t1;
    if (!encode_tensor_map_2d(st.encode_tiled, &t0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->wq, (uint64_t)row_bytes,
                              (uint64_t)d.N, (uint64_t)row_bytes, 128, 16, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !encode_tensor_map_2d(st.encode_tiled, &t1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, dual ? w2->wq : w->wq,
                              (uint64_t)row_bytes, (uint64_t)d.N, (uint64_t)row_bytes, 128, 16,
                              CU_TENSOR_MAP_SWIZZLE_128B))
    {
        put_message(errbuf, errbuf_len, "cuTensorMapEncodeTiled failed for the weight tensor");
        return NNF_B200_ECUDA;
    }

    GemvParams p{};
    p.scale[0] = w->scale;
    p.zp[0] = static_cast<const uint8_t*>(w->zp);
    if (dual)
    {
        p.scale[1] = w2->scale;
        p.zp[1] = static_cast<const uint8_t*>(w2->zp);
    }
    p.x = x;
    p.gain = static_cast<const float*>(gain);
    p.bias = static_cast<const float*>(bias);
    p.y = y;
    p.status = st.status;
    p.M = d.M, p.N = d.N, p.K = d.K;
    p.group = d.group_size > 0 ? d.group_size : d.K;
    p.G = d.K / p.group;
    p.zp_row_bytes = (d.w_bits == 4) ? (p.G + 1) / 2 : p.G;
    p.units = d.K / ue;
    p.slices = plan.slices;
    p.row_tiles = plan.row_tiles;
    p.splits = plan.splits;
    p.ctas_per_split = plan.ctas_per_split;
    p.x_f32 = d.x_dtype == NNF_B200_F32;
    p.y_f32 = d.y_dtype == NNF_B200_F32;
    p.scale_f32 = d.scale_dtype == NNF_B200_F32;
    p.rmsnorm = d.prologue == NNF_B200_PROLOGUE_RMSNORM;
    p.has_bias = bias != nullptr;
    p.eps = d.rms_eps;
    p.depth = plan.depth;
    p.slot_floats = (int)plan.slot_floats;
    const size_t scale_bytes = (size_t)d.N * p.G * (p.scale_f32 ? 4 : 2);
    const size_t zp_bytes = (size_t)d.N * p.zp_row_bytes;
    auto word_ok = [](const void* ptr, size_t bytes) {
        return (reinterpret_cast<uintptr_t>(ptr) & 3u) == 0 && (bytes & 3u) == 0;
    };
    p.fast_params = word_ok(w->scale, scale_bytes) && word_ok(w->zp, zp_bytes) &&
                    (!dual || (word_ok(w2->scale, scale_bytes) && word_ok(w2->zp, zp_bytes)));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (plan.splits > 1)
    {
        // The array keeps the previous call's contents: the per-tile arrival counters have to start at zero.
        const size_t cnt = ((size_t)plan.row_tiles * sizeof(unsigned) + 255) / 256 * 256;
        if (cudaMemsetAsync(st.scratch, 0, cnt, s) != cudaSuccess)
        {
            put_message(errbuf, errbuf_len, "cudaMemsetAsync on the built-in scratch array failed");
            return NNF_B200_ECUDA;
        }
        p.ws_count = static_cast<unsigned*>(st.scratch);
        p.ws_slots = reinterpret_cast<float*>(static_cast<char*>(st.scratch) + cnt);
    }
    cudaError_t e = dispatch(d.w_bits, plan, p, t0, t1, plan.splits * plan.ctas_per_split, s);
    if (e != cudaSuccess)
    {
        put_message(errbuf, errbuf_len, cudaGetErrorString(e));
        return NNF_B200_ECUDA;
    }
    return NNF_B200_OK;
}
