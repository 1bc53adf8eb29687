// Small-M (decode) dequantize-fused linear for sm_100a, register-pipeline form:
//     y[M,N] = epi(pro(x)[M,K] . dequant(W)[N,K]^T),  M <= 16.
//
// Fused replacement of the reference's Convert -> Subtract -> Multiply element-wise kernels
// (src/nnfusion/core/kernels/cuda_gpu/kernels/elementwise.hpp:33-157, elementwise_fused.cpp:42-189)
// followed by the cuBLAS Dot (src/nnfusion/core/kernels/cuda_gpu/kernels/dot.cpp:27-372): the
// weights are read once, at their packed size, and never materialised in fp32.
//
// The kernel is HBM-bound, so its shape is about getting requests out early and keeping them out:
//   * a weight row is cut into 128-byte "slices" (256 uint4 / 128 uint8 elements).  Warp w of a CTA owns slice
//     (first slice of the CTA's K range + w) for the whole launch: the activations it needs are loaded once and live
//     in registers as mma B fragments;
//   * CTAs are persistent and take a contiguous range of 16-row tiles.  Every thread reads exactly the four 16-byte
//     pieces per tile and weight set that it multiplies (rows g / g+8 of the tile, two 64-byte units of the warp's
//     slice) with 128-bit ld.global.nc straight into registers, PD stages ahead; the first PD stages leave before
//     anything else happens in the kernel.  There is no shared-memory ring, no producer warp and no barrier on the
//     weight path;
//   * what the register pipeline cannot hold in flight is asked for with bulk prefetches into L2
//     (cp.async.bulk.prefetch.L2), a bounded window of tiles ahead of the loads, so that HBM streams from the first
//     microsecond while the loads themselves only see L2 latency;
//   * the scales and zero-points of a batch of tiles arrive in shared memory by cp.async, every thread copying its
//     share of 16-byte pieces, double-buffered across batches; the kernel contains no wait on another agent at all;
//   * nibbles/bytes become exact fp16 integers with one LOP3/PRMT per pair (the 0x6400 / 0x5400 exponent trick) and
//     feed mma.sync.m16n8k16 with W as the 16-row operand and up to 8 batch rows as the 8-column operand;
//     accumulation is fp32; the offset and the zero-point leave the fp32 sum of each 64-byte unit afterwards,
//     acc - (C1 + zp * C2), then the group scale multiplies: sum((q - zp) * x) * scale;
//   * warps meet once per batch of tiles: partial sums wait in shared memory and are added in a fixed order; with
//     split-K every split stores its tile sums into its own workspace slot and the split that arrives last (a
//     counter per tile) adds the slots in a fixed order: results are bitwise repeatable and no CTA waits on another.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdio>
#include <mutex>

#include "nnf_internal.h"
#include "sm100_ptx.cuh"

namespace
{
using namespace nnf::ptx;

constexpr int kMaxWarps = 16;
constexpr int kBatch = 32; // most row tiles between two reductions over the warps

struct DirectParams
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
    int* status; // device status word: set to 1 when a bounded wait gave up
    int M, N, K;
    int group, G, zp_row_bytes;
    int units;     // 64-byte units per weight row
    int row_bytes; // bytes of one packed weight row
    int row_tiles, splits;
    int slices_lo, slices_rem; // slices / splits and its remainder
    int tiles_lo, tiles_rem;   // row_tiles / CTAs per split and its remainder
    int x_f32, y_f32, scale_f32, rmsnorm, has_bias;
    int has_addend;  // bias points at an [M,N] tensor of y's type instead of fp32 [N]
    int batch;       // row tiles between two reductions over the warps (<= kBatch)
    int tq;          // accumulator column pairs kept: 1, 2 or 4
    int bulk_params; // scales / zero-points of a batch arrive by bulk copy in shared memory
    int range_params; // ... and only the columns of this CTA's K range (rows are whole 16-byte pieces)
    int sc_row_bytes; // bytes of one row of scales
    int pmode;       // see the kernel's PMODE
    int scale_tile_bytes, zp_tile_bytes;
    // Rows of scales / zero-points as they lie in shared memory: whole rows, or (range_params) only the 16-byte
    // pieces that hold the columns of this CTA's K range, the widest range over the splits.
    int sm_sc_row, sm_zp_row;
    int xfrag_bytes;    // shared memory per warp for the activation fragments of batch rows 8..15 (0 when M <= 8)
    int prefetch_tiles; // L2 prefetch window in row tiles ahead of the register pipeline (0: no prefetch)
    int l1_lines;       // weight loads take lines in L1 (long launches)
    // K split: the CTAs that share a tile form a thread-block cluster (grid.y = cluster size = splits) and their sums
    // meet in the shared memory of the cluster's first CTA instead of the workspace.
    int cluster;
    int off_cslots;     // shared-memory offset of [splits][batch][slot_floats] floats (cluster only)
    int slot_floats;
    float eps;
    // shared-memory byte offsets (DirectSmem, computed once on the host)
    int off_bars, off_red, off_ss, off_flags;
    // a 64-byte unit's quantisation group = unit / group_units, done as a multiplication
    int group_units;
    uint32_t group_magic; // ceil(2^32 / group_units); exact for units below 2^16
    // Sum over the ranks of a tensor-parallel group inside this launch (ar_world > 1): see "exchange" in the kernel.
    const char* ar_bufs[8]; // every rank's fp32 partial-output buffer (two halves), own included, as mapped here
    uint32_t* ar_flags[8];  // every rank's flag words [row tile][sender], then one call counter per row tile
    size_t ar_half_stride;  // bytes between the two halves of a buffer
    uint32_t ar_epoch;      // call number from the host, or 0: counted in the words after the flags
    int ar_rank, ar_world;
};

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Same, starting a sum: the addend is zero.
__device__ __forceinline__ void mma16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// (w & MASK) | orv.  The OR-ed constant comes in a register that the caller fills once (see held_constant): with
// two immediates the compiler re-creates one of them in front of every use.
template <uint32_t MASK>
__device__ __forceinline__ uint32_t and_or(uint32_t w, uint32_t orv)
{
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(w), "n"(MASK), "r"(orv)); // (a & b) | c
    return r;
}
__device__ __forceinline__ uint32_t held_constant(uint32_t v)
{
    uint32_t r;
    asm volatile("mov.u32 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}
// A value the compiler must keep where it is: without this it recomputes loop invariants (lane offsets, tile
// counts, strides) from the kernel parameters in every trip of the main loop.
__device__ __forceinline__ int held(int v)
{
    int r;
    asm volatile("mov.b32 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}
__device__ __forceinline__ uint32_t pack_h2(__half a, __half b)
{
    return (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16);
}

// 16 bytes of weights, read once.  Without a line in L1 the load comes back sooner, which is what a short launch
// needs; with one, an SM sustains more bytes in flight, which is what a long launch needs (the host chooses).
__device__ __forceinline__ uint4 ldg_stream(const uint8_t* p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ldg_stream_l1(const uint8_t* p)
{
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// Ask for `bytes` (a multiple of 16, from a 16-byte aligned address) to be brought into L2; nothing comes back.
__device__ __forceinline__ void l2_prefetch(const uint8_t* p, uint32_t bytes)
{
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
// 16 bytes global -> shared without passing through registers; both addresses 16-byte aligned.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit()
{
    asm volatile("cp.async.commit_group;" ::: "memory");
}
// Wait until at most one of this thread's copy groups (the most recent) is still in flight.
__device__ __forceinline__ void cp_async_wait_but_one()
{
    asm volatile("cp.async.wait_group 1;" ::: "memory");
}
__device__ __forceinline__ unsigned short lds_u16(uint32_t addr)
{
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds_f32(uint32_t addr)
{
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u8(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

template <int WBITS>
struct Fmt
{
    static constexpr int UE = (WBITS == 4) ? 128 : 64; // elements per 64-byte unit
    static constexpr int LE = UE / 4;                  // elements per lane per 16-byte chunk
    static constexpr int NF = LE / 2;                  // half2 fragments per chunk
};

// The 16-byte pieces of a row of scales and of a row of zero-points that hold the quantisation groups of the slices
// [slice0, slice0 + slices) (a slice is slice_elems elements of K): first byte and number of pieces of each.
struct ParamRange
{
    int sc_b0, sc_pieces, zp_b0, zp_pieces;
};
__host__ __device__ inline ParamRange param_range(int slice0, int slices, int slice_elems, int K, int group, int sbytes,
                                                  int wbits, int sc_row_bytes, int zp_row_bytes)
{
    const int e0 = slice0 * slice_elems;
    const int e1 = (slice0 + slices) * slice_elems < K ? (slice0 + slices) * slice_elems : K;
    const int g0 = e0 / group, g1 = (e1 + group - 1) / group;
    ParamRange r;
    r.sc_b0 = (g0 * sbytes) & ~15;
    const int sc_end = (g1 * sbytes + 15) & ~15;
    r.sc_pieces = ((sc_end < sc_row_bytes ? sc_end : sc_row_bytes) - r.sc_b0) >> 4;
    const int z0 = wbits == 4 ? g0 >> 1 : g0, z1 = wbits == 4 ? (g1 + 1) >> 1 : g1;
    r.zp_b0 = z0 & ~15;
    const int zp_end = (z1 + 15) & ~15;
    r.zp_pieces = ((zp_end < zp_row_bytes ? zp_end : zp_row_bytes) - r.zp_b0) >> 4;
    return r;
}

// Shared-memory footprint, shared by host and device.  All sizes in bytes.
struct DirectSmem
{
    size_t params, bars, red, ss, flags, xsm, cslots, total;
    __host__ __device__ DirectSmem(int sets, int mb, int warps, int batch, int tq, int pset_bytes, int xfrag_bytes,
                                   int nbuf = 2, int cluster_splits = 0)
    {
        // (scales, zero-points) of a batch per weight set; two batches take turns unless one holds all tiles
        params = (size_t)nbuf * batch * sets * pset_bytes;
        bars = 0;
        red = sizeof(float) * (size_t)warps * batch * sets * mb * 8 * tq * 4;
        ss = sizeof(float) * ((size_t)warps * 8 * mb + 8 * mb);
        flags = sizeof(int) * (2 * kBatch + 4); // last-arriver flags, call numbers, "all peers answered"
        xsm = ((size_t)warps * xfrag_bytes + 15) / 16 * 16;
        // the splits' sums of a batch, in the first CTA of a cluster: [split][tile][sets * mb * 128 + 8 * mb] floats
        cslots = sizeof(float) * (size_t)cluster_splits * batch * ((size_t)sets * mb * 128 + 8 * mb);
        total = params + bars + red + ss + flags + xsm + cslots;
    }
};

// One pipeline stage: this lane's 16 bytes of rows g / g+8 of a tile, both units of the warp's slice, one weight set.
struct Stage
{
    uint4 w[2][2]; // [unit][row half]
};

// PMODE: how a lane finds its (scale, zero-point) pairs, settled by the host for the whole launch.
//   0  anything (plain loads when the parameters are not in shared memory);
//   1  parameters in shared memory, uint4 weights in groups of 128 with fp16 scales and an even number of groups
//      per row: the two scales of a slice sit side by side in one aligned word, the two zero-points in one byte;
//   2  parameters in shared memory, both units of every slice in one group (per-row parameters, uint8 weights in
//      groups of 128, ...): one scale and one zero-point per row half.
// M1: one batch row (the decode case): only accumulator column 0 is finished and kept.
template <int WBITS, int MB, bool XSPLIT, bool DUAL, int PD, int PMODE, bool M1>
__global__ void __launch_bounds__(kMaxWarps * 32, 1)
    dq_gemv_direct_kernel(const DirectParams p)
{
    using F = Fmt<WBITS>;
    constexpr int SETS = DUAL ? 2 : 1;
    static_assert(PD % SETS == 0, "a stage's weight set must not depend on the trip through the pipeline");
    constexpr int XS = XSPLIT ? 2 : 1;
    constexpr int NF = F::NF;
    constexpr int MPAD = 8 * MB;
    // 16 batch rows: the B fragments of rows 8..15 are parked in shared memory.
    constexpr bool XSM = (MB == 2);

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // The next launch on the stream may start as soon as SMs become free (it waits for this grid's results itself).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int nwarps = blockDim.x >> 5;
    const int nthreads = blockDim.x;
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    // grid = (CTAs per split, splits); quotients come from the host: nothing here waits for an integer division
    const int split = blockIdx.y, cta = blockIdx.x;
    const int my_slices = p.slices_lo + (split < p.slices_rem ? 1 : 0); // K ranges differ by at most one slice
    const int slice0 = split * p.slices_lo + min(split, p.slices_rem);
    const int slice = slice0 + warp;
    const bool has_slice = warp < my_slices;
    const int ntiles = held(p.tiles_lo + (cta < p.tiles_rem ? 1 : 0));
    const int tile0 = cta * p.tiles_lo + min(cta, p.tiles_rem);
    const int nstages = ntiles * SETS;
    const bool unit_ok[2] = {has_slice && 2 * slice < p.units, has_slice && 2 * slice + 1 < p.units};

    // ---------------------------------------------------------------- weights: the first PD stages leave at once
    // Every load is unconditional: a unit past the end of the row reads the unit before it (its activations are
    // zero, and the unpacking makes finite numbers of any bits); rows past N read row N - 1 (never stored).
    // (a warp without a slice asks for nothing; it still walks through the arithmetic with zero activations, which
    // leaves zeros where the other warps leave their sums)
    const int lane_off = held(has_slice ? slice * 128 + t * 16 : 0);
    const int unit1 = unit_ok[1] ? 64 : 0;
    const int last_row = held(p.N - 1);
    int issue_row = tile0 * 16 + g;            // row g of the next tile to ask for
    int to_issue = has_slice ? nstages : 0;    // stages not asked for yet
    const bool l1_lines = p.l1_lines != 0;
    // A CTA's shared memory may be written from another CTA of its cluster only once it runs: everybody arrives at
    // the cluster's barrier here and waits there before its first such write (end of the first batch).
    if (p.cluster)
        asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    bool cluster_met = false;
    auto issue = [&](Stage& b, int s) {
        const uint8_t* base = (s == 0 ? p.wq[0] : p.wq[1]) + lane_off;
        const uint8_t* r0 = base + (size_t)min(issue_row, last_row) * (size_t)p.row_bytes;
        const uint8_t* r1 = base + (size_t)min(issue_row + 8, last_row) * (size_t)p.row_bytes;
        if (l1_lines)
        {
            b.w[0][0] = ldg_stream_l1(r0);
            b.w[1][0] = ldg_stream_l1(r0 + unit1);
            b.w[0][1] = ldg_stream_l1(r1);
            b.w[1][1] = ldg_stream_l1(r1 + unit1);
        }
        else
        {
            b.w[0][0] = ldg_stream(r0);
            b.w[1][0] = ldg_stream(r0 + unit1);
            b.w[0][1] = ldg_stream(r1);
            b.w[1][1] = ldg_stream(r1 + unit1);
        }
        if (s == SETS - 1)
            issue_row += 16;
        to_issue--;
    };
    Stage buf[PD];
#pragma unroll
    for (int u = 0; u < PD; u++)
    {
        if (to_issue > 0)
            issue(buf[u], u % SETS);
        else
            buf[u].w[0][0] = buf[u].w[0][1] = buf[u].w[1][0] = buf[u].w[1][1] = make_uint4(0u, 0u, 0u, 0u);
    }

    // ---------------------------------------------------------------- L2 prefetch of what follows
    // A tile's rows are contiguous in memory, so one request per tile and weight set brings in all of K.  The
    // splits of a K-split launch walk the same tiles side by side on different SMs: split (tile mod splits) asks for
    // the whole tile on behalf of all of them (requests of a few KB each would keep the copy engine busier than
    // the loads they are meant to help).
    auto prefetch_tile = [&](int jt_, int s) { // local tile, weight set; one thread
        const int tile = tile0 + jt_;
        const int rows = min(16, p.N - tile * 16);
        l2_prefetch((s == 0 ? p.wq[0] : p.wq[1]) + (size_t)tile * 16 * p.row_bytes, (uint32_t)(rows * p.row_bytes));
    };
    constexpr int kDirectTiles = PD / SETS; // tiles the register pipeline has asked for already
    const int my_turn = held(p.splits == 1 ? 0 : split); // tiles with (local index mod splits) == my_turn are mine
    {
        const int pf_end = min(ntiles, kDirectTiles + p.prefetch_tiles);
        for (int i = kDirectTiles * SETS + tid; i < pf_end * SETS; i += nthreads)
            if (p.splits == 1 || (i / SETS) % p.splits == my_turn)
                prefetch_tile(i / SETS, i % SETS);
    }

    // ---------------------------------------------------------------- parameters: smem layout, first copies
    const int tq = p.tq;
    const int tq_shift = tq >> 1; // tq is 1, 2 or 4
    const int pt_shift = 5 + tq_shift + (MB == 2 ? 1 : 0);
    const int per_tile = 1 << pt_shift; // MB * 8 * tq * 4 floats: one warp's partial sums of one tile and weight set
    const int sm_scale_tile = 16 * p.sm_sc_row, sm_zp_tile = 16 * p.sm_zp_row; // one tile's rows in shared memory
    const int pset_bytes = sm_scale_tile + sm_zp_tile;
    // (pointers stay derived from the array itself, never from an integer, so that every access below is compiled
    // as a shared-memory access with a 32-bit address rather than as a generic one)
    uint8_t* pbuf = smem_raw; // [2 batches][SETS][scales of the batch's tiles | zero-points of the batch's tiles]
    float* red = reinterpret_cast<float*>(smem_raw + p.off_red);        // [nwarps][batch][SETS][per_tile]
    float* ss_w = reinterpret_cast<float*>(smem_raw + p.off_ss);        // [nwarps][MPAD]
    float* ss_cta = ss_w + nwarps * MPAD;                               // [MPAD]
    int* last_flag = reinterpret_cast<int*>(smem_raw + p.off_flags);    // [kBatch]
    // [warp][unit][xs][fragment pair][lane] x 8 bytes: B fragments of batch rows 8..15
    const uint32_t xsm_s = smem_u32(last_flag + 2 * kBatch + 4) + (uint32_t)(warp * p.xfrag_bytes) + (uint32_t)lane * 8u;
    const uint32_t pbuf_s = smem_u32(pbuf);
    const uint32_t pbatch_bytes = (uint32_t)(p.batch * SETS * pset_bytes); // one batch's parameters
    const uint32_t pzp_off = (uint32_t)(p.batch * sm_scale_tile);          // zero-points follow the batch's scales

    // Parameters of the local tiles [first, first + count) into buffer `which`: every thread copies its share of
    // 16-byte pieces with cp.async and closes one copy group (an empty one when there is nothing to copy, so that
    // "all groups but the newest" always means "everything up to the batch before").  No barrier object, no
    // copy-engine request: the batch's data is complete once every thread has waited for its own groups and the CTA
    // has met at a barrier.
    auto copy_params = [&](int first, int count, int which) {
        if (p.bulk_params && p.range_params && count > 0)
        {
            // K split over several CTAs: a CTA uses only the groups of its own slices, and its rows in shared memory
            // hold only the 16-byte pieces with those columns (a row there starts at column byte sc_b0 / zp_b0).
            // (worked out here, where it is needed, rather than kept in registers through the main loop)
            const ParamRange pr = param_range(slice0, my_slices, 2 * F::UE, p.K, p.group, p.scale_f32 ? 4 : 2, WBITS,
                                              p.sc_row_bytes, p.zp_row_bytes);
            const int sc_b0 = pr.sc_b0, sc_pieces = pr.sc_pieces, zp_b0 = pr.zp_b0, zp_pieces = pr.zp_pieces;
            const int rows = count * 16;
            const int per_row = sc_pieces + zp_pieces;
#pragma unroll
            for (int s = 0; s < SETS; s++)
            {
                const uint32_t dst = pbuf_s + which * pbatch_bytes + s * (uint32_t)(p.batch * pset_bytes);
                const size_t row0 = (size_t)(tile0 + first) * 16;
                const char* sc_src = static_cast<const char*>(s == 0 ? p.scale[0] : p.scale[1]) + row0 * p.sc_row_bytes + sc_b0;
                const uint8_t* zp_src = (s == 0 ? p.zp[0] : p.zp[1]) + row0 * p.zp_row_bytes + zp_b0;
                for (int i = tid; i < rows * per_row; i += nthreads)
                {
                    const int row = i / per_row, c = i - row * per_row;
                    if (c < sc_pieces)
                        cp_async16(dst + (uint32_t)(row * p.sm_sc_row + c * 16),
                                   sc_src + (size_t)row * p.sc_row_bytes + c * 16);
                    else
                        cp_async16(dst + pzp_off + (uint32_t)(row * p.sm_zp_row + (c - sc_pieces) * 16),
                                   zp_src + (size_t)row * p.zp_row_bytes + (c - sc_pieces) * 16);
                }
            }
        }
        else if (p.bulk_params && count > 0)
        {
            const int nsc = (count * p.scale_tile_bytes) >> 4, nzp = (count * p.zp_tile_bytes) >> 4;
#pragma unroll
            for (int s = 0; s < SETS; s++)
            {
                const uint32_t dst = pbuf_s + which * pbatch_bytes + s * (uint32_t)(p.batch * pset_bytes);
                const size_t tile = (size_t)(tile0 + first);
                const char* sc_src = static_cast<const char*>(s == 0 ? p.scale[0] : p.scale[1]) + tile * p.scale_tile_bytes;
                const uint8_t* zp_src = (s == 0 ? p.zp[0] : p.zp[1]) + tile * p.zp_tile_bytes;
                for (int i = tid; i < nsc + nzp; i += nthreads)
                {
                    if (i < nsc)
                        cp_async16(dst + (uint32_t)i * 16u, sc_src + (size_t)i * 16);
                    else
                        cp_async16(dst + pzp_off + (uint32_t)(i - nsc) * 16u, zp_src + (size_t)(i - nsc) * 16);
                }
            }
        }
        cp_async_commit();
    };
    copy_params(0, min(p.batch, ntiles), 0);
    copy_params(p.batch, min(p.batch, max(ntiles - p.batch, 0)), 1);

    // Everything above reads only constants (weights, scales, zero-points).  The activations, the output and the workspace may belong
    // to the launch before this one on the stream: when this kernel was launched as its programmatic dependent, it
    // has been running beside that launch's tail until here.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---------------------------------------------------------------- activations: ask first, set up meanwhile
    // fp16 activations that are used as they are: the raw loads leave now and are permuted into fragments below.
    const bool plain = !XSPLIT && !p.x_f32 && !p.rmsnorm;
    uint32_t xf[2][XSM ? 1 : MB][XS][NF];
    uint4 xraw[2][MB][F::LE / 8];
    if (plain)
    {
#pragma unroll
        for (int l = 0; l < 2; l++)
#pragma unroll
            for (int mb = 0; mb < MB; mb++)
            {
                const int m = g + 8 * mb;
                const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __half*>(p.x) + (size_t)m * p.K +
                                                                 (unit_ok[l] ? 2 * slice + l : 0) * F::UE + t * F::LE);
#pragma unroll
                for (int j = 0; j < F::LE / 8; j++)
                    xraw[l][mb][j] = (unit_ok[l] && m < p.M) ? __ldg(src + j) : make_uint4(0u, 0u, 0u, 0u);
            }
    }

    int grp_of[2];
#pragma unroll
    for (int l = 0; l < 2; l++)
    {
        // a unit that does not exist (a warp without a slice, the tail of the row) multiplies zero activations with
        // the parameters of the CTA's first unit: finite numbers that are in shared memory whichever columns were
        // copied
        const uint32_t unit = (uint32_t)(unit_ok[l] ? 2 * slice + l : 2 * slice0);
        grp_of[l] = p.group_units == 1 ? (int)unit : (int)__umulhi(unit, p.group_magic);
    }
    // Byte offsets of this lane's scales / zero-points inside a tile's parameter block: rows g and g + 8 of the
    // tile, groups of the two units of the slice.
    const int sbytes = p.scale_f32 ? 4 : 2;
    // first column byte of the rows in shared memory (0 unless only this CTA's K range was copied)
    ParamRange col0{0, 0, 0, 0};
    if (p.bulk_params && p.range_params)
        col0 = param_range(slice0, my_slices, 2 * F::UE, p.K, p.group, sbytes, WBITS, p.sc_row_bytes, p.zp_row_bytes);
    int soff[2][2], zoff[2][2];
#pragma unroll
    for (int l = 0; l < 2; l++)
#pragma unroll
        for (int h = 0; h < 2; h++)
        {
            soff[l][h] = (g + 8 * h) * p.sm_sc_row + grp_of[l] * sbytes - col0.sc_b0;
            zoff[l][h] = (g + 8 * h) * p.sm_zp_row + (WBITS == 4 ? grp_of[l] >> 1 : grp_of[l]) - col0.zp_b0;
        }
    const int zsh[2] = {(WBITS == 4) ? 4 * (grp_of[0] & 1) : 0, (WBITS == 4) ? 4 * (grp_of[1] & 1) : 0};


    // ---------------------------------------------------------------- activations -> B fragments in registers
    // Corrections for accumulator columns 2t, 2t+1, taken out of every unit's fp32 sum: nc1 = -sum(offset_k * x_k),
    // nc2 = -sum(x_k) (times the zero-point).
    float nc1[2][MB][2], nc2[2][MB][2];
    float ss_local[MB];
#pragma unroll
    for (int mb = 0; mb < MB; mb++)
        ss_local[mb] = 0.f;
#pragma unroll
    for (int l = 0; l < 2; l++)
    {
        const int k0 = (unit_ok[l] ? 2 * slice + l : 0) * F::UE + t * F::LE;
#pragma unroll
        for (int mb = 0; mb < MB; mb++)
        {
            const int m = g + 8 * mb;
            const bool live = unit_ok[l] && m < p.M;
            uint32_t frag[XS][NF];
            if (plain)
            {
                // Element order inside a fragment mirrors the order the weight unpacking produces:
                // uint4 word i yields pairs (n0,n4) (n1,n5) (n2,n6) (n3,n7); uint8 word i yields (b0,b1) (b2,b3).
#pragma unroll
                for (int j = 0; j < F::LE / 8; j++)
                {
                    const uint4 v = xraw[l][mb][j];
                    if (WBITS == 4)
                    {
                        frag[0][4 * j + 0] = __byte_perm(v.x, v.z, 0x5410);
                        frag[0][4 * j + 1] = __byte_perm(v.x, v.z, 0x7632);
                        frag[0][4 * j + 2] = __byte_perm(v.y, v.w, 0x5410);
                        frag[0][4 * j + 3] = __byte_perm(v.y, v.w, 0x7632);
                    }
                    else
                    {
                        frag[0][4 * j + 0] = v.x, frag[0][4 * j + 1] = v.y;
                        frag[0][4 * j + 2] = v.z, frag[0][4 * j + 3] = v.w;
                    }
                }
            }
            else
            {
                float xv[F::LE];
                if (live)
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
                    if (XSPLIT)
                        lo[j] = __float2half_rn(xv[j] - __half2float(hi[j]));
                }
#pragma unroll
                for (int f = 0; f < NF; f++)
                {
                    const int e0 = (WBITS == 4) ? 8 * (f >> 2) + (f & 3) : 2 * f;
                    const int e1 = (WBITS == 4) ? e0 + 4 : e0 + 1;
                    frag[0][f] = pack_h2(hi[e0], hi[e1]);
                    if (XSPLIT)
                        frag[XS - 1][f] = pack_h2(lo[e0], lo[e1]);
                }
            }
            {
                // C1 and C2 of the unit for every batch row, summed by the tensor core exactly as it will sum the
                // products: rows 0-7 of the left operand hold the offsets the unpacking leaves in place (uint4:
                // 1024 on even fragments, 64 on odd ones; uint8: 1024), rows 8-15 hold ones.  Every lane ends up
                // with the sums of accumulator columns 2t and 2t+1.
                constexpr uint32_t off_even = 0x64006400u, off_odd = (WBITS == 4) ? 0x54005400u : 0x64006400u;
                constexpr uint32_t ones = 0x3C003C00u;
                float d[4];
#pragma unroll
                for (int f = 0; f < NF; f += 2)
#pragma unroll
                    for (int xsn = 0; xsn < XS; xsn++)
                    {
                        if (f == 0 && xsn == 0)
                            mma16816_first(d, off_even, ones, off_odd, ones, frag[xsn][f], frag[xsn][f + 1]);
                        else
                            mma16816(d, off_even, ones, off_odd, ones, frag[xsn][f], frag[xsn][f + 1]);
                    }
                nc1[l][mb][0] = -d[0], nc1[l][mb][1] = -d[1];
                nc2[l][mb][0] = -d[2], nc2[l][mb][1] = -d[3];
            }
            if (XSM && mb == 1)
            {
#pragma unroll
                for (int xsn = 0; xsn < XS; xsn++)
#pragma unroll
                    for (int f = 0; f < NF; f += 2)
                        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(
                                         xsm_s + (uint32_t)(((l * XS + xsn) * (NF / 2) + f / 2) * 256)),
                                     "r"(frag[xsn][f]), "r"(frag[xsn][f + 1])
                                     : "memory");
            }
            else
            {
#pragma unroll
                for (int xsn = 0; xsn < XS; xsn++)
#pragma unroll
                    for (int f = 0; f < NF; f++)
                        xf[l][XSM ? 0 : mb][xsn][f] = frag[xsn][f];
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
    cp_async_wait_but_one(); // this thread's pieces of the first batch's parameters have landed
    __syncthreads();         // ... and everybody's; ss_w visible
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

    // ---------------------------------------------------------------- arithmetic on one stage
    const uint32_t k6400 = held_constant(0x64006400u), k5400 = held_constant(0x54005400u);
    const bool same_grp = grp_of[1] == grp_of[0];
    // this lane's scale / zero-point of unit 0 for rows g and g + 8, as offsets into a tile's parameter block
    const uint32_t so[2] = {(uint32_t)held(soff[0][0]), (uint32_t)held(soff[0][1])};
    const uint32_t zo[2] = {(uint32_t)held(zoff[0][0]), (uint32_t)held(zoff[0][1])};

    // tot: this warp's sums for rows g / g+8 (index 0,1 / 2,3) and batch columns 2t / 2t+1.
    auto compute = [&](const Stage& b, int tile, int s, uint32_t sc_s, uint32_t zp_s, float (&tot)[MB][4]) {
        // (scale, zero-point) of rows g / g+8 for both halves of the slice
        float sc[2][2], nz[2][2];
        if (PMODE == 1)
        {
#pragma unroll
            for (int h = 0; h < 2; h++)
            {
                uint32_t sp;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(sp) : "r"(sc_s + so[h]));
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&sp));
                sc[0][h] = f.x, sc[1][h] = f.y;
                const uint32_t zb = lds_u8(zp_s + zo[h]);
                nz[0][h] = (float)(zb & 0xFu), nz[1][h] = (float)(zb >> 4);
            }
        }
        else if (PMODE == 2)
        {
#pragma unroll
            for (int h = 0; h < 2; h++)
            {
                const uint32_t sa = sc_s + so[h];
                sc[0][h] = sc[1][h] = p.scale_f32 ? lds_f32(sa) : __half2float(__ushort_as_half(lds_u16(sa)));
                const uint32_t zb = lds_u8(zp_s + zo[h]);
                nz[0][h] = nz[1][h] = (float)((WBITS == 4) ? (zb >> zsh[0]) & 0xFu : zb);
            }
        }
        else if (p.bulk_params)
        {
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int l = 0; l < 2; l++)
                {
                    if (l == 1 && same_grp)
                    {
                        sc[1][h] = sc[0][h], nz[1][h] = nz[0][h];
                        continue;
                    }
                    const uint32_t sa = sc_s + (uint32_t)soff[l][h];
                    sc[l][h] = p.scale_f32 ? lds_f32(sa) : __half2float(__ushort_as_half(lds_u16(sa)));
                    const uint32_t zb = lds_u8(zp_s + (uint32_t)zoff[l][h]);
                    nz[l][h] = (float)((WBITS == 4) ? (zb >> zsh[l]) & 0xFu : zb);
                }
        }
        else
        {
#pragma unroll
            for (int h = 0; h < 2; h++)
            {
                const int row = min(tile * 16 + g + 8 * h, p.N - 1);
#pragma unroll
                for (int l = 0; l < 2; l++)
                {
                    const size_t sidx = (size_t)row * p.G + grp_of[l];
                    const void* sp = s == 0 ? p.scale[0] : p.scale[1];
                    const uint8_t* zp = s == 0 ? p.zp[0] : p.zp[1];
                    sc[l][h] = p.scale_f32 ? __ldg(static_cast<const float*>(sp) + sidx)
                                           : __half2float(__ldg(static_cast<const __half*>(sp) + sidx));
                    if (WBITS == 4)
                        nz[l][h] = (float)((__ldg(zp + (size_t)row * p.zp_row_bytes + (grp_of[l] >> 1)) >> zsh[l]) & 0xFu);
                    else
                        nz[l][h] = (float)__ldg(zp + sidx);
                }
            }
        }
        // one accumulation chain per unit (the units may belong to different quantisation groups)
        float acc[2][MB][4];
#pragma unroll
        for (int w4 = 0; w4 < 4; w4++)
#pragma unroll
            for (int l = 0; l < 2; l++)
            {
                uint32_t a[2][4]; // [row half][pair]
#pragma unroll
                for (int h = 0; h < 2; h++)
                {
                    const uint4 v = b.w[l][h];
                    const uint32_t w = w4 == 0 ? v.x : (w4 == 1 ? v.y : (w4 == 2 ? v.z : v.w));
                    if (WBITS == 4)
                    {
                        const uint32_t w8 = w >> 8;
                        a[h][0] = and_or<0x000F000Fu>(w, k6400);  // 1024 + (n0, n4)
                        a[h][1] = and_or<0x00F000F0u>(w, k5400);  //   64 + (n1, n5)
                        a[h][2] = and_or<0x000F000Fu>(w8, k6400); // 1024 + (n2, n6)
                        a[h][3] = and_or<0x00F000F0u>(w8, k5400); //   64 + (n3, n7)
                    }
                    else
                    {
                        a[h][0] = __byte_perm(w, 0x64646464u, 0x4140); // 1024 + (b0, b1)
                        a[h][1] = __byte_perm(w, 0x64646464u, 0x4342); // 1024 + (b2, b3)
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
                        {
                            uint32_t b0, b1;
                            if (!XSM || mb == 0)
                                b0 = xf[l][XSM ? 0 : mb][xsn][f], b1 = xf[l][XSM ? 0 : mb][xsn][f + 1];
                            else
                                asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];"
                                             : "=r"(b0), "=r"(b1)
                                             : "r"(xsm_s + (uint32_t)(((l * XS + xsn) * (NF / 2) + f / 2) * 256)));
                            if (w4 == 0 && q == 0 && xsn == 0) // first product of this chain
                                mma16816_first(acc[l][mb], a[0][q], a[1][q], a[0][q + 1], a[1][q + 1], b0, b1);
                            else
                                mma16816(acc[l][mb], a[0][q], a[1][q], a[0][q + 1], a[1][q + 1], b0, b1);
                        }
                }
            }
        auto finish_col = [&](int mb, int c) {
            const float u0 = acc[0][mb][c] + fmaf(nz[0][c >> 1], nc2[0][mb][c & 1], nc1[0][mb][c & 1]);
            const float u1 = acc[1][mb][c] + fmaf(nz[1][c >> 1], nc2[1][mb][c & 1], nc1[1][mb][c & 1]);
            tot[mb][c] = fmaf(sc[1][c >> 1], u1, sc[0][c >> 1] * u0);
        };
#pragma unroll
        for (int mb = 0; mb < MB; mb++)
#pragma unroll
            for (int c = 0; c < 4; c += (M1 ? 2 : 1))
                finish_col(mb, c);
    };

    // Final value of one output element from its summed parts.
    auto finish = [&](float a0, float a1, float ssum, int m, int n) -> float {
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
        if (p.has_addend)
            v += p.y_f32 ? reinterpret_cast<const float*>(p.bias)[(size_t)m * p.N + n]
                         : __half2float(reinterpret_cast<const __half*>(p.bias)[(size_t)m * p.N + n]);
        return v;
    };
    auto store_y = [&](int m, int n, float v) {
        if (p.y_f32)
            static_cast<float*>(p.y)[(size_t)m * p.N + n] = v;
        else
            static_cast<__half*>(p.y)[(size_t)m * p.N + n] = __float2half_rn(v);
    };
    // Index e in [0, per_tile) of a warp's partial sums = ((mb * 8 + g) * tq + t) * 4 + c  <->  row of the tile,
    // batch row m, and the index o of the same value in a workspace slot ([mb][lane][c], all 32 lanes).
    auto decode = [&](int e, int& row, int& m, int& o) {
        const int c = e & 3, r1 = e >> 2;
        const int tt = r1 & (tq - 1), r2 = r1 >> tq_shift;
        const int gg = r2 & 7, mb = r2 >> 3;
        row = gg + 8 * (c >> 1);
        m = 8 * mb + 2 * tt + (c & 1);
        o = ((mb * 32 + gg * 4 + tt) << 2) + c;
    };
    const int warp_stride = p.batch * SETS * per_tile; // floats between two warps' partial sums
    auto sum_warps = [&](int j, int s, int e) -> float {
        const float* r = red + (j * SETS + s) * per_tile + e;
        float part[kMaxWarps]; // all loads first: a rolled loop would pay the shared-memory latency sixteen times
#pragma unroll
        for (int w = 0; w < kMaxWarps; w++)
            part[w] = w < nwarps ? r[w * warp_stride] : 0.f;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kMaxWarps; w++)
            v += part[w];
        return v;
    };

    // ---- exchange: summing over the ranks of a tensor-parallel group inside this launch (ar_world > 1)
    // Every rank runs this kernel with the same launch shape, so the CTA that holds the final sum of a row tile here
    // (for splits == 1 the tile's own CTA, otherwise the split that arrived last) has one partner per rank.  It
    // writes its fp32 sums into EVERY rank's buffer (slot [sender] of the half in use: plain stores, over NVLink for
    // the peers'), tells every peer "tile t, call e" with one release store per peer, waits (bounded) for the peers'
    // words for the same tile, then finds everybody's sums in its own memory and adds them in rank order: every
    // rank stores the same bits, and one NVLink hop (data and flag travel together) stands between a tile's last
    // sum and its result.  Calls alternate between the two halves of the buffers (half = e & 1): a rank can be one
    // call ahead of a peer that is still reading a tile, never two, because the same tile's flag of the call in
    // between is needed first.  Nothing here waits on a CTA of this GPU,
    // and the peers' CTAs announce before they wait, so no cycle of waits can form.  A wait that gives up raises
    // the status word; the tile is then left unwritten.
    const bool ar = !DUAL && p.ar_world > 1;
    uint32_t* const ep_s = reinterpret_cast<uint32_t*>(last_flag) + kBatch; // [kBatch] call number per tile
    int* const ar_ok = reinterpret_cast<int*>(ep_s + kBatch);
    auto ar_begin = [&](int first, int count, bool by_last_flag) {
        uint32_t* counters = p.ar_flags[p.ar_rank] + (size_t)p.row_tiles * 8;
        if (tid < count && (!by_last_flag || last_flag[tid] != 0))
        {
            uint32_t e = p.ar_epoch;
            if (e == 0)
            {
                e = __ldcg(counters + tile0 + first + tid) + 1; // only the CTA that finishes the tile touches it
                if (e == 0)
                    e = 2; // 0 means "count for me": skip it, keeping the parity
            }
            ep_s[tid] = e;
        }
        if (tid == 0)
            *ar_ok = 1;
        __syncthreads();
    };
    const size_t ar_slot = (size_t)p.M * p.N * sizeof(float); // one sender's sums inside a half
    auto ar_put = [&](int j, int m, int n, float v) {
        const size_t off = (size_t)(ep_s[j] & 1u) * p.ar_half_stride + (size_t)p.ar_rank * ar_slot +
                           ((size_t)m * p.N + n) * sizeof(float);
        for (int r = 0; r < p.ar_world; r++)
            *reinterpret_cast<float*>(const_cast<char*>(p.ar_bufs[r]) + off) = v;
    };
    auto ar_end = [&](int first, int count, bool by_last_flag) {
        auto owns = [&](int j) { return !by_last_flag || last_flag[j] != 0; };
        uint32_t* counters = p.ar_flags[p.ar_rank] + (size_t)p.row_tiles * 8;
        // this rank's sums (in every rank's memory) are ordered before the announcements by the barrier and the
        // release stores (cumulative over what the barrier made visible to the storing thread)
        __syncthreads();
        // pair (tile j, peer r) = idx: every announcement leaves before the first wait starts
        for (int idx = tid; idx < count * p.ar_world; idx += nthreads)
        {
            const int j = idx / p.ar_world, r = idx - j * p.ar_world;
            if (r != p.ar_rank && owns(j))
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.ar_flags[r] + (size_t)(tile0 + first + j) * 8 + p.ar_rank),
                             "r"(ep_s[j])
                             : "memory");
        }
        for (int idx = tid; idx < count * p.ar_world; idx += nthreads)
        {
            const int j = idx / p.ar_world, r = idx - j * p.ar_world;
            if (r != p.ar_rank && owns(j))
            {
                const uint32_t e = ep_s[j];
                const uint32_t* mine = p.ar_flags[p.ar_rank] + (size_t)(tile0 + first + j) * 8 + r;
                bool seen = false;
                for (uint32_t i = 0; i < (1u << 19) && !seen; i++) // roughly 0.4 s
                {
                    uint32_t v;
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
                    seen = (int32_t)(v - e) >= 0;
                    if (!seen)
                        __nanosleep(40);
                }
                if (!seen)
                {
                    *ar_ok = 0;
                    atomicExch(p.status, 1);
                }
            }
        }
        if (p.ar_epoch == 0 && tid < count && owns(tid))
            __stcg(counters + tile0 + first + tid, ep_s[tid]);
        __syncthreads();
        if (!*ar_ok)
            return;
        for (int idx = tid; idx < count * per_tile; idx += nthreads) // everybody's sums in rank order
        {
            const int j = idx >> pt_shift, e = idx & (per_tile - 1);
            if (!owns(j))
                continue;
            int row, m, o;
            decode(e, row, m, o);
            const int n = (tile0 + first + j) * 16 + row;
            if (m < p.M && n < p.N)
            {
                const char* half = p.ar_bufs[p.ar_rank] + (size_t)(ep_s[j] & 1u) * p.ar_half_stride +
                                   ((size_t)m * p.N + n) * sizeof(float);
                float v = 0.f;
                for (int r = 0; r < p.ar_world; r++)
                    v += __ldcv(reinterpret_cast<const float*>(half + (size_t)r * ar_slot));
                store_y(m, n, finish(v, 0.f, 0.f, m, n));
            }
        }
    };

    // Add up the warps' partial sums of the local tiles [first, first + count) and write the results out.
    // (the caller brackets it with the CTA's barriers)
    auto flush = [&](int first, int count) {
        if (p.splits == 1)
        {
            if (ar)
                ar_begin(first, count, false);
            for (int idx = tid; idx < count * per_tile; idx += nthreads)
            {
                const int j = idx >> pt_shift, e = idx & (per_tile - 1);
                int row, m, o;
                decode(e, row, m, o);
                const int n = (tile0 + first + j) * 16 + row;
                if (m < p.M && n < p.N)
                {
                    if (ar)
                        ar_put(j, m, n, sum_warps(j, 0, e));
                    else
                        store_y(m, n, finish(sum_warps(j, 0, e), DUAL ? sum_warps(j, 1, e) : 0.f,
                                             p.rmsnorm ? ss_cta[m] : 0.f, m, n));
                }
            }
            if (ar)
                ar_end(first, count, false);
        }
        else if (p.cluster)
        {
            // The splits of these tiles are the CTAs of one cluster (rank = split).  1. every CTA writes its sums
            // (and its share of the sum of squares) into the first CTA's shared memory; 2. the cluster meets at its
            // barrier; 3. the first CTA adds the splits' sums in split order.  No global memory, no counter, and
            // the hardware schedules a cluster's CTAs together: nothing here can wait for a CTA that is not running.
            float* const cslots = reinterpret_cast<float*>(smem_raw + p.off_cslots);
            uint32_t remote; // the same array in the first CTA
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(cslots)), "r"(0));
            const uint32_t my_part = remote + (uint32_t)(split * p.batch * p.slot_floats) * 4u;
            if (!cluster_met)
            {
                asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
                cluster_met = true;
            }
            auto put = [&](uint32_t float_index, float v) {
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(my_part + float_index * 4u), "f"(v) : "memory");
            };
            for (int idx = tid; idx < count * per_tile; idx += nthreads)
            {
                const int j = idx >> pt_shift, e = idx & (per_tile - 1);
                int row, m, o;
                decode(e, row, m, o);
                if (m >= p.M)
                    continue;
                put((uint32_t)(j * p.slot_floats + o), sum_warps(j, 0, e));
                if (DUAL)
                    put((uint32_t)(j * p.slot_floats + MB * 128 + o), sum_warps(j, 1, e));
            }
            if (p.rmsnorm)
                for (int idx = tid; idx < count * MPAD; idx += nthreads)
                {
                    const int j = idx / MPAD, mm = idx - j * MPAD;
                    put((uint32_t)(j * p.slot_floats + SETS * MB * 128 + mm), ss_cta[mm]);
                }
            asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
            if (tid < count)
                last_flag[tid] = (split == 0);
            __syncthreads();
            if (ar)
                ar_begin(first, count, true);
            if (split == 0)
                for (int idx = tid; idx < count * per_tile; idx += nthreads)
                {
                    const int j = idx >> pt_shift, e = idx & (per_tile - 1);
                    int row, m, o;
                    decode(e, row, m, o);
                    const int n = (tile0 + first + j) * 16 + row;
                    if (m < p.M && n < p.N)
                    {
                        float a0 = 0.f, a1 = 0.f, ssum = 0.f;
                        for (int sp = 0; sp < p.splits; sp++) // fixed order: repeatable
                        {
                            const float* slot = cslots + (size_t)(sp * p.batch + j) * p.slot_floats;
                            a0 += slot[o];
                            if (DUAL)
                                a1 += slot[MB * 128 + o];
                            if (p.rmsnorm)
                                ssum += slot[SETS * MB * 128 + m];
                        }
                        if (ar)
                            ar_put(j, m, n, a0);
                        else
                            store_y(m, n, finish(a0, a1, ssum, m, n));
                    }
                }
            if (ar)
                ar_end(first, count, true);
            // another batch follows: its sums must not land before the first CTA has read these
            if (first + count < ntiles)
                asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
        }
        else
        {
            // 1. publish this split's sums (and its share of the sum of squares)
            for (int idx = tid; idx < count * per_tile; idx += nthreads)
            {
                const int j = idx >> pt_shift, e = idx & (per_tile - 1);
                int row, m, o;
                decode(e, row, m, o);
                if (m >= p.M)
                    continue;
                const int rt = tile0 + first + j;
                float* slot = p.ws_slots + ((size_t)split * p.row_tiles + rt) * p.slot_floats;
                __stcg(slot + o, sum_warps(j, 0, e));
                if (DUAL)
                    __stcg(slot + MB * 128 + o, sum_warps(j, 1, e));
            }
            if (p.rmsnorm)
                for (int idx = tid; idx < count * MPAD; idx += nthreads)
                {
                    const int j = idx / MPAD, mm = idx - j * MPAD;
                    const int rt = tile0 + first + j;
                    __stcg(p.ws_slots + ((size_t)split * p.row_tiles + rt) * p.slot_floats + SETS * MB * 128 + mm,
                           ss_cta[mm]);
                }
            __threadfence();
            __syncthreads();
            // 2. one arrival per tile; the last split to arrive owns the tile's final sum
            if (tid < count)
            {
                const int rt = tile0 + first + tid;
                const unsigned old = atomicAdd(p.ws_count + rt, 1u);
                last_flag[tid] = (old == (unsigned)(p.splits - 1));
                if (last_flag[tid])
                    p.ws_count[rt] = 0u; // leave the counter zeroed for the next call
            }
            __syncthreads();
            __threadfence();
            if (ar)
                ar_begin(first, count, true);
            // 3. fixed-order sum over the splits
            for (int idx = tid; idx < count * per_tile; idx += nthreads)
            {
                const int j = idx >> pt_shift, e = idx & (per_tile - 1);
                if (!last_flag[j])
                    continue;
                int row, m, o;
                decode(e, row, m, o);
                const int rt = tile0 + first + j;
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
                            ssum += __ldcg(slot + SETS * MB * 128 + m);
                    }
                    if (ar)
                        ar_put(j, m, n, a0);
                    else
                        store_y(m, n, finish(a0, a1, ssum, m, n));
                }
            }
            if (ar)
                ar_end(first, count, true);
        }
    };

    // ---------------------------------------------------------------- main loop
    // Batches of tiles; a batch that is not the last has a whole number of trips through the register pipeline
    // (the host picks the batch length that way), so a stage's place in the pipeline is known at compile time.
    const uint32_t red_lane_s = smem_u32(red) + (uint32_t)(warp * warp_stride) * 4u + (uint32_t)(g * tq + t) * 16u;
    const uint32_t red_step = (uint32_t)held(per_tile * 4);
    const uint32_t set_stride = (uint32_t)held(p.batch * pset_bytes);
    const bool keeps = t < tq; // does this lane hold batch rows that exist?
    int which = 0; // parameter buffer of the batch
    int jt = 0;      // local tile of the stage at hand
    // the tile that enters the L2 window when tile jt is done (never, without prefetching)
    const int pf_ahead = held(kDirectTiles + p.prefetch_tiles);
    const int pf_until = held(p.prefetch_tiles > 0 ? ntiles - pf_ahead : 0);
    int pf_turn = pf_ahead % p.splits; // (jt + pf_ahead) mod splits, kept by counting
    for (int first = 0; first < ntiles; first += p.batch)
    {
        const int count = min(p.batch, ntiles - first);
        uint32_t sc_s = pbuf_s + which * pbatch_bytes, zp_s = sc_s + pzp_off;
        uint32_t red_a = red_lane_s;
        const int nst = count * SETS;
        for (int q = 0; q < nst; q += PD)
        {
#pragma unroll
            for (int u = 0; u < PD; u++)
            {
                if (q + u < nst)
                {
                    const int s = u % SETS;
                    float tot[MB][4];
                    compute(buf[u], tile0 + jt, s, sc_s + s * set_stride, zp_s + s * set_stride, tot);
                    if (to_issue > 0)
                        issue(buf[u], s);
                    if (keeps)
                    {
#pragma unroll
                        for (int mb = 0; mb < MB; mb++)
                            sts128(red_a + (uint32_t)(mb * 8 * tq) * 16u,
                                   make_uint4(__float_as_uint(tot[mb][0]), M1 ? 0u : __float_as_uint(tot[mb][1]),
                                              __float_as_uint(tot[mb][2]), M1 ? 0u : __float_as_uint(tot[mb][3])));
                    }
                    red_a += red_step;
                    if (s == SETS - 1)
                    {
                        sc_s += (uint32_t)sm_scale_tile, zp_s += (uint32_t)sm_zp_tile;
                        // keep the L2 window full: warp 0 of the split whose turn it is asks for the tile that
                        // enters it (a handful of instructions per tile; everybody else only skips a branch)
                        if (warp == 0 && jt < pf_until && lane < SETS && pf_turn == my_turn)
                            prefetch_tile(jt + pf_ahead, lane);
                        pf_turn = pf_turn + 1 == p.splits ? 0 : pf_turn + 1;
                        jt++;
                    }
                }
            }
        }
        __syncthreads();
        // everybody has read this batch's parameters: the batch after the next one may land there
        copy_params(first + 2 * p.batch, min(p.batch, max(ntiles - first - 2 * p.batch, 0)), which);
        flush(first, count);
        cp_async_wait_but_one(); // the next batch's parameters (asked for a batch ago) have landed
        __syncthreads();
        which ^= 1;
    }
}

// Raise a kernel's dynamic shared-memory limit once per device (the attribute belongs to the device that is
// current when it is set).
template <int WBITS, int MB, bool XSPLIT, bool DUAL, int PD, int PMODE, bool M1>
cudaError_t ensure_smem(size_t smem)
{
    static size_t configured[nnf::kMaxDevices] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        return e;
    if (dev < 0 || dev >= nnf::kMaxDevices)
        return cudaErrorInvalidDevice;
    if (smem <= std::max(configured[dev], (size_t)48 * 1024))
        return cudaSuccess;
    e = cudaFuncSetAttribute(dq_gemv_direct_kernel<WBITS, MB, XSPLIT, DUAL, PD, PMODE, M1>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
        configured[dev] = smem;
    return e;
}

template <int WBITS, int MB, bool XSPLIT, bool DUAL, int PD, int PMODE, bool M1>
cudaError_t launch(const DirectParams& p_in, const nnf::GemvPlan& plan, cudaStream_t stream)
{
    cudaError_t e = ensure_smem<WBITS, MB, XSPLIT, DUAL, PD, PMODE, M1>(plan.smem_bytes);
    if (e != cudaSuccess)
        return e;
    DirectParams p = p_in;
    if (p.cluster)
    {
        // Clusters only when the device holds all of them at once (asked once per launch shape and device).
        struct Seen
        {
            int dev, splits, threads, ctas;
            size_t smem;
            bool ok;
        };
        static std::mutex mu;
        static Seen seen[64]; // launch shapes asked about so far (a full table answers "no clusters" for new ones)
        static int nseen = 0;
        int dev = 0;
        e = cudaGetDevice(&dev);
        if (e != cudaSuccess)
            return e;
        std::lock_guard<std::mutex> lock(mu);
        const Seen* hit = nullptr;
        for (int i = 0; i < nseen; i++)
        {
            const Seen& q = seen[i];
            if (q.dev == dev && q.splits == plan.splits && q.threads == plan.warps * 32 &&
                q.ctas == plan.ctas_per_split && q.smem == (size_t)plan.smem_bytes)
                hit = &q;
        }
        if (!hit && nseen < 64)
        {
            cudaLaunchConfig_t qc = {};
            qc.gridDim = dim3(plan.ctas_per_split, plan.splits);
            qc.blockDim = dim3(plan.warps * 32);
            qc.dynamicSmemBytes = plan.smem_bytes;
            cudaLaunchAttribute qa[1];
            qa[0].id = cudaLaunchAttributeClusterDimension;
            qa[0].val.clusterDim.x = 1, qa[0].val.clusterDim.y = (unsigned)plan.splits, qa[0].val.clusterDim.z = 1;
            qc.attrs = qa, qc.numAttrs = 1;
            int clusters = 0;
            const cudaError_t qe = cudaOccupancyMaxActiveClusters(
                &clusters, dq_gemv_direct_kernel<WBITS, MB, XSPLIT, DUAL, PD, PMODE, M1>, &qc);
            (void)cudaGetLastError();
            seen[nseen] = Seen{dev, plan.splits, plan.warps * 32, plan.ctas_per_split, (size_t)plan.smem_bytes,
                               qe == cudaSuccess && clusters >= plan.ctas_per_split};
            hit = &seen[nseen++];
        }
        if (!hit || !hit->ok)
            p.cluster = 0;
    }
    (void)cudaGetLastError(); // do not inherit a stale error left behind by an unrelated earlier call
    // Programmatic dependent launch: the CTAs may start while the launch before this one on the stream is still
    // finishing; they stream their weights at once and wait (griddepcontrol.wait) before touching anything else.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.ctas_per_split, plan.splits);
    cfg.blockDim = dim3(plan.warps * 32);
    cfg.dynamicSmemBytes = plan.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    nnf::overlap_attribute(attr, &cfg.numAttrs);
    if (p.cluster)
    {
        attr[cfg.numAttrs].id = cudaLaunchAttributeClusterDimension;
        attr[cfg.numAttrs].val.clusterDim.x = 1;
        attr[cfg.numAttrs].val.clusterDim.y = (unsigned)plan.splits;
        attr[cfg.numAttrs].val.clusterDim.z = 1;
        cfg.numAttrs++;
    }
    cfg.attrs = attr;
    return cudaLaunchKernelEx(&cfg, dq_gemv_direct_kernel<WBITS, MB, XSPLIT, DUAL, PD, PMODE, M1>, p);
}

// Pipeline depth per variant: what the register file holds next to the activation fragments.
#define NNF_DIRECT_FOR_EACH_VARIANT(X)                                                                            \
    X(4, 1, false, false, 2)                                                                                      \
    X(4, 1, false, true, 2)                                                                                       \
    X(4, 1, true, false, 2)                                                                                       \
    X(4, 1, true, true, 2)                                                                                        \
    X(4, 2, false, false, 2)                                                                                      \
    X(4, 2, false, true, 2)                                                                                       \
    X(8, 1, false, false, 2)                                                                                      \
    X(8, 1, false, true, 2)                                                                                       \
    X(8, 1, true, false, 2)                                                                                       \
    X(8, 1, true, true, 2)                                                                                        \
    X(8, 2, false, false, 2)                                                                                      \
    X(8, 2, false, true, 2)                                                                                       \
    X(8, 2, true, false, 2)                                                                                       \
    X(8, 2, true, true, 2)

cudaError_t dispatch(int wbits, const nnf::GemvPlan& plan, const DirectParams& p, cudaStream_t stream)
{
    // the specialised parameter paths exist where they matter: side-by-side pairs for uint4, one group per slice
    // for uint8
#define NNF_X(WB, MBV, XSP, DU, PDV)                                                                              \
    if (wbits == WB && plan.mb == MBV && plan.xsplit == XSP && plan.dual == DU)                                   \
    {                                                                                                             \
        if (p.pmode == 1 && WB == 4)                                                                              \
        {                                                                                                         \
            if (p.M == 1 && MBV == 1 && !XSP) /* the decode case gets its own instantiation */                    \
                return launch<WB, MBV, XSP, DU, PDV, (WB == 4 ? 1 : 0), (MBV == 1 && !XSP)>(p, plan, stream);     \
            return launch<WB, MBV, XSP, DU, PDV, (WB == 4 ? 1 : 0), false>(p, plan, stream);                      \
        }                                                                                                         \
        if (p.pmode == 2 && WB == 8)                                                                              \
            return launch<WB, MBV, XSP, DU, PDV, (WB == 8 ? 2 : 0), false>(p, plan, stream);                      \
        return launch<WB, MBV, XSP, DU, PDV, 0, false>(p, plan, stream);                                          \
    }
    NNF_DIRECT_FOR_EACH_VARIANT(NNF_X)
#undef NNF_X
    return cudaErrorInvalidValue;
}
} // namespace

namespace nnf
{
// Launch shape of the register-pipeline kernel for a descriptor; fills the fields of `plan` that the ring kernel's
// planner leaves alone.  Returns false when the kernel does not serve the descriptor (zero-points removed before the
// multiply).
bool gemv_direct_plan(const nnf_b200_ctx* ctx, const nnf_b200_linear_desc& d, GemvPlan* plan)
{
    if (d.flags & NNF_B200_FLAG_EXACT_ZP)
        return false;
    GemvPlan pl = *plan; // mb, tq, dual, xsplit, row_tiles, slices, tile byte counts come from the common part
    const int sms = ctx ? ctx->sm_count : 148;
    const int smem_cap = ctx ? ctx->smem_optin : 227 * 1024;
    const int sets = pl.dual ? 2 : 1;
    const int pset = pl.pset_bytes; // 0: ragged last tile, parameters by plain loads
    pl.xfrag_bytes = (pl.mb == 2) ? 2 * (pl.xsplit ? 2 : 1) * ((d.w_bits == 4 ? 16 : 8) / 2) * 256 : 0;

    // K splits: every candidate from "as few as 16 warps allow" upwards is rated by how evenly it loads the SMs,
    // in warp-stages per SM against the ideal; more splits cost workspace traffic, so they must earn their place.
    const int smin = (pl.slices + kMaxWarps - 1) / kMaxWarps;
    int best_s = 0, best_per = 0, best_res = 1;
    double best_score = -1.0;
    auto rate = [&](int s) {
        const int warps = (pl.slices + s - 1) / s;
        int resident = std::max(1, std::min(4, kMaxWarps / warps));
        int per_split = std::min(std::max(1, (sms * resident) / s), pl.row_tiles);
        const int steps = (pl.row_tiles + per_split - 1) / per_split;
        const int ctas = per_split * s;
        const int per_sm = (ctas + sms - 1) / sms; // CTAs the busiest SM runs
        const double load = (double)per_sm * steps * warps;
        const double ideal = (double)pl.row_tiles * pl.slices / sms;
        double score = ideal / load - 0.01 * (s - smin);
        if (warps < std::min(8, pl.slices))
            score -= 0.5; // narrow CTAs pay the fixed cost of a CTA (activation fragments, barriers) too often
        if (warps * std::min(resident, per_sm) < 8)
            score -= 0.1; // too few warps per SM to keep enough bytes in flight
        if (s == 2 && smin == 2)
            score += 0.1; // halves of K meet in a cluster's shared memory, finer splits through the workspace: about
                          // 2 us per launch (measured: two [7168,8192] matrices 20.4 us cut 3 ways, 15.8 us in halves)
        if (score > best_score + 1e-9)
            best_score = score, best_s = s, best_per = per_split, best_res = std::min(resident, per_sm);
    };
    if (d.split_k > 0)
    {
        if ((pl.slices + d.split_k - 1) / d.split_k > kMaxWarps)
            return false; // the common planner reports the error
        rate(std::min(d.split_k, pl.slices));
    }
    else
        for (int s = smin; s <= std::min(pl.slices, smin * 4 + 4); s++)
            rate(s);
    if (best_s == 0)
        return false;
    pl.splits = best_s;
    pl.ctas_per_split = best_per;
    pl.warps = (pl.slices + pl.splits - 1) / pl.splits;
    const int steps = (pl.row_tiles + pl.ctas_per_split - 1) / pl.ctas_per_split;
    pl.depth = 2; // stages in the register pipeline (the PD of every instantiated variant)
    // Rows of scales / zero-points in shared memory: whole rows, or, when K is split and the rows are whole 16-byte
    // pieces, only the pieces with the columns of a CTA's own K range (the widest range over the splits).
    {
        const int group = d.group_size > 0 ? d.group_size : d.K;
        const int G = d.K / group, sbytes = d.scale_dtype == NNF_B200_F32 ? 4 : 2;
        const int sc_row = G * sbytes, zp_row = d.w_bits == 4 ? (G + 1) / 2 : G;
        pl.sm_sc_row = sc_row, pl.sm_zp_row = zp_row;
        pl.range_layout = pset > 0 && pl.splits > 1 && sc_row % 16 == 0 && zp_row % 16 == 0;
        if (pl.range_layout)
        {
            const int lo = pl.slices / pl.splits, rem = pl.slices % pl.splits;
            int sc_pieces = 0, zp_pieces = 0;
            for (int i = 0; i < pl.splits; i++)
            {
                const ParamRange r = param_range(i * lo + std::min(i, rem), lo + (i < rem ? 1 : 0),
                                                 d.w_bits == 4 ? 256 : 128, d.K, group, sbytes, d.w_bits, sc_row, zp_row);
                sc_pieces = std::max(sc_pieces, r.sc_pieces), zp_pieces = std::max(zp_pieces, r.zp_pieces);
            }
            pl.sm_sc_row = 16 * sc_pieces, pl.sm_zp_row = 16 * zp_pieces;
        }
        pl.pset_sm = pset > 0 ? 16 * (pl.sm_sc_row + pl.sm_zp_row) : 0;
    }
    // The longest batch whose parameters (two buffers, or one when a single batch holds every tile of a CTA) and
    // partial sums fit next to `best_res` CTAs per SM: every batch ends with a reduction over the warps during which
    // no weight is asked for, 2.5 to 3 us each.
    pl.batch = 0;
    for (int b = std::min(kBatch, steps); b >= 1; b--)
    {
        if (b < steps && (b * sets) % pl.depth != 0)
            continue; // every batch but the last is a whole number of trips through the register pipeline
        const int nbuf = b >= steps ? 1 : 2;
        if ((int)DirectSmem(sets, pl.mb, pl.warps, b, pl.tq, pl.pset_sm, pl.xfrag_bytes, nbuf).total + 1024 <=
            smem_cap / best_res)
        {
            pl.batch = b;
            pl.param_bufs = nbuf;
            break;
        }
    }
    if (pl.batch == 0)
        return false;
    pl.smem_bytes = DirectSmem(sets, pl.mb, pl.warps, pl.batch, pl.tq, pl.pset_sm, pl.xfrag_bytes, pl.param_bufs).total;
    // K split 2 to 8 ways: the splits of a tile as one cluster, if the sums' meeting place fits as well.  The launch
    // falls back to the workspace when the device cannot hold every cluster at once: 148 SMs hold 74 clusters of 2
    // one-per-SM CTAs but only 45 of 3, 33 of 4, 26 of 5, 22 of 6 and 15 of 7 or 8 (the occupancy calculator's
    // answers), so in practice halves of K meet in shared memory and finer splits do when a split has few CTAs.
    pl.cluster = 0;
#ifndef NNF_NO_CLUSTER
    if (pl.splits >= 2 && pl.splits <= 8)
    {
        const size_t with = DirectSmem(sets, pl.mb, pl.warps, pl.batch, pl.tq, pl.pset_sm, pl.xfrag_bytes, pl.param_bufs,
                                       pl.splits).total;
        if ((int)with + 1024 <= smem_cap / best_res)
            pl.cluster = 1, pl.smem_bytes = with;
    }
#endif
    // L2 window ahead of the register pipeline: about 192 KB per CTA (whole tiles, shared by the K splits)
    const int row_bytes = d.w_bits == 4 ? d.K / 2 : d.K;
    pl.prefetch_tiles = std::max(1, std::min(64, (192 * 1024 * pl.splits) / (sets * 16 * row_bytes)));
    // Weight loads that take lines in L1, measured over 36 projection shapes: launches whose K is cut 5 and more
    // ways gain 8 to 21 %, two-matrix launches of more weight bytes than L2 holds gain 7 to 27 %; every other launch
    // is up to 9 % faster without (its loads come back sooner, and it is too short or too narrow to be bound by
    // the bytes an SM keeps in flight).
    const size_t weight_bytes = (size_t)sets * d.N * row_bytes;
    pl.l1_lines = (pl.splits >= 5 && steps >= 8) || (pl.dual && weight_bytes >= ((size_t)128 << 20));
    pl.slot_floats = (size_t)sets * pl.mb * 128 + 8 * pl.mb;
    pl.workspace_bytes = 0;
    if (pl.splits > 1)
    {
        const size_t cnt = ((size_t)pl.row_tiles * sizeof(unsigned) + 255) / 256 * 256;
        pl.workspace_bytes = cnt + (size_t)pl.splits * pl.row_tiles * pl.slot_floats * sizeof(float);
    }
    pl.direct = 1;
    *plan = pl;
    return true;
}

cudaError_t gemv_direct_dispatch(const nnf_b200_linear_desc& d, const GemvPlan& plan, const void* x,
                                 const nnf_b200_qweight* w, const nnf_b200_qweight* w2, const void* gain,
                                 const void* bias, void* y, int* status, void* workspace, cudaStream_t stream,
                                 const nnf_b200_peers* peers)
{
    DirectParams p{};
    if (peers && peers->world > 1)
    {
        if (plan.dual)
            return cudaErrorInvalidValue;
        for (int r = 0; r < peers->world; r++)
        {
            p.ar_bufs[r] = static_cast<const char*>(peers->bufs[r]);
            p.ar_flags[r] = static_cast<uint32_t*>(peers->flags[r]);
        }
        p.ar_half_stride = peers->half_stride_bytes;
        p.ar_epoch = peers->epoch;
        p.ar_rank = peers->rank, p.ar_world = peers->world;
    }
    const int ue = (d.w_bits == 4) ? 128 : 64;
    p.wq[0] = static_cast<const uint8_t*>(w->wq);
    p.scale[0] = w->scale;
    p.zp[0] = static_cast<const uint8_t*>(w->zp);
    p.wq[1] = p.wq[0], p.scale[1] = p.scale[0], p.zp[1] = p.zp[0];
    if (plan.dual)
    {
        p.wq[1] = static_cast<const uint8_t*>(w2->wq);
        p.scale[1] = w2->scale;
        p.zp[1] = static_cast<const uint8_t*>(w2->zp);
    }
    p.row_bytes = (d.w_bits == 4) ? d.K / 2 : d.K;
    p.x = x;
    p.gain = static_cast<const float*>(gain);
    p.bias = static_cast<const float*>(bias);
    p.y = y;
    p.status = status;
    p.M = d.M, p.N = d.N, p.K = d.K;
    p.group = d.group_size > 0 ? d.group_size : d.K;
    p.G = d.K / p.group;
    p.zp_row_bytes = (d.w_bits == 4) ? (p.G + 1) / 2 : p.G;
    p.units = d.K / ue;
    p.row_tiles = plan.row_tiles;
    p.splits = plan.splits;
    p.slices_lo = plan.slices / plan.splits, p.slices_rem = plan.slices % plan.splits;
    p.tiles_lo = plan.row_tiles / plan.ctas_per_split, p.tiles_rem = plan.row_tiles % plan.ctas_per_split;
    p.x_f32 = d.x_dtype == NNF_B200_F32;
    p.y_f32 = d.y_dtype == NNF_B200_F32;
    p.scale_f32 = d.scale_dtype == NNF_B200_F32;
    p.rmsnorm = d.prologue == NNF_B200_PROLOGUE_RMSNORM;
    p.has_addend = d.epilogue == NNF_B200_EPILOGUE_ADD;
    p.has_bias = bias != nullptr && !p.has_addend;
    p.eps = d.rms_eps;
    p.batch = plan.batch;
    p.tq = plan.tq;
    p.scale_tile_bytes = plan.scale_tile_bytes;
    p.zp_tile_bytes = plan.zp_tile_bytes;
    p.xfrag_bytes = plan.xfrag_bytes;
    p.prefetch_tiles = plan.prefetch_tiles;
    p.l1_lines = plan.l1_lines;
    p.slot_floats = (int)plan.slot_floats;
    // Bulk copies of the quantisation parameters need whole tiles inside the tensors and 16-byte aligned sources.
    auto ok16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
    p.bulk_params = plan.pset_bytes > 0 && ok16(w->scale) && ok16(w->zp) &&
                    (!plan.dual || (ok16(w2->scale) && ok16(w2->zp)));
    {
        const DirectSmem lay(plan.dual ? 2 : 1, plan.mb, plan.warps, plan.batch, plan.tq,
                             p.bulk_params ? plan.pset_sm : 0, plan.xfrag_bytes, plan.param_bufs,
                             plan.cluster ? plan.splits : 0);
        p.off_bars = (int)lay.params;
        p.off_red = p.off_bars + (int)lay.bars;
        p.off_ss = p.off_red + (int)lay.red;
        p.off_flags = p.off_ss + (int)lay.ss;
        p.off_cslots = p.off_flags + (int)lay.flags + (int)lay.xsm;
        p.cluster = plan.cluster;
    }
    p.group_units = p.group / ue;
    p.group_magic = p.group_units > 1 ? (uint32_t)((0x100000000ull + p.group_units - 1) / p.group_units) : 0u;
    p.sc_row_bytes = p.G * (p.scale_f32 ? 4 : 2);
    p.range_params = p.bulk_params && plan.range_layout;
    p.sm_sc_row = plan.sm_sc_row, p.sm_zp_row = plan.sm_zp_row;
    p.pmode = 0;
    if (p.bulk_params && d.w_bits == 4 && p.group == 128 && !p.scale_f32 && (p.G & 1) == 0)
        p.pmode = 1;
    else if (p.bulk_params && p.group % (2 * ue) == 0)
        p.pmode = 2;
    if (plan.splits > 1)
    {
        const size_t cnt = ((size_t)plan.row_tiles * sizeof(unsigned) + 255) / 256 * 256;
        p.ws_count = static_cast<unsigned*>(workspace);
        p.ws_slots = reinterpret_cast<float*>(static_cast<char*>(workspace) + cnt);
    }
    return dispatch(d.w_bits, plan, p, stream);
}
} // namespace nnf
