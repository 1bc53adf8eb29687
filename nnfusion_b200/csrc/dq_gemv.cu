// Small-M (decode) dequantize-fused linear for sm_100a:  y[M,N] = epi(pro(x)[M,K] . dequant(W)[N,K]^T), M <= 16.
//
// Fused replacement of the reference's Convert -> Subtract -> Multiply element-wise kernels
// (src/nnfusion/core/kernels/cuda_gpu/kernels/elementwise.hpp:33-157, elementwise_fused.cpp:42-189)
// followed by the cuBLAS Dot (src/nnfusion/core/kernels/cuda_gpu/kernels/dot.cpp:27-372): the
// weights are read once, at their packed size, and never materialised in fp32.
//
// The kernel is HBM-bound and, next to that, bound by instruction issue and by the latency of whatever sits between
// the start of the CTA and its first arithmetic; its shape follows from all three:
//   * a weight row is cut into 128-byte "slices" (256 uint4 / 128 uint8 elements).  Warp w of a CTA owns slice
//     (first slice of the CTA's K range + w) for the whole launch, so the activations it needs are loaded once and
//     live in registers as mma B fragments (fp16 activations are only permuted, never converted);
//   * CTAs are persistent: CTA c of a K split walks over the 16-row tiles c, c + P, c + 2P ...  A warp of its own
//     asks for the data with bulk copies (cp.async.bulk, no tensor map to fetch first): one per weight row and tile
//     for the CTA's K range, two for the tile's scales and zero-points, all counted on one mbarrier per ring slot.
//     Rows sit 64 bytes (mod 128) apart in shared memory, which keeps the 16-byte fragment loads free of bank
//     conflicts.  The ring is as deep as shared memory allows, for small problems deep enough to hold the CTA's
//     whole share, so that every byte is requested at once; nothing on the critical path is a dependent global load;
//   * nibbles/bytes become exact fp16 integers with one LOP3/PRMT per pair (the 0x6400 / 0x5400 exponent trick)
//     and feed mma.sync.m16n8k16 with W as the 16-row operand and up to 8 batch rows as the 8-column operand (the
//     contraction index is permuted identically on both sides, so nothing is shuffled); accumulation is fp32 and
//     the group scale multiplies the fp32 sum of each 64-byte unit, i.e. sum((q - zp) * x) * scale;
//   * warps never meet inside a batch of tiles: each keeps its partial sums in shared memory and hands its ring slot
//     back through an mbarrier.  Once per batch the partial sums of the CTA's warps are added in a fixed order;
//     with split-K each split stores its tile sums into its own workspace slot and the split that arrives last (a
//     counter per tile) adds the slots in a fixed order, so results are bitwise repeatable.  Nothing ever waits on
//     another CTA, and every mbarrier wait is bounded.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "nnf_internal.h"
#include "sm100_ptx.cuh"

namespace
{
using namespace nnf::ptx;

constexpr int kMaxWarps = 16;
constexpr int kBatch = 16;           // most row tiles between two reductions over the warps
constexpr int kMaxDepth = 8;         // deepest load ring

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
    int* status; // device status word: set to 1 when a bounded wait gave up
    int M, N, K;
    int group, G, zp_row_bytes;
    int units;  // 64-byte units per weight row
    int slices; // ceil(units / 2)
    int row_tiles, splits, ctas_per_split;
    int slices_lo, slices_rem; // slices / splits and its remainder
    int steps_lo, steps_rem;   // row_tiles / ctas_per_split and its remainder
    int x_f32, y_f32, scale_f32, rmsnorm, has_bias;
    int has_addend; // bias points at an [M,N] tensor of y's type instead of fp32 [N]
    int depth;       // ring depth in row tiles
    int batch;       // row tiles between two reductions over the warps (<= kBatch)
    int tq;          // accumulator column pairs kept: 1, 2 or 4, at least ceil(min(M, 8) / 2); 4 when M > 8
    int row_bytes;   // bytes of one packed weight row
    int bulk_params; // scales / zero-points of a tile arrive by bulk copy in shared memory
    int lsu_weights; // weights arrive by per-thread cp.async (each thread fetches exactly the bytes it will read)
                     // instead of bulk copies: the bulk-copy engine moves 16 bytes per clock and SM, which caps a
                     // launch at 4.6 TB/s over 148 SMs
    int scale_tile_bytes, zp_tile_bytes, pset_bytes; // per tile and weight set
    int xfrag_bytes; // shared memory per warp for the activation fragments of batch rows 8..15 (0 when M <= 8)
    // Sum over the ranks of a tensor-parallel group inside this launch (ar_world > 1): see the end of flush().
    const char* ar_bufs[8]; // every rank's fp32 partial-output buffer (two halves), own included, as mapped here
    uint32_t* ar_flags[8];  // every rank's flag words [row tile][sender], then one call counter per row tile
    size_t ar_half_stride;  // bytes between the two halves of a buffer
    uint32_t ar_epoch;      // call number from the host, or 0: counted in the words after the flags
    int ar_rank, ar_world;
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
// A constant the compiler cannot see through, so that it stays in its register.
__device__ __forceinline__ uint32_t held_constant(uint32_t v)
{
    uint32_t r;
    asm volatile("mov.u32 %0, %1;" : "=r"(r) : "r"(v));
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

// Untiled bulk copy global -> shared: both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
                 : "memory");
}
template <int OFF>
__device__ __forceinline__ uint4 lds128_at(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr), "n"(OFF));
    return v;
}
__device__ __forceinline__ unsigned short lds_u16(uint32_t addr)
{
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u8(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit()
{
    asm volatile("cp.async.commit_group;" ::: "memory");
}
// Wait until at most n of this thread's most recent groups are still in flight (n < 8).
__device__ __forceinline__ void cp_async_wait(int n)
{
    switch (n)
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
__device__ __forceinline__ void named_barrier(int id, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

template <int WBITS>
struct Fmt
{
    static constexpr int UE = (WBITS == 4) ? 128 : 64; // elements per 64-byte unit
    static constexpr int LE = UE / 4;                  // elements per lane per 16-byte chunk
    static constexpr int NF = LE / 2;                  // half2 fragments per chunk
};

// Shared-memory footprint, shared by host and device.  All sizes in bytes.
struct SmemLayout
{
    size_t ring, pring, bars, red, ss, flags, xsm, total;
    // xfrag_bytes: activation fragments of batch rows 8..15 kept per warp in shared memory (0 when M <= 8)
    __host__ __device__ SmemLayout(int sets, int mb, int warps, int depth, int batch, int tq, int pset_bytes,
                                   int xfrag_bytes)
    {
        ring = (size_t)depth * sets * 16 * (warps * 128 + 64);
        pring = (size_t)depth * sets * pset_bytes;
        bars = 8 * 2 * kMaxDepth;
        red = sizeof(float) * (size_t)warps * batch * sets * mb * 8 * tq * 4;
        ss = sizeof(float) * ((size_t)warps * 8 * mb + 8 * mb);
        flags = sizeof(int) * (2 * kBatch + 4); // last-arriver flags, call numbers, "all peers answered"
        xsm = (size_t)warps * xfrag_bytes;
        total = ring + pring + bars + red + ss + flags + xsm;
    }
};

// EXACT = true : zero-points are removed from the fp16 integers before the multiply (bit-exact integers into the
//                tensor core).
// EXACT = false: the tensor core multiplies x by (offset + q) and the offset and zero-point are taken out of the
//                fp32 sum afterwards, acc - (C1 + zp * C2), with C1 = sum(offset_k * x_k), C2 = sum(x_k) over the
//                64-byte unit.  Same fp32 accumulation, about 40 % fewer unpack instructions.
// FAST = true : the quantisation parameters of every tile arrive in shared memory and the scales are fp16 (the
//                caller checks both); the inner loop then contains no choice that depends on the launch.
template <int WBITS, int MB, bool XSPLIT, bool DUAL, bool EXACT, bool FAST>
__global__ void __launch_bounds__((kMaxWarps + 1) * 32, 1)
    dq_gemv_kernel(const GemvParams p)
{
    using F = Fmt<WBITS>;
    constexpr int SETS = DUAL ? 2 : 1;
    constexpr int XS = XSPLIT ? 2 : 1;
    constexpr int NF = F::NF;
    constexpr int MPAD = 8 * MB;
    // 16 batch rows, one weight set: the B fragments of rows 8..15 are parked in shared memory (see xsm_s below).
    // With two weight sets the ring needs that memory more than the registers need relief (measured).
    constexpr bool XSM = (MB == 2) && !DUAL;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // The next launch on the stream may start as soon as SMs become free (it waits for this grid's results itself).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int nwarps = (blockDim.x >> 5) - 1; // arithmetic warps; the last warp of the CTA only asks for data
    const int nthreads = nwarps * 32;
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int tq = p.tq;
    const int tq_shift = tq >> 1;                        // tq is 1, 2 or 4
    const int pt_shift = 5 + tq_shift + (MB == 2 ? 1 : 0);
    const int per_tile = 1 << pt_shift; // MB * 8 * tq * 4 floats: one warp's partial sums of one tile and weight set

    // ring: [depth][SETS][16 rows] of (nwarps * 128 + 64) bytes, warp w's 128 bytes of a row at w * 128; then per
    // slot and set the tile's scales and zero-points
    const SmemLayout lay(SETS, MB, nwarps, p.depth, p.batch, tq, p.pset_bytes, p.xfrag_bytes);
    // (pointers stay derived from the array itself, never from an integer, so that every access below is compiled
    // as a shared-memory access with a 32-bit address rather than as a generic one)
    uint8_t* ring = smem_raw;
    uint8_t* pring = ring + lay.ring;
    uint64_t* bars = reinterpret_cast<uint64_t*>(pring + lay.pring); // full[kMaxDepth], empty[kMaxDepth]
    float* red = reinterpret_cast<float*>(bars + 2 * kMaxDepth);     // [nwarps][batch][SETS][per_tile]
    float* ss_w = red + lay.red / sizeof(float);                     // [nwarps][MPAD]
    float* ss_cta = ss_w + nwarps * MPAD;                            // [MPAD]
    int* last_flag = reinterpret_cast<int*>(ss_cta + MPAD);          // [kBatch]
    // With 16 batch rows the B fragments of rows 8..15 do not fit the register file next to those of rows 0..7
    // (96 registers per thread): they live here, [warp][unit][xs][fragment pair][lane] x 8 bytes, and every product
    // fetches its pair with one conflict-free 8-byte load.
    uint32_t* ep_s = reinterpret_cast<uint32_t*>(last_flag + kBatch); // [kBatch] call number per tile of the batch
    int* ar_ok = reinterpret_cast<int*>(ep_s + kBatch);               // have all peers answered?
    const uint32_t xsm_s = smem_u32(ar_ok + 4) + (uint32_t)(warp * p.xfrag_bytes) + (uint32_t)lane * 8u;
    const uint32_t ring_s = smem_u32(ring), pring_s = smem_u32(pring);
    // Shared-memory bytes between two rows of a tile.  When a CTA takes whole rows, a tile is one contiguous piece of
    // memory and arrives with a single copy, rows back to back (the fragment loads then pay a two-way bank conflict,
    // which is cheap next to sixteen separate copies).
    const bool lsu = p.lsu_weights != 0;
    const bool use_full = !lsu || p.bulk_params; // does anything arrive through the slots' "full" barriers?
    const bool whole_rows = !lsu && p.splits == 1 && p.row_bytes == nwarps * 128;
    const int row_stride = whole_rows ? nwarps * 128 : nwarps * 128 + 64;
    const uint32_t full_s = smem_u32(bars), empty_s = full_s + 8 * kMaxDepth;

    // grid = (CTAs per split, splits); quotients come from the host: nothing here waits for an integer division
    const int split = blockIdx.y, cta_in_split = blockIdx.x;
    const int my_slices = p.slices_lo + (split < p.slices_rem ? 1 : 0); // K ranges differ by at most one slice
    const int slice0 = split * p.slices_lo + min(split, p.slices_rem);
    const int slice = slice0 + warp;
    const bool has_slice = warp < my_slices;
    const int nsteps = p.steps_lo + (cta_in_split < p.steps_rem ? 1 : 0);

    // ---------------------------------------------------------------- producer (last warp of the CTA)
    // Per row tile: for every row that exists the CTA's K range of the packed weights, and the tile's quantisation
    // parameters, all counted on the slot's barrier.  expect() is called by one lane, copy() by the whole warp.
    const int seg_bytes = min(my_slices * 128, p.row_bytes - slice0 * 128);
    auto tile_rows = [&](int step) { return min(16, p.N - (cta_in_split + step * p.ctas_per_split) * 16); };
    auto expect = [&](int step) {
        uint32_t bytes = lsu ? 0u : (uint32_t)(SETS * tile_rows(step) * seg_bytes);
        if (p.bulk_params)
            bytes += (uint32_t)(SETS * (p.scale_tile_bytes + p.zp_tile_bytes));
        mbar_arrive_expect_tx(full_s + 8 * (step % p.depth), bytes);
    };
    auto copy = [&](int step) {
        const int slot = step % p.depth;
        const uint32_t bar = full_s + 8 * slot;
        const int tile = cta_in_split + step * p.ctas_per_split;
        const int rows = tile_rows(step);
        if (lsu)
        {
            // the arithmetic warps fetch their own weights
        }
        else if (whole_rows)
        {
            if (lane < SETS)
                bulk_load(ring_s + (uint32_t)((slot * SETS + lane) * 16 * row_stride),
                          (lane == 0 ? p.wq[0] : p.wq[1]) + (size_t)(tile * 16) * p.row_bytes,
                          (uint32_t)(rows * p.row_bytes), bar);
        }
        else
        {
            for (int c = lane; c < SETS * 16; c += 32)
            {
                const int s = c >> 4, r = c & 15;
                if (r < rows)
                    bulk_load(ring_s + (uint32_t)(((slot * SETS + s) * 16 + r) * row_stride),
                              (s == 0 ? p.wq[0] : p.wq[1]) + (size_t)(tile * 16 + r) * p.row_bytes +
                                  (size_t)slice0 * 128,
                              (uint32_t)seg_bytes, bar);
            }
        }
        if (p.bulk_params && lane >= 32 - 2 * SETS)
        {
            const int c = lane - (32 - 2 * SETS), s = c >> 1;
            const uint32_t pd = pring_s + (uint32_t)((slot * SETS + s) * p.pset_bytes);
            if (c & 1)
                bulk_load(pd + (uint32_t)p.scale_tile_bytes, p.zp[s] + (size_t)tile * p.zp_tile_bytes,
                          (uint32_t)p.zp_tile_bytes, bar);
            else
                bulk_load(pd, static_cast<const char*>(p.scale[s]) + (size_t)tile * p.scale_tile_bytes,
                          (uint32_t)p.scale_tile_bytes, bar);
        }
    };
    if (warp == nwarps)
    {
        // A warp of its own: asking for data never waits for anybody's activation loads, and the arithmetic warps
        // never wait for the requests to be issued.  The first ring-full leaves at once; slots are then refilled
        // as the arithmetic warps hand them back.
        if (lane < p.depth)
        {
            // lane i owns ring slot i: barrier operations take tens of nanoseconds each, so they run side by side
            mbar_init(full_s + 8 * lane, 1);
            mbar_init(empty_s + 8 * lane, (uint32_t)nwarps);
            fence_barrier_init();
            if (lane < nsteps && use_full)
                expect(lane);
        }
        __syncwarp();
        asm volatile("bar.arrive 2, %0;" ::"r"(nthreads + 32) : "memory"); // barriers are ready
        if (!use_full)
            return; // nothing travels through the slots' barriers
        for (int i = 0; i < p.depth && i < nsteps; i++)
            copy(i);
        bool gave_up = false;
        for (int st = p.depth; st < nsteps; st++)
        {
            if (lane == 0)
            {
                if (!mbar_wait(empty_s + 8 * (st % p.depth), (uint32_t)(st / p.depth - 1) & 1u))
                    gave_up = true;
                expect(st);
            }
            __syncwarp();
            copy(st);
        }
        if (gave_up)
            atomicExch(p.status, 1);
        return;
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
    // Shared-memory addresses that never change for this lane: its 16 bytes of rows g / g + 8 of slot 0 (unit 1
    // sits 64 bytes further).
    const uint32_t wrow[2] = {ring_s + (uint32_t)(warp * 128 + g * row_stride + t * 16),
                              ring_s + (uint32_t)(warp * 128 + (g + 8) * row_stride + t * 16)};
    const uint32_t wset_bytes = (uint32_t)(16 * row_stride);
    // With per-thread fetching a thread asks for exactly the four 16-byte pieces per weight set that it will read,
    // so no other thread is involved and no barrier guards them: cp.async groups, one per tile, the ring's depth
    // in flight.  Rows past N read row N - 1 (never stored); a unit past the end of the row is skipped (its
    // activations are zero and the unpacking makes finite numbers of any bits).
    auto fetch_tile = [&](int step) {
        const int slot = step % p.depth;
        const int tile = cta_in_split + step * p.ctas_per_split;
#pragma unroll
        for (int s = 0; s < SETS; s++)
#pragma unroll
            for (int h = 0; h < 2; h++)
            {
                const int row = min(tile * 16 + g + 8 * h, p.N - 1);
                const uint8_t* src = (s == 0 ? p.wq[0] : p.wq[1]) + (size_t)row * p.row_bytes + slice * 128 + t * 16;
                const uint32_t dst = wrow[h] + (uint32_t)(slot * SETS + s) * wset_bytes;
                if (unit_ok[0])
                    cp_async16(dst, src);
                if (unit_ok[1])
                    cp_async16(dst + 64, src + 64);
            }
    };
    if (lsu)
    {
        // The first tile leaves before anything else happens (weights are constants: this needs no
        // griddepcontrol.wait).  The rest of the ring follows once the activation loads are out, which would
        // otherwise queue behind 160 KB of weights.  One group per slot, empty ones included, keeps the count uniform.
        if (nsteps > 0 && has_slice)
            fetch_tile(0);
        cp_async_commit();
    }

    // Byte offsets of this lane's scales / zero-points inside a slot's parameter block: rows g and g + 8 of the
    // tile, groups of the two units of the slice.
    const int sbytes = p.scale_f32 ? 4 : 2;
    int soff[2][2], zoff[2][2];
#pragma unroll
    for (int l = 0; l < 2; l++)
#pragma unroll
        for (int h = 0; h < 2; h++)
        {
            soff[l][h] = ((g + 8 * h) * p.G + grp_of[l]) * sbytes;
            zoff[l][h] = p.scale_tile_bytes + (g + 8 * h) * p.zp_row_bytes + (WBITS == 4 ? grp_of[l] >> 1 : grp_of[l]);
        }

    // Everything above reads only constants (weights, scales, zero-points).  The activations, the output and the
    // workspace may belong to the launch before this one on the stream: when this kernel was launched as its
    // programmatic dependent, it has been running beside that launch's tail until here.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---------------------------------------------------------------- activations -> B fragments in registers
    uint32_t xf[2][MB][XS][NF];
    float c1[2][MB][2], c2[2][MB][2]; // offset / zero-point corrections for accumulator columns 2t, 2t+1
    float ss_local[MB];
#pragma unroll
    for (int mb = 0; mb < MB; mb++)
        ss_local[mb] = 0.f;
    const bool plain = !XSPLIT && !p.x_f32 && !p.rmsnorm; // fp16 activations used as they are
    // fp16 activations: all loads first, so that they are on their way before the bulk of the weight requests
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
                                                                 unit_of[l] * F::UE + t * F::LE);
#pragma unroll
                for (int j = 0; j < F::LE / 8; j++)
                    xraw[l][mb][j] = (unit_ok[l] && m < p.M) ? __ldg(src + j) : make_uint4(0u, 0u, 0u, 0u);
            }
    }
    if (lsu)
    {
        for (int i = 1; i < p.depth; i++)
        {
            if (i < nsteps && has_slice)
                fetch_tile(i);
            cp_async_commit();
        }
    }
#pragma unroll
    for (int l = 0; l < 2; l++)
    {
        const int k0 = unit_of[l] * F::UE + t * F::LE;
#pragma unroll
        for (int mb = 0; mb < MB; mb++)
        {
            const int m = g + 8 * mb;
            const bool live = unit_ok[l] && m < p.M;
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
                        xf[l][mb][0][4 * j + 0] = __byte_perm(v.x, v.z, 0x5410);
                        xf[l][mb][0][4 * j + 1] = __byte_perm(v.x, v.z, 0x7632);
                        xf[l][mb][0][4 * j + 2] = __byte_perm(v.y, v.w, 0x5410);
                        xf[l][mb][0][4 * j + 3] = __byte_perm(v.y, v.w, 0x7632);
                    }
                    else
                    {
                        xf[l][mb][0][4 * j + 0] = v.x, xf[l][mb][0][4 * j + 1] = v.y;
                        xf[l][mb][0][4 * j + 2] = v.z, xf[l][mb][0][4 * j + 3] = v.w;
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
                    xf[l][mb][0][f] = pack_h2(hi[e0], hi[e1]);
                    if (XSPLIT)
                        xf[l][mb][XS - 1][f] = pack_h2(lo[e0], lo[e1]);
                }
            }
            if (!EXACT)
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
                            mma16816_first(d, off_even, ones, off_odd, ones, xf[l][mb][xsn][f], xf[l][mb][xsn][f + 1]);
                        else
                            mma16816(d, off_even, ones, off_odd, ones, xf[l][mb][xsn][f], xf[l][mb][xsn][f + 1]);
                    }
                c1[l][mb][0] = d[0], c1[l][mb][1] = d[1];
                c2[l][mb][0] = d[2], c2[l][mb][1] = d[3];
            }
            if (XSM && mb == 1)
            {
                // park the fragments of batch rows 8..15 in shared memory right away: their registers are needed
#pragma unroll
                for (int xsn = 0; xsn < XS; xsn++)
#pragma unroll
                    for (int f = 0; f < NF; f += 2)
                        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(
                                         xsm_s + (uint32_t)(((l * XS + xsn) * (NF / 2) + f / 2) * 256)),
                                     "r"(xf[l][1][xsn][f]), "r"(xf[l][1][xsn][f + 1])
                                     : "memory");
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
    asm volatile("bar.sync 2, %0;" ::"r"(nthreads + 32) : "memory"); // ring barriers initialised, ss_w visible
    if (p.rmsnorm)
    {
        if (tid < MPAD)
        {
            float v = 0.f;
            for (int w = 0; w < nwarps; w++)
                v += ss_w[w * MPAD + tid];
            ss_cta[tid] = v;
        }
        named_barrier(1, nthreads);
    }

    // ---------------------------------------------------------------- arithmetic on one landed row tile
    auto row_of = [&](int step, int h) { return min((cta_in_split + step * p.ctas_per_split) * 16 + g + 8 * h, p.N - 1); };
    float tot[SETS][MB][4];
    const uint32_t k6400 = held_constant(0x64006400u), k5400 = held_constant(0x54005400u);
    // This lane's scales / zero-points in slot 0's parameter block.
    uint32_t sa[2][2], za[2][2];
#pragma unroll
    for (int l = 0; l < 2; l++)
#pragma unroll
        for (int h = 0; h < 2; h++)
            sa[l][h] = pring_s + (uint32_t)soff[l][h], za[l][h] = pring_s + (uint32_t)zoff[l][h];
    const int zsh[2] = {(WBITS == 4) ? 4 * (grp_of[0] & 1) : 0, (WBITS == 4) ? 4 * (grp_of[1] & 1) : 0};
    const bool one_col = p.M == 1; // only accumulator column 0 carries a batch row

    auto compute = [&](int step, int slot) {
#pragma unroll
        for (int s = 0; s < SETS; s++)
        {
            // (scale, zero-point) of rows g / g+8 for both halves of the slice
            float sc[2][2];
            uint32_t zq[2][2];
            if (FAST)
            {
                const uint32_t pb = (uint32_t)((slot * SETS + s) * p.pset_bytes);
#pragma unroll
                for (int l = 0; l < 2; l++)
#pragma unroll
                    for (int h = 0; h < 2; h++)
                    {
                        sc[l][h] = __half2float(__ushort_as_half(lds_u16(sa[l][h] + pb)));
                        zq[l][h] = (WBITS == 4) ? (lds_u8(za[l][h] + pb) >> zsh[l]) & 0xFu : lds_u8(za[l][h] + pb);
                    }
            }
            else if (p.bulk_params)
            {
                const uint8_t* pb = pring + (size_t)(slot * SETS + s) * p.pset_bytes;
#pragma unroll
                for (int l = 0; l < 2; l++)
#pragma unroll
                    for (int h = 0; h < 2; h++)
                    {
                        sc[l][h] = p.scale_f32 ? *reinterpret_cast<const float*>(pb + soff[l][h])
                                               : __half2float(*reinterpret_cast<const __half*>(pb + soff[l][h]));
                        const uint32_t zb = pb[zoff[l][h]];
                        zq[l][h] = (WBITS == 4) ? (zb >> zsh[l]) & 0xFu : zb;
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
                            zq[l][h] = (__ldg(p.zp[s] + (size_t)row * p.zp_row_bytes + (grp_of[l] >> 1)) >> zsh[l]) & 0xFu;
                        else
                            zq[l][h] = __ldg(p.zp[s] + sidx);
                    }
                }
            }
            // this lane's 16 bytes of rows g / g+8, both units of the warp's slice
            const uint32_t wb = (uint32_t)(slot * SETS + s) * wset_bytes;
            uint32_t wq[2][2][4]; // [unit][row half][word]
#pragma unroll
            for (int l = 0; l < 2; l++)
#pragma unroll
                for (int h = 0; h < 2; h++)
                {
                    const uint4 v = l ? lds128_at<64>(wrow[h] + wb) : lds128_at<0>(wrow[h] + wb);
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
                        const uint32_t w = wq[l][h][w4];
                        if (WBITS == 4)
                        {
                            const uint32_t w8 = w >> 8;
                            a[h][0] = and_or<0x000F000Fu>(w, k6400);  // 1024 + (n0, n4)
                            a[h][1] = and_or<0x00F000F0u>(w, k5400);  //   64 + (n1, n5)
                            a[h][2] = and_or<0x000F000Fu>(w8, k6400); // 1024 + (n2, n6)
                            a[h][3] = and_or<0x00F000F0u>(w8, k5400); //   64 + (n3, n7)
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
                            {
                                uint32_t b0, b1;
                                if (!XSM || mb == 0)
                                    b0 = xf[l][mb][xsn][f], b1 = xf[l][mb][xsn][f + 1];
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
            float zf[2][2];
#pragma unroll
            for (int l = 0; l < 2; l++)
#pragma unroll
                for (int h = 0; h < 2; h++)
                    zf[l][h] = (float)zq[l][h];
            auto finish_col = [&](int mb, int c) {
                float u0 = acc[0][mb][c], u1 = acc[1][mb][c];
                if (!EXACT)
                {
                    u0 -= fmaf(zf[0][c >> 1], c2[0][mb][c & 1], c1[0][mb][c & 1]);
                    u1 -= fmaf(zf[1][c >> 1], c2[1][mb][c & 1], c1[1][mb][c & 1]);
                }
                tot[s][mb][c] = fmaf(sc[1][c >> 1], u1, sc[0][c >> 1] * u0);
            };
#pragma unroll
            for (int mb = 0; mb < MB; mb++)
            {
                finish_col(mb, 0);
                finish_col(mb, 2);
                if (!one_col)
                {
                    finish_col(mb, 1);
                    finish_col(mb, 3);
                }
                else
                    tot[s][mb][1] = tot[s][mb][3] = 0.f;
            }
        }
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
        float v = 0.f;
        for (int w = 0; w < nwarps; w++)
            v += r[w * warp_stride];
        return v;
    };

    // ---- summing over the ranks of a tensor-parallel group, fused into the launch (ar_world > 1)
    // The CTA that holds the final sum of a row tile on this rank (for splits == 1 the tile's own CTA, otherwise the
    // split that arrived last) writes it as fp32 into this rank's peer-visible buffer, tells every peer "tile t,
    // call e" with one release store, waits (bounded) for the peers' words for the same tile, reads their sums
    // with plain peer loads and adds everything in rank order: every rank stores the same bits.  Calls alternate
    // between the two halves of the buffers (half = e & 1): a rank can be one call ahead of a peer that is still
    // reading a tile, never two, because the same tile's flag of the call in between is needed first.  Nothing here
    // waits on a CTA of this GPU, and the peers' CTAs announce before they wait, so no cycle of waits can form.
    const bool ar = p.ar_world > 1;
    auto ar_exchange = [&](int first, int count, bool by_last_flag) {
        auto owns = [&](int j) { return !by_last_flag || last_flag[j] != 0; };
        uint32_t* counters = p.ar_flags[p.ar_rank] + (size_t)p.row_tiles * 8;
        // 0. the call number of every tile of the batch that this CTA finishes
        if (tid < count && owns(tid))
        {
            const int rt = cta_in_split + (first + tid) * p.ctas_per_split;
            uint32_t e = p.ar_epoch;
            if (e == 0)
            {
                e = __ldcg(counters + rt) + 1; // only the CTA that finishes the tile touches the word
                if (e == 0)
                    e = 2;                     // 0 means "count for me": skip it, keeping the parity
            }
            ep_s[tid] = e;
        }
        if (tid == 0)
            *ar_ok = 1;
        named_barrier(1, nthreads);
    };
    auto ar_finish = [&](int first, int count, bool by_last_flag) {
        auto owns = [&](int j) { return !by_last_flag || last_flag[j] != 0; };
        uint32_t* counters = p.ar_flags[p.ar_rank] + (size_t)p.row_tiles * 8;
        // this rank's sums (written by all threads above) are ordered before the announcements below by the barrier
        // and the release stores, which are cumulative over what the barrier made visible to the storing thread
        named_barrier(1, nthreads);
        // 1. announce to every peer, 2. wait for every peer: thread (tile j, peer r)
        if (tid < count * p.ar_world)
        {
            const int j = tid / p.ar_world, r = tid - j * p.ar_world;
            if (r != p.ar_rank && owns(j))
            {
                const int rt = cta_in_split + (first + j) * p.ctas_per_split;
                const uint32_t e = ep_s[j];
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.ar_flags[r] + (size_t)rt * 8 + p.ar_rank), "r"(e)
                             : "memory");
                const uint32_t* mine = p.ar_flags[p.ar_rank] + (size_t)rt * 8 + r;
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
            __stcg(counters + cta_in_split + (first + tid) * p.ctas_per_split, ep_s[tid]);
        named_barrier(1, nthreads);
        if (!*ar_ok)
            return;
        // 3. everybody's sums in rank order
        for (int idx = tid; idx < count * per_tile; idx += nthreads)
        {
            const int j = idx >> pt_shift, e = idx & (per_tile - 1);
            if (!owns(j))
                continue;
            int row, m, o;
            decode(e, row, m, o);
            const int n = (cta_in_split + (first + j) * p.ctas_per_split) * 16 + row;
            if (m < p.M && n < p.N)
            {
                const size_t off = (size_t)(ep_s[j] & 1u) * p.ar_half_stride + ((size_t)m * p.N + n) * sizeof(float);
                float v = 0.f;
                for (int r = 0; r < p.ar_world; r++)
                    v += __ldcv(reinterpret_cast<const float*>(p.ar_bufs[r] + off));
                store_y(m, n, finish(v, 0.f, 0.f, m, n));
            }
        }
    };
    // Where a finished sum goes: to y, or (summing over ranks) into this rank's peer-visible buffer.
    auto emit = [&](int j, int m, int n, float a0, float a1, float ssum) {
        if (!ar)
            store_y(m, n, finish(a0, a1, ssum, m, n));
        else
            *reinterpret_cast<float*>(const_cast<char*>(p.ar_bufs[p.ar_rank]) + (size_t)(ep_s[j] & 1u) * p.ar_half_stride +
                                      ((size_t)m * p.N + n) * sizeof(float)) = a0;
    };

    // Add up the warps' partial sums of tiles [first, first + count) and write the results out.
    auto flush = [&](int first, int count) {
        named_barrier(1, nthreads);
        if (p.splits == 1)
        {
            if (ar)
                ar_exchange(first, count, false);
            for (int idx = tid; idx < count * per_tile; idx += nthreads)
            {
                const int j = idx >> pt_shift, e = idx & (per_tile - 1);
                int row, m, o;
                decode(e, row, m, o);
                const int n = (cta_in_split + (first + j) * p.ctas_per_split) * 16 + row;
                if (m < p.M && n < p.N)
                    emit(j, m, n, sum_warps(j, 0, e), DUAL ? sum_warps(j, 1, e) : 0.f, p.rmsnorm ? ss_cta[m] : 0.f);
            }
            if (ar)
                ar_finish(first, count, false);
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
                const int rt = cta_in_split + (first + j) * p.ctas_per_split;
                float* slot = p.ws_slots + ((size_t)split * p.row_tiles + rt) * p.slot_floats;
                __stcg(slot + o, sum_warps(j, 0, e));
                if (DUAL)
                    __stcg(slot + MB * 128 + o, sum_warps(j, 1, e));
            }
            if (p.rmsnorm)
                for (int idx = tid; idx < count * MPAD; idx += nthreads)
                {
                    const int j = idx / MPAD, mm = idx - j * MPAD;
                    const int rt = cta_in_split + (first + j) * p.ctas_per_split;
                    __stcg(p.ws_slots + ((size_t)split * p.row_tiles + rt) * p.slot_floats + SETS * MB * 128 + mm,
                           ss_cta[mm]);
                }
            __threadfence();
            named_barrier(1, nthreads);
            // 2. one arrival per tile; the last split to arrive owns the tile's final sum
            if (tid < count)
            {
                const int rt = cta_in_split + (first + tid) * p.ctas_per_split;
                const unsigned old = atomicAdd(p.ws_count + rt, 1u);
                last_flag[tid] = (old == (unsigned)(p.splits - 1));
                if (last_flag[tid])
                    p.ws_count[rt] = 0u; // leave the counter zeroed for the next call
            }
            named_barrier(1, nthreads);
            __threadfence();
            if (ar)
                ar_exchange(first, count, true);
            // 3. fixed-order sum over the splits
            for (int idx = tid; idx < count * per_tile; idx += nthreads)
            {
                const int j = idx >> pt_shift, e = idx & (per_tile - 1);
                if (!last_flag[j])
                    continue;
                int row, m, o;
                decode(e, row, m, o);
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
                            ssum += __ldcg(slot + SETS * MB * 128 + m);
                    }
                    emit(j, m, n, a0, a1, ssum);
                }
            }
            if (ar)
                ar_finish(first, count, true);
        }
        named_barrier(1, nthreads);
    };

    // ---------------------------------------------------------------- main loop
    // Inside a batch the warps only meet through the ring's barriers: full (bytes have landed) and empty (every warp
    // has taken what it needs from the slot, so the producer may ask for the tile that lands there next).
    int slot = 0;
    uint32_t parity = 0;
    bool timed_out = false;
    for (int first = 0; first < nsteps; first += p.batch)
    {
        const int count = min(p.batch, nsteps - first);
        for (int j = 0; j < count; j++)
        {
            const int st = first + j;
            if (use_full && !mbar_wait(full_s + 8 * slot, parity))
                timed_out = true;
            __syncwarp(); // lanes may leave the polling loop on different rounds; the MMAs below are warp-wide
            if (lsu)
                cp_async_wait(p.depth - 1); // this thread's pieces of tile st have landed
            float4* my = reinterpret_cast<float4*>(red + warp * warp_stride + j * SETS * per_tile);
            if (has_slice)
                compute(st, slot);
            else
            {
#pragma unroll
                for (int s = 0; s < SETS; s++)
#pragma unroll
                    for (int mb = 0; mb < MB; mb++)
#pragma unroll
                        for (int c = 0; c < 4; c++)
                            tot[s][mb][c] = 0.f;
            }
            if (t < tq)
            {
#pragma unroll
                for (int s = 0; s < SETS; s++)
#pragma unroll
                    for (int mb = 0; mb < MB; mb++)
                        my[(s * MB + mb) * 8 * tq + g * tq + t] =
                            make_float4(tot[s][mb][0], tot[s][mb][1], tot[s][mb][2], tot[s][mb][3]);
            }
            if (lsu)
            {
                // what this thread read from the slot is in its registers: ask for the tile that lands there next
                if (st + p.depth < nsteps && has_slice)
                    fetch_tile(st + p.depth);
                cp_async_commit();
            }
            __syncwarp();
            if (lane == 0)
                mbar_arrive(empty_s + 8 * slot);
            if (++slot == p.depth)
                slot = 0, parity ^= 1;
        }
        flush(first, count);
    }
    if (timed_out)
        atomicExch(p.status, 1);
}

// Raise the kernel's dynamic shared-memory limit (monotonically: the attribute is a plain setter).
template <int WBITS, int MB, bool XSPLIT, bool DUAL, bool EXACT, bool FAST>
cudaError_t ensure_smem(size_t smem)
{
    static size_t configured[nnf::kMaxDevices] = {}; // the attribute belongs to the device that is current
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        return e;
    if (dev < 0 || dev >= nnf::kMaxDevices)
        return cudaErrorInvalidDevice;
    if (smem <= std::max(configured[dev], (size_t)48 * 1024))
        return cudaSuccess;
    e = cudaFuncSetAttribute(dq_gemv_kernel<WBITS, MB, XSPLIT, DUAL, EXACT, FAST>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
        configured[dev] = smem;
    return e;
}

template <int WBITS, int MB, bool XSPLIT, bool DUAL, bool EXACT, bool FAST>
cudaError_t launch(const GemvParams& p, int warps, int /*grid*/, size_t smem, cudaStream_t stream)
{
    cudaError_t e = ensure_smem<WBITS, MB, XSPLIT, DUAL, EXACT, FAST>(smem);
    if (e != cudaSuccess)
        return e;
    (void)cudaGetLastError(); // do not inherit a stale error left behind by an unrelated earlier call
    // Programmatic dependent launch: the CTAs may start while the launch before this one on the stream is still
    // finishing; they stream their weights at once and wait (griddepcontrol.wait) before touching anything else.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.ctas_per_split, p.splits);
    cfg.blockDim = dim3((warps + 1) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    nnf::overlap_attribute(attr, &cfg.numAttrs);
    cfg.attrs = attr;
    return cudaLaunchKernelEx(&cfg, dq_gemv_kernel<WBITS, MB, XSPLIT, DUAL, EXACT, FAST>, p);
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
    {                                                                                                             \
        if (plan.exact)                                                                                           \
            return launch<WB, MBV, XSP, DU, true, false>(p, plan.warps, grid, plan.smem_bytes, stream);           \
        /* the lean inner loop is built for fp16 activations only: fp32 ones pay for their second half anyway */  \
        if (!XSP && p.bulk_params && !p.scale_f32)                                                                \
            return launch<WB, MBV, false, DU, false, true>(p, plan.warps, grid, plan.smem_bytes, stream);         \
        return launch<WB, MBV, XSP, DU, false, false>(p, plan.warps, grid, plan.smem_bytes, stream);              \
    }
    NNF_GEMV_FOR_EACH_VARIANT(NNF_X)
#undef NNF_X
    return cudaErrorInvalidValue;
}

// Ring depth and batch length for a CTA of `warps` warps that walks over at most `steps` row tiles, within `cap`
// bytes of shared memory.  Bytes in flight come first (about 96 KB per SM cover the HBM latency at full rate), then
// the batch length, which only sets how often the warps meet.
bool choose_ring(int sets, int mb, int warps, int tq, int pset_bytes, int xfrag_bytes, int steps, int cap, int* depth,
                 int* batch)
{
    const int want_d = std::min(kMaxDepth, std::max(1, steps)), want_b = std::min(kBatch, std::max(1, steps));
    const size_t slot_bytes = (size_t)sets * 16 * (warps * 128 + 64) + (size_t)sets * pset_bytes;
    const size_t target = std::min((size_t)want_d * slot_bytes, (size_t)96 * 1024);
    int best_d = 0, best_b = 0;
    int last_b = 0;
    for (int b : {want_b, 8, 4, 2, 1})
    {
        if (b > want_b || b == last_b)
            continue;
        last_b = b;
        for (int d = want_d; d >= 1; d--)
        {
            if ((int)SmemLayout(sets, mb, warps, d, b, tq, pset_bytes, xfrag_bytes).total + 1024 > cap)
                continue;
            if (d > best_d)
                best_d = d, best_b = b;
            if ((size_t)d * slot_bytes >= target)
            {
                *depth = d, *batch = b;
                return true;
            }
            break; // the deepest ring for this batch length is too shallow: try a shorter batch
        }
    }
    *depth = best_d, *batch = best_b;
    return best_d > 0;
}

// Everything the kernel needs to know that does not depend on where the operands live.
void fill_params(GemvParams& p, const nnf_b200_linear_desc& d, const nnf::GemvPlan& plan, const void* x,
                 const nnf_b200_qweight* w, const nnf_b200_qweight* w2, const void* gain, const void* bias, void* y,
                 int* status, void* workspace, const nnf_b200_peers* peers = nullptr)
{
    if (peers && peers->world > 1)
    {
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
    p.row_bytes = (d.w_bits == 4) ? d.K / 2 : d.K;
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
    p.status = status;
    p.M = d.M, p.N = d.N, p.K = d.K;
    p.group = d.group_size > 0 ? d.group_size : d.K;
    p.G = d.K / p.group;
    p.zp_row_bytes = (d.w_bits == 4) ? (p.G + 1) / 2 : p.G;
    p.units = d.K / ue;
    p.slices = plan.slices;
    p.row_tiles = plan.row_tiles;
    p.splits = plan.splits;
    p.ctas_per_split = plan.ctas_per_split;
    p.slices_lo = plan.slices / plan.splits, p.slices_rem = plan.slices % plan.splits;
    p.steps_lo = plan.row_tiles / plan.ctas_per_split, p.steps_rem = plan.row_tiles % plan.ctas_per_split;
    p.x_f32 = d.x_dtype == NNF_B200_F32;
    p.y_f32 = d.y_dtype == NNF_B200_F32;
    p.scale_f32 = d.scale_dtype == NNF_B200_F32;
    p.rmsnorm = d.prologue == NNF_B200_PROLOGUE_RMSNORM;
    p.has_addend = d.epilogue == NNF_B200_EPILOGUE_ADD;
    p.has_bias = bias != nullptr && !p.has_addend;
    p.eps = d.rms_eps;
    p.depth = plan.depth;
    p.batch = plan.batch;
    p.tq = plan.tq;
    p.scale_tile_bytes = plan.scale_tile_bytes;
    p.zp_tile_bytes = plan.zp_tile_bytes;
    p.pset_bytes = plan.pset_bytes;
    p.xfrag_bytes = plan.xfrag_bytes;
    p.slot_floats = (int)plan.slot_floats;
    // Bulk copies of the quantisation parameters need whole tiles inside the tensors and 16-byte aligned sources.
    auto ok16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
    p.bulk_params = plan.pset_bytes > 0 && ok16(w->scale) && ok16(w->zp) &&
                    (!plan.dual || (ok16(w2->scale) && ok16(w2->zp)));
    // How the weights travel: bulk copies from the producer warp, or cp.async from the arithmetic threads
    // themselves.
    p.lsu_weights = plan.lsu_weights;
    if (plan.splits > 1)
    {
        const size_t cnt = ((size_t)plan.row_tiles * sizeof(unsigned) + 255) / 256 * 256;
        p.ws_count = static_cast<unsigned*>(workspace);
        p.ws_slots = reinterpret_cast<float*>(static_cast<char*>(workspace) + cnt);
    }
}
} // namespace

namespace nnf
{
int gemv_configure(nnf_b200_ctx*)
{
    return NNF_B200_OK;
}

int gemv_plan(const nnf_b200_ctx* ctx, const nnf_b200_linear_desc& d, GemvPlan* plan, std::string* why,
              bool allow_direct)
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
    pl.tq = d.M > 4 ? 4 : (d.M > 2 ? 2 : 1);
    pl.dual = d.epilogue == NNF_B200_EPILOGUE_SILU_MUL;
    pl.exact = (d.flags & NNF_B200_FLAG_EXACT_ZP) != 0;
    // fp32 activations are carried as fp16 hi + lo where the register budget allows it
    pl.xsplit = d.x_dtype == NNF_B200_F32 && !(d.w_bits == 4 && pl.mb == 2);
    pl.row_tiles = (d.N + 15) / 16;
    const int units = d.K / ue;
    pl.slices = (units + 1) / 2;
    const int G = d.K / group;
    pl.scale_tile_bytes = 16 * G * (d.scale_dtype == NNF_B200_F32 ? 4 : 2);
    pl.zp_tile_bytes = 16 * ((d.w_bits == 4) ? (G + 1) / 2 : G);
    // whole tiles of parameters only: a ragged last tile makes the kernel read them with plain loads
    pl.pset_bytes = (d.N % 16 == 0) ? pl.scale_tile_bytes + pl.zp_tile_bytes : 0;
    // activation fragments of batch rows 8..15: 2 units x (1 or 2 halves of fp32 x) x NF/2 pairs x 32 lanes x 8 bytes
    pl.xfrag_bytes = (pl.mb == 2 && !pl.dual) ? 2 * (pl.xsplit ? 2 : 1) * ((d.w_bits == 4 ? 16 : 8) / 2) * 256 : 0;
    if (d.split_k > 0 && (pl.slices + d.split_k - 1) / d.split_k > kMaxWarps)
    {
        *why = "split_k too small: more than " + std::to_string(kMaxWarps) + " slices of 128 bytes per split";
        return NNF_B200_EINVAL;
    }
    if (allow_direct && gemv_direct_plan(ctx, d, &pl))
    {
        *plan = pl;
        return NNF_B200_OK;
    }
    const int sms = ctx ? ctx->sm_count : 148;
    const int smem_cap = ctx ? ctx->smem_optin : 227 * 1024;
    const int sets = pl.dual ? 2 : 1;
    // Warps per CTA: one per slice of the CTA's K range; split K when a row has more slices than that.  The
    // widest CTA whose partial sums and a useful ring fit in shared memory is taken.
    bool fits = false;
    for (int max_warps : {16, 12, 8, 6, 4, 2, 1})
    {
        pl.splits = (pl.slices + max_warps - 1) / max_warps;
        if (d.split_k > 0)
            pl.splits = std::min(d.split_k, pl.slices);
        pl.warps = (pl.slices + pl.splits - 1) / pl.splits;
        // CTAs per SM by registers (the kernel is compiled for at most 120 per thread: 544 threads per SM, one
        // warp of each CTA being its producer), then the ring that lets that many CTAs share the shared memory.
        for (int resident = std::max(1, 544 / ((pl.warps + 1) * 32)); resident >= 1 && !fits; resident = resident > 1 ? 1 : 0)
        {
            int per_split = std::max(1, (sms * resident) / pl.splits);
            per_split = std::min(per_split, pl.row_tiles);
            const int steps = (pl.row_tiles + per_split - 1) / per_split;
            if (choose_ring(sets, pl.mb, pl.warps, pl.tq, pl.pset_bytes, pl.xfrag_bytes, steps, smem_cap / resident,
                            &pl.depth, &pl.batch))
            {
                fits = true;
                pl.ctas_per_split = per_split;
                // Bulk copies move 16 bytes per clock and SM (4.6 TB/s over 148 SMs), cp.async from the arithmetic
                // threads more, at the price of instructions: measured, the latter wins once the ring has to be
                // refilled (large matrices) and loses when the whole share fits the ring, or with 16 batch rows.
                pl.lsu_weights = pl.mb == 1 && steps > pl.depth;
            }
        }
        if (fits || d.split_k > 0)
            break;
    }
    if (!fits)
    {
        *why = "shared memory: the launch shape does not fit";
        return NNF_B200_ENOTSUP;
    }
    pl.smem_bytes = SmemLayout(sets, pl.mb, pl.warps, pl.depth, pl.batch, pl.tq, pl.pset_bytes, pl.xfrag_bytes).total;
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

// Launches whichever small-M kernel the plan names.
static cudaError_t gemv_dispatch(const nnf_b200_linear_desc& d, const GemvPlan& plan, const void* x,
                                 const nnf_b200_qweight* w, const nnf_b200_qweight* w2, const void* gain,
                                 const void* bias, void* y, int* status, void* workspace,
                                 const nnf_b200_peers* peers, cudaStream_t stream)
{
    if (plan.direct)
        return gemv_direct_dispatch(d, plan, x, w, w2, gain, bias, y, status, workspace, stream, peers);
    GemvParams p{};
    fill_params(p, d, plan, x, w, w2, gain, bias, y, status, workspace, peers);
    return dispatch(d.w_bits, plan, p, plan.splits * plan.ctas_per_split, stream);
}

int gemv_launch(nnf_b200_ctx* ctx, cudaStream_t stream, const nnf_b200_linear_desc& d, const GemvPlan& plan,
                const void* x, const nnf_b200_qweight* w, const nnf_b200_qweight* w2, const void* gain,
                const void* bias, void* y, void* workspace, const nnf_b200_peers* peers)
{
    const int grid = plan.splits * plan.ctas_per_split;
    cudaError_t e = gemv_dispatch(d, plan, x, w, w2, gain, bias, y, ctx->dev_status, workspace, peers, stream);
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
// raises the kernel's shared-memory limit and queries device attributes, so it should be made outside of any stream
// capture.  All calls share the one array (and it keeps what the previous call left): calls
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
    int sm_count = 0;
    int smem_optin = 0;
};
StaticDeviceState g_static_state[nnf::kMaxDevices];
std::mutex g_static_mutex; // guards the once-per-device set-up

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
    std::string why;
    int rc = check_linear_call(desc, x, w, w2, gain, bias, y, nullptr, &why);
    if (rc == NNF_B200_OK && (desc->kernel == NNF_B200_KERNEL_GEMM || desc->M > 16))
    {
        rc = NNF_B200_ENOTSUP;
        why = "this entry point serves the small-M kernel only (M <= 16)";
    }
    if (rc != NNF_B200_OK)
    {
        put_message(errbuf, errbuf_len, why.c_str());
        return rc;
    }
    const nnf_b200_linear_desc& d = *desc;

    // ---- once per device, with that device current (host threads take turns)
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    {
        put_message(errbuf, errbuf_len, "no current CUDA device");
        return NNF_B200_ECUDA;
    }
    StaticDeviceState st;
    {
        std::lock_guard<std::mutex> guard(g_static_mutex);
        StaticDeviceState& slot = g_static_state[dev];
        if (!slot.ready)
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
            if (cudaDeviceGetAttribute(&slot.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
                cudaDeviceGetAttribute(&slot.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess ||
                cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess || major != 10)
            {
                put_message(errbuf, errbuf_len, "device attributes unavailable, or not an sm_100 device");
                return NNF_B200_ENOTSUP;
            }
            slot.scratch = sp;
            slot.status = static_cast<int*>(tp);
            slot.ready = true;
        }
        st = slot;
    }

    // ---- launch shape; the only kernel served here is the small-M one, which is the one that needs scratch
    nnf_b200_ctx shape_ctx; // plain host struct, used only to carry the device's SM count and shared-memory limit
    shape_ctx.device = dev;
    shape_ctx.sm_count = st.sm_count;
    shape_ctx.smem_optin = st.smem_optin;
    GemvPlan plan;
    rc = gemv_plan(&shape_ctx, d, &plan, &why);
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
    }
    cudaError_t e = gemv_dispatch(d, plan, x, w, w2, gain, bias, y, st.status, st.scratch, nullptr, s);
    if (e != cudaSuccess)
    {
        put_message(errbuf, errbuf_len, cudaGetErrorString(e));
        return NNF_B200_ECUDA;
    }
    return NNF_B200_OK;
}

extern "C" __attribute__((visibility("default"))) int nnf_b200_static_scratch_status(void* stream)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= nnf::kMaxDevices)
        return NNF_B200_ECUDA;
    int* word = nullptr;
    {
        std::lock_guard<std::mutex> guard(g_static_mutex);
        if (!g_static_state[dev].ready)
            return NNF_B200_OK; // nothing has run on this device through the allocation-free entry point yet
        word = g_static_state[dev].status;
    }
    int host = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(&host, word, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaMemsetAsync(word, 0, sizeof(int), s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess)
        return NNF_B200_ECUDA;
    return host != 0 ? NNF_B200_ETIMEDOUT : NNF_B200_OK;
}
