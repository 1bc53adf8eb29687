// Large-M (prefill) dequantize-fused linear for sm_100a on the 5th-generation tensor cores.
//
//   y[M,N] = epi( x[M,K] . dequant(W)[N,K]^T )        x fp16, W uint4 / uint8 with group scales and zero-points
//
// Fused replacement of the reference's Convert -> Subtract -> Multiply element-wise kernels that materialise the
// dequantised weights (src/nnfusion/core/kernels/cuda_gpu/kernels/elementwise.hpp:33-157,
// elementwise_fused.cpp:42-189) followed by cublasHgemm / cublasSgemm behind cuda::Dot
// (src/nnfusion/core/kernels/cuda_gpu/kernels/dot.cpp:103-125,264-363).
//
// A tile of the output is computed transposed,  D[128 weight rows, 256 batch rows] = Wdq[128, K] . X[256, K]^T,  so
// that the dequantised weights are the MMA's A operand and can be handed to the tensor core through TENSOR MEMORY
// instead of shared memory.  One persistent CTA per SM; the launch's work, tiles x raw chunks of K, is cut into equal
// shares, so that a tile at a seam is computed by two or more CTAs: each writes its fp32 partial sums to a slot of the
// workspace, and the one that arrives last at the tile adds the slots in the order of their K ranges (bitwise
// repeatable) and runs the epilogue.  Roles inside a CTA:
//   * warps "TMA" : one thread streams x tiles (256 rows x 64 fp16, 128-byte swizzle, the MMA's B operand), another
//                   raw packed-weight chunks (128 rows x 128 bytes, 128-byte swizzle), into shared-memory rings;
//   * warps "DQ"  : thread r owns weight row r of the tile = TMEM lane r.  Per 64-element k-block it reads its 32
//                   (uint4) or 64 (uint8) bytes from the raw ring, turns them into fp16 (q - zp) * scale with the
//                   exponent trick (PRMT + LOP3 + HSUB2 + HMUL2 per pair, exact integer before the scale), and
//                   writes the 32 packed registers into the A stage in TMEM with tcgen05.st.  Four groups of four
//                   warps take the k-blocks in turn, so that the conversion keeps ahead of the tensor core;
//   * warp "MMA"  : one thread issues tcgen05.mma.kind::f16 (A from TMEM, B from the shared-memory descriptor,
//                   fp32 accumulator D in TMEM, 128 x 256 x 16 per instruction) and releases stages with
//                   tcgen05.commit;
//   * epilogue    : the DQ warps read D with tcgen05.ld, apply bias / addend / SiLU(gate) * up, convert and store y.
// SiLU(x . Wg^T) * (x . Wu^T) runs as two launches: the first leaves the gate products in y, the second multiplies
// SiLU of what it finds in y into its own products.  Every mbarrier wait is bounded; on a time-out the CTA raises a
// status flag, skips its remaining work, and still frees its tensor memory.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "nnf_internal.h"
#include "sm100_ptx.cuh"

namespace
{
using namespace nnf::ptx;

// BXV: batch rows per tile, 256, or 64 for launches of up to 64 batch rows (a quarter of the activation bytes, of the
// tensor time and of the accumulator to read back and, for shared tiles, to pass through the workspace).
template <int WBITS, int BXV = 256>
struct Cfg
{
    static_assert(BXV == 256 || BXV == 64, "batch tile of 256 or 64 rows");
    static constexpr int BN = 128;              // weight rows per tile  (UMMA M, TMEM lanes)
    static constexpr int BX = BXV;              // batch rows per tile   (UMMA N, accumulator columns)
    static constexpr int BK = 64;               // k-block: one 128-byte swizzle row of fp16
    // One ring index for the x tile in shared memory and the converted weights in tensor memory, and one pair of
    // barriers for every PAIR of k-blocks: the MMA thread, whose own time per k-block is what bounds the kernel,
    // then waits once and releases once per eight MMAs.
    static constexpr int PAIRS = 3;             // ring depth in pairs of k-blocks
    static constexpr int STAGES = 2 * PAIRS;    // k-block stages
    static constexpr int WSTAGES = 2;
    static constexpr int KB_PER_CHUNK = (WBITS == 4) ? 4 : 2; // k-blocks per 128-byte raw chunk
    static constexpr int RAW_BYTES = (WBITS == 4) ? 32 : 64;  // raw bytes per row and k-block
    static constexpr int DQ_GROUPS = 4;                       // groups of 4 warps that take the k-blocks in turn
    static constexpr int DQ_WARPS = 4 * DQ_GROUPS;
    static constexpr int THREADS = (DQ_WARPS + 3) * 32;
    static constexpr int X_STAGE_BYTES = BX * 128;
    static constexpr int W_STAGE_BYTES = BN * 128;
    static constexpr int A_COL0 = BX;            // first TMEM column of the A stages
    static constexpr int A_STAGE_COLS = BK / 2;  // 64 fp16 per lane = 32 columns
    static constexpr int TMEM_COLS = BX == 256 ? 512 : 256;
    // full / empty per ring stage, full / empty per raw-weight stage, then: accumulator full, accumulator drained,
    // partial sums written, ticket known
    static constexpr int NUM_BARRIERS = 2 * PAIRS + 2 * WSTAGES + 4;
    static constexpr size_t SMEM_BYTES =
        1024 + (size_t)STAGES * X_STAGE_BYTES + (size_t)WSTAGES * W_STAGE_BYTES + NUM_BARRIERS * 8 + 64;
    static constexpr int SLOT_FLOATS = BX * BN; // one tile's accumulator as fp32: a partial sum in the workspace
    static_assert(A_COL0 + STAGES * A_STAGE_COLS <= TMEM_COLS, "tensor memory budget");
};

struct GemmParams
{
    const void* scale;
    const uint8_t* zp;
    const float* bias;
    void* y;
    int* status;
    uint32_t* counters; // [tiles] arrivals at a tile that several CTAs share; zero before and after a launch
    float* slots;       // [2 * CTAs][SLOT_FLOATS] partial sums of shared tiles
    int M, N, K;
    int group, G, zp_row_bytes;
    int y_f32, scale_f32, has_bias;
    int has_addend; // bias points at an [M,N] tensor of y's type instead of fp32 [N]
    int m_tiles;    // batch tiles; tile t covers batch tile t % m_tiles of weight-row tile t / m_tiles
    int tiles;      // output tiles in all
    int whole_tiles; // every tile is computed by one CTA (no partial sums)
    int kbpg_shift; // log2(group_size / 64) if that is a power of two, else -1
    int cpt;        // raw chunks (the unit of work) per tile: ceil(K / 64 / KB_PER_CHUNK)
};

constexpr uint32_t kGemmSpin = 1u << 22;

// Bounded wait that also gives up as soon as another role of the CTA has raised the abort flag.
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag)
{
    for (uint32_t i = 0; i < kGemmSpin; i++)
    {
        if (mbar_try_wait(bar, parity))
            return true;
        __nanosleep(40); // a waiting role should not compete with the working ones for issue slots and power
        if ((i & 255u) == 255u && *abort_flag)
            return false;
    }
    *abort_flag = 1;
    return false;
}

// Same for the thread that issues the MMAs: it is the kernel's critical path, so it polls without backing off.
__device__ __forceinline__ bool wait_hot(uint32_t bar, uint32_t parity, volatile int* abort_flag)
{
    for (uint32_t i = 0; i < kGemmSpin; i++)
    {
        if (mbar_try_wait(bar, parity))
            return true;
        if ((i & 1023u) == 1023u && *abort_flag)
            return false;
    }
    *abort_flag = 1;
    return false;
}

// UMMA shared-memory descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t smem_addr)
{
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}

// The CTA's share of the launch: units [u, u_end) of tiles * cpt raw chunks, walked as segments that each lie
// inside one tile.  Every role of the CTA walks the same list.
struct Segment
{
    int tile;     // output tile
    int c0, c1;   // raw chunks [c0, c1) of the tile
    int kb0, kb1; // k-blocks [kb0, kb1)
    bool whole;   // the CTA computes the tile alone
};

template <int KB_PER_CHUNK>
struct WorkList
{
    int u, u_end; // tiles * cpt fits 31 bits (checked on the host)
    __device__ WorkList(const GemmParams& p)
    {
        // whole tiles only: the shares are cut at tile boundaries
        const long long U = p.whole_tiles ? (long long)p.tiles : (long long)p.tiles * p.cpt;
        const int scale = p.whole_tiles ? p.cpt : 1;
        u = (int)((long long)blockIdx.x * U / gridDim.x) * scale;
        u_end = (int)((long long)(blockIdx.x + 1) * U / gridDim.x) * scale;
    }
    __device__ bool next(const GemmParams& p, Segment& s)
    {
        if (u >= u_end)
            return false;
        s.tile = u / p.cpt;
        s.c0 = u - s.tile * p.cpt;
        s.c1 = min(p.cpt, s.c0 + (u_end - u));
        s.kb0 = s.c0 * KB_PER_CHUNK;
        s.kb1 = min(p.K / 64, s.c1 * KB_PER_CHUNK);
        s.whole = s.c0 == 0 && s.c1 == p.cpt;
        u += s.c1 - s.c0;
        return true;
    }
};

// The CTA whose share holds unit u: the largest c with floor(c * U / G) <= u.
__device__ __forceinline__ int cta_of_unit(long long u, long long U, int G)
{
    return (int)(((u + 1) * G + U - 1) / U) - 1;
}

// Where CTA c keeps its partial sum of tile t: slot 2c if t is the first tile of its share, else 2c + 1 (a share has
// at most two tiles that it does not compute alone, its first and its last).
__device__ __forceinline__ int slot_of(int c, int t, long long U, int G, int cpt)
{
    const int first_tile = (int)(((long long)c * U / G) / cpt);
    return 2 * c + (t == first_tile ? 0 : 1);
}

// One finished value on its way to y: SiLU(gate) * v when a gate value is given, bias of the weight row (0 without),
// full-size addend, conversion.
__device__ __forceinline__ void store_value(const GemmParams& p, int m, int n, float v, bool gated, float g, float bias)
{
    const size_t at = (size_t)m * p.N + n;
    if (gated)
        v *= g > -80.f ? __fdividef(g, 1.0f + __expf(-g)) : 0.f; // SiLU(g) = g / (1 + e^-g), ~1e-6 relative; 0 far left
    v += bias;
    if (p.has_addend)
        v += p.y_f32 ? reinterpret_cast<const float*>(p.bias)[at]
                     : __half2float(reinterpret_cast<const __half*>(p.bias)[at]);
    if (p.y_f32)
        static_cast<float*>(p.y)[at] = v;
    else
        static_cast<__half*>(p.y)[at] = __float2half_rn(v);
}

// The gate product that an earlier launch left at y[m, n], as raw bits (fp32, or fp16 in the low half).
__device__ __forceinline__ uint32_t gate_bits(const GemmParams& p, int m, int n)
{
    const size_t at = (size_t)m * p.N + n;
    return p.y_f32 ? static_cast<const uint32_t*>(p.y)[at] : (uint32_t)static_cast<const unsigned short*>(p.y)[at];
}
// (a gate product that left the fp16 range on its way through y comes back as the largest fp16 number, so that SiLU
// stays finite: SiLU(-inf) would be -inf / inf)
__device__ __forceinline__ float gate_value(const GemmParams& p, uint32_t bits)
{
    if (p.y_f32)
        return __uint_as_float(bits);
    return fminf(fmaxf(__half2float(__ushort_as_half((unsigned short)bits)), -65504.f), 65504.f);
}

// GATED: y holds the gate products of an earlier launch (the second half of SiLU(gate) * up).
template <int WBITS, bool GATED, int BXV>
__global__ void __launch_bounds__(Cfg<WBITS, BXV>::THREADS, 1)
    dq_gemm_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap_x,
                   const __grid_constant__ CUtensorMap tmap_w)
{
    using C = Cfg<WBITS, BXV>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* xs = base;                                             // [STAGES][BX][128 B]
    uint8_t* wsm = xs + (size_t)C::STAGES * C::X_STAGE_BYTES;       // [WSTAGES][128][128 B]
    uint64_t* bars = reinterpret_cast<uint64_t*>(wsm + (size_t)C::WSTAGES * C::W_STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::NUM_BARRIERS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile uint32_t* ticket_slot = reinterpret_cast<volatile uint32_t*>(tmem_slot + 2);

    const uint32_t bar0 = smem_u32(bars);
    // full(q): the x tiles of pair q have landed (TMA transaction bytes) and every conversion thread has stored its
    // row of both stages (2 * 128 arrivals; where a segment ends on a single k-block, its threads arrive twice);
    // empty(q): the MMAs that read the pair have completed (tcgen05.commit).
    auto full = [&](int q) { return bar0 + 8u * q; };
    auto empty = [&](int q) { return bar0 + 8u * (C::PAIRS + q); };
    auto full_w = [&](int s) { return bar0 + 8u * (2 * C::PAIRS + s); };
    auto empty_w = [&](int s) { return bar0 + 8u * (2 * C::PAIRS + C::WSTAGES + s); };
    const uint32_t acc_full = bar0 + 8u * (C::NUM_BARRIERS - 4);     // a segment's MMAs have completed
    const uint32_t acc_empty = bar0 + 8u * (C::NUM_BARRIERS - 3);    // every conversion thread has read its part of D
    const uint32_t part_done = bar0 + 8u * (C::NUM_BARRIERS - 2);    // every conversion thread has written its partial sums
    const uint32_t ticket_ready = bar0 + 8u * (C::NUM_BARRIERS - 1); // the tile's arrival count is in ticket_slot

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int KB = p.K / C::BK;
    constexpr int TMA_WARP = C::DQ_WARPS, MMA_WARP = C::DQ_WARPS + 1, TMAW_WARP = C::DQ_WARPS + 2;

    // ---------------------------------------------------------------- set-up (once per CTA)
    if (tid == 0)
    {
        for (int q = 0; q < C::PAIRS; q++)
        {
            mbar_init(full(q), 2 * 128 + 1); // every row of both stages and the x tiles
            mbar_init(empty(q), 1);
        }
        for (int s = 0; s < C::WSTAGES; s++)
        {
            mbar_init(full_w(s), 1);
            mbar_init(empty_w(s), C::KB_PER_CHUNK * 128); // 128 rows read per k-block of the chunk
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, C::DQ_WARPS * 32);
        mbar_init(part_done, C::DQ_WARPS * 32);
        mbar_init(ticket_ready, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == MMA_WARP)
    {
        tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS); // whole warp; the address lands in shared memory
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    WorkList<C::KB_PER_CHUNK> work(p);
    Segment sg;
    // Launched as the programmatic dependent of the kernel before it on the stream, this CTA may have started while
    // that kernel's last CTAs were still running.  Weights, scales and zero-points are constants: the raw-chunk
    // producer and the conversion into tensor memory start at once.  The activations, the result, the addend and
    // the workspace may be the earlier kernel's: the activation producer waits before its first load and the
    // conversion warps before their first read-back.  The launch behind this one may be scheduled from here on.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == TMA_WARP)
    {
        // ------------------------------------------------------------ TMA producer: activation tiles
        if (lane == 0)
        {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            bool ok = true;
            uint32_t pr = 0; // pairs of k-blocks of this CTA so far: ring position (every segment starts a pair)
            while (ok && work.next(p, sg))
            {
                const int m0 = (sg.tile % p.m_tiles) * C::BX;
                for (int kb = sg.kb0; kb < sg.kb1; kb += 2, pr++)
                {
                    const int q = pr % C::PAIRS;
                    const uint32_t ph = (pr / C::PAIRS) & 1u;
                    ok = wait_or_abort(empty(q), ph ^ 1u, abort_flag);
                    if (!ok)
                        break;
                    const int nkb = min(2, sg.kb1 - kb);
                    mbar_arrive_expect_tx(full(q), (uint32_t)(nkb * C::X_STAGE_BYTES));
                    for (int h = 0; h < nkb; h++)
                        tma_load_2d(smem_u32(xs + (size_t)(2 * q + h) * C::X_STAGE_BYTES), &tmap_x, full(q),
                                    (kb + h) * C::BK, m0);
                }
            }
        }
    }
    else if (warp == TMAW_WARP)
    {
        // ------------------------------------------------------------ TMA producer: raw weight chunks
        // A loop of its own: the chunks run as far ahead as their ring allows (WSTAGES * KB_PER_CHUNK k-blocks),
        // so that their load latency and the conversion stay off the tensor core's critical path.
        if (lane == 0)
        {
            bool ok = true;
            uint32_t wc = 0; // chunks of this CTA so far
            while (ok && work.next(p, sg))
            {
                const int n0 = (sg.tile / p.m_tiles) * C::BN;
                for (int chunk = sg.c0; chunk < sg.c1; chunk++, wc++)
                {
                    const int s = wc % C::WSTAGES;
                    const uint32_t ph = (wc / C::WSTAGES) & 1u;
                    ok = wait_or_abort(empty_w(s), ph ^ 1u, abort_flag);
                    if (!ok)
                        break;
                    mbar_arrive_expect_tx(full_w(s), C::W_STAGE_BYTES);
                    tma_load_2d(smem_u32(wsm + (size_t)s * C::W_STAGE_BYTES), &tmap_w, full_w(s), chunk * 128, n0);
                }
            }
        }
    }
    else if (warp == MMA_WARP)
    {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0)
        {
            // instruction descriptor: fp32 accumulate, fp16 A and B, both K-major, N = BX, M = 128
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(C::BX >> 3) << 17) | ((uint32_t)(C::BN >> 4) << 24);
            bool ok = true;
            uint32_t si = 0;
            // Ring position kept as (slot, phase) with the slot's addresses carried along: this one thread feeds the
            // tensor core next to four busy conversion warps on its scheduler, so every instruction it does not
            // need to issue between two MMAs is tensor time.
            int q = 0;
            uint32_t phase = 0;
            const uint64_t xdesc0 = smem_desc_k_sw128(smem_u32(xs));
            const uint32_t a_tmem0 = tmem_base + (uint32_t)C::A_COL0;
            uint64_t xdesc = xdesc0;  // of slot q: two stages of x ...
            uint32_t a_tmem = a_tmem0; // ... and two stages of converted weights
            uint32_t bar_full = full(0), bar_empty = empty(0);
            while (ok && work.next(p, sg))
            {
                if (si > 0)
                {
                    // the accumulator still holds the previous segment until the conversion warps have read it
                    ok = wait_hot(acc_empty, (si - 1) & 1u, abort_flag);
                    if (!ok)
                        break;
                    tcgen05_fence_after();
                }
                uint32_t accumulate = 0u; // the segment's first MMA overwrites D
                for (int kb = sg.kb0; kb < sg.kb1; kb += 2)
                {
                    ok = wait_hot(bar_full, phase, abort_flag);
                    if (!ok)
                        break;
                    tcgen05_fence_after();
                    // (the descriptor's address field counts 16-byte units: stage and k step are plain additions)
#pragma unroll
                    for (int kk = 0; kk < C::BK / 16; kk++)
                    {
                        tcgen05_mma_ts(tmem_base, a_tmem + kk * 8, xdesc + (uint64_t)(kk * 2), idesc, accumulate);
                        accumulate = 1u;
                    }
                    if (kb + 1 < sg.kb1)
                    {
#pragma unroll
                        for (int kk = 0; kk < C::BK / 16; kk++)
                            tcgen05_mma_ts(tmem_base, a_tmem + C::A_STAGE_COLS + kk * 8,
                                           xdesc + (uint64_t)((C::X_STAGE_BYTES >> 4) + kk * 2), idesc, 1u);
                    }
                    tcgen05_commit(bar_empty); // arrives when the MMAs above have consumed the pair
                    if (++q == C::PAIRS)
                    {
                        q = 0, phase ^= 1u;
                        xdesc = xdesc0, a_tmem = a_tmem0, bar_full = full(0), bar_empty = empty(0);
                    }
                    else
                    {
                        xdesc += (uint64_t)(2 * (C::X_STAGE_BYTES >> 4)), a_tmem += 2 * C::A_STAGE_COLS;
                        bar_full += 8u, bar_empty += 8u;
                    }
                }
                if (ok)
                    tcgen05_commit(acc_full);
                si++;
            }
        }
    }
    else
    {
        // ------------------------------------------------------------ dequantise into tensor memory
        const int grp = warp >> 2;                   // 0 .. DQ_GROUPS-1
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;           // row of the tile = TMEM lane
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int kb_per_group = p.group / C::BK;
        const uint32_t wsm_s = smem_u32(wsm);
        bool ok = true;
        uint32_t pr_base = 0; // pairs of k-blocks of this CTA before the segment in hand: ring position of its first
        uint32_t wc_base = 0; // raw chunks likewise
        uint32_t si = 0, npart = 0;

        // Scales and zero-points: the raw words of this group's next two k-blocks wait in registers, in two sets
        // that take turns.  Nothing touches a loaded word before its k-block is converted (a move, a shift or a
        // conversion right after the load would make the thread sit out the whole load latency there), and the first
        // two of a segment are asked for before the previous segment's accumulator is read back.
        struct RawParams
        {
            uint32_t s, z;
            int g;
        };
        RawParams pa{0, 0, 0}, pb{0, 0, 0};
        // This thread's row of scales and of zero-points (rows past N read the last row's, never stored).
        struct RowParams
        {
            const char* scale;
            const uint8_t* zp;
        };
        auto row_of = [&](int tile) {
            const size_t n = (size_t)min((tile / p.m_tiles) * C::BN + r, p.N - 1);
            return RowParams{static_cast<const char*>(p.scale) + n * p.G * (p.scale_f32 ? 4 : 2),
                             p.zp + n * (WBITS == 4 ? p.zp_row_bytes : p.G)};
        };
        auto ask = [&](const RowParams& n, int kb, int kb_last, RawParams& q) {
            const int kbc = min(kb, kb_last);
            q.g = p.kbpg_shift >= 0 ? (kbc >> p.kbpg_shift) : kbc / kb_per_group;
            if (p.scale_f32)
                q.s = __ldg(reinterpret_cast<const uint32_t*>(n.scale) + q.g);
            else
                q.s = __ldg(reinterpret_cast<const unsigned short*>(n.scale) + q.g);
            q.z = __ldg(n.zp + (WBITS == 4 ? q.g >> 1 : q.g));
        };
        bool asked = false;
        bool dep_waited = false; // has this thread waited for the kernel before this one on the stream?

        while (ok && work.next(p, sg))
        {
            const RowParams n = row_of(sg.tile);
            if (!asked)
            {
                ask(n, sg.kb0 + grp, sg.kb1 - 1, pa);
                ask(n, sg.kb0 + grp + C::DQ_GROUPS, sg.kb1 - 1, pb);
            }

            // One k-block: raw bytes -> 64 fp16 (q - zp) * scale in k order (register i holds k = 2i in its low half
            // and k = 2i + 1 in its high half) -> this thread's row of the A stage in tensor memory -> tell the MMA
            // thread.  The group's k-block after next gets its parameters asked for on the way.
            auto one = [&](int kb, RawParams& q) -> bool {
                const int chunk = kb / C::KB_PER_CHUNK, j = kb % C::KB_PER_CHUNK;
                const uint32_t wci = wc_base + (uint32_t)(chunk - sg.c0);
                const int sw = wci % C::WSTAGES;
                if (!wait_or_abort(full_w(sw), (wci / C::WSTAGES) & 1u, abort_flag))
                    return false;
                // this row's raw bytes: 16-byte chunk c of row r is stored at chunk c ^ (r & 7)
                const uint32_t row = wsm_s + (uint32_t)(sw * C::W_STAGE_BYTES + r * 128);
                constexpr int NV = C::RAW_BYTES / 16;
                uint4 raw[NV];
#pragma unroll
                for (int v = 0; v < NV; v++)
                    raw[v] = lds128(row + (uint32_t)(((j * NV + v) ^ (r & 7)) * 16));
                const float sc = p.scale_f32 ? __uint_as_float(q.s) : __half2float(__ushort_as_half((unsigned short)q.s));
                const uint32_t zq = WBITS == 4 ? (q.z >> (4 * (q.g & 1))) & 0xFu : q.z;
                ask(n, kb + 2 * C::DQ_GROUPS, sg.kb1 - 1, q);
                const __half2 s2 = __float2half2_rn(sc);
                uint32_t a[32];
                if (WBITS == 4)
                {
                    const uint32_t zc = (0x6400u | zq) | ((0x5400u | (zq << 4)) << 16); // (1024 + zp, 64 + zp)
#pragma unroll
                    for (int v = 0; v < NV; v++)
                    {
                        const uint32_t w4[4] = {raw[v].x, raw[v].y, raw[v].z, raw[v].w};
#pragma unroll
                        for (int wi = 0; wi < 4; wi++)
#pragma unroll
                            for (int b = 0; b < 4; b++)
                            {
                                // byte b of the word holds elements 2b (bits 0-3) and 2b+1 (bits 4-7)
                                uint32_t t = __byte_perm(w4[wi], 0u, 0x1111u * b);
                                asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t) : "r"(t), "n"(0x00F0000Fu), "n"(0x54006400u));
                                __half2 h = __hsub2(*reinterpret_cast<__half2*>(&t), *reinterpret_cast<const __half2*>(&zc));
                                h = __hmul2(h, s2);
                                a[(v * 4 + wi) * 4 + b] = *reinterpret_cast<uint32_t*>(&h);
                            }
                    }
                }
                else
                {
                    const uint32_t zc = (0x6400u | zq) * 0x00010001u; // 1024 + zp in both halves
#pragma unroll
                    for (int v = 0; v < NV; v++)
                    {
                        const uint32_t w4[4] = {raw[v].x, raw[v].y, raw[v].z, raw[v].w};
#pragma unroll
                        for (int wi = 0; wi < 4; wi++)
#pragma unroll
                            for (int b = 0; b < 2; b++)
                            {
                                uint32_t t = __byte_perm(w4[wi], 0x64646464u, b ? 0x4342 : 0x4140); // 1024 + (b0, b1)
                                __half2 h = __hsub2(*reinterpret_cast<__half2*>(&t), *reinterpret_cast<const __half2*>(&zc));
                                h = __hmul2(h, s2);
                                a[(v * 4 + wi) * 2 + b] = *reinterpret_cast<uint32_t*>(&h);
                            }
                    }
                }
                // hand the converted k-block to the tensor core: wait for the A stage, store, publish
                const int rel = kb - sg.kb0;
                const uint32_t prv = pr_base + (uint32_t)(rel >> 1);
                const int pq = prv % C::PAIRS, sa = 2 * pq + (rel & 1);
                // (the vote brings the warp's lanes back together: each polled on its own and may have left the loop
                // on a different round, and the tensor-memory store below is a warp-wide instruction that every
                // lane must execute in the same issue)
                if (!__all_sync(0xffffffffu, wait_or_abort(empty(pq), ((prv / C::PAIRS) & 1u) ^ 1u, abort_flag)))
                    return false;
                tcgen05_fence_after();
                tmem_st_32x32(tmem_base + lane_addr + (uint32_t)(C::A_COL0 + sa * C::A_STAGE_COLS), a);
                tcgen05_wait_st();
                tcgen05_fence_before();
                // The raw stage goes back to the copy engine only now: one arrival per k-block read (the tile's last
                // k-block also stands in for the k-blocks that a short last chunk does not have).  The arrival must
                // not be issued before the shared-memory loads have delivered, and nothing but an instruction that
                // needs their data makes an instruction wait for them: the tensor-memory store above consumed every
                // loaded word.  (Issued right behind the loads, the arrival could pass a load that was queued behind
                // a burst of global stores; the next chunk then landed first and the load read its bytes.)
                mbar_arrive_n(empty_w(sw), kb == KB - 1 ? (uint32_t)(C::KB_PER_CHUNK - j) : 1u);
                // a segment that ends on the first k-block of a pair: its threads also stand in for the second
                mbar_arrive_n(full(pq), ((rel & 1) == 0 && kb == sg.kb1 - 1) ? 2u : 1u);
                return true;
            };
            // The groups take the k-blocks in turn.  A group's warps sit on different schedulers next to the other
            // groups' warps, which hide one another's waits: no second register buffer.
            for (int kb = sg.kb0 + grp; ok && kb < sg.kb1; kb += 2 * C::DQ_GROUPS)
            {
                ok = one(kb, pa);
                if (ok && kb + C::DQ_GROUPS < sg.kb1)
                    ok = one(kb + C::DQ_GROUPS, pb);
            }
            pr_base += (uint32_t)((sg.kb1 - sg.kb0 + 1) >> 1);
            wc_base += (uint32_t)(sg.c1 - sg.c0);
            {
                WorkList<C::KB_PER_CHUNK> ahead = work;
                Segment nx;
                asked = ahead.next(p, nx);
                if (asked)
                {
                    const RowParams n_next = row_of(nx.tile);
                    ask(n_next, nx.kb0 + grp, nx.kb1 - 1, pa);
                    ask(n_next, nx.kb0 + grp + C::DQ_GROUPS, nx.kb1 - 1, pb);
                }
            }

            // -------------------------------------------------------- the segment's accumulator
            // D holds y transposed (lane = weight row n, column = batch row m): for one m the 32 lanes of a warp
            // hold 32 consecutive n.  A tile computed by this CTA alone goes through the epilogue to y; a shared
            // tile's accumulator goes to this CTA's slot in the workspace as fp32, and the CTA that arrives last
            // at the tile adds the slots in the order of their K ranges and writes y.  Each warp reads its two
            // 32-column pieces of D with both loads in flight, then lets the MMA thread have the accumulator back.
            const int n_base = (sg.tile / p.m_tiles) * C::BN, m0 = (sg.tile % p.m_tiles) * C::BX;
            const int nrow = n_base + r;
            // 256 columns: two 32-column pieces per warp.  64 columns: one piece for the warps of the first two groups,
            // none for the others (which only say that they are done with D).
            static_assert(C::BX / 32 == 2 * C::DQ_GROUPS || C::BX / 32 == C::DQ_GROUPS / 2, "pieces per warp");
            constexpr bool kWide = C::BX / 32 == 2 * C::DQ_GROUPS;
            const bool has_piece = kWide || grp < C::BX / 32; // the same for every lane of a warp
            const int col0 = grp * 32, col1 = (grp + C::DQ_GROUPS) * 32;
            // With the gate products in y, those of the first piece are asked for before the accumulator is ready.
            const float bias = (p.has_bias && nrow < p.N) ? __ldg(p.bias + nrow) : 0.f;
            const bool gated = GATED && sg.whole;
            uint32_t gb[GATED ? 32 : 1] = {};
            // (rows and columns past the edge read the last valid ones: plain loads whose results nothing touches
            // until the values are needed)
            auto ask_gates = [&](int col) {
                if (GATED && gated)
                {
                    const int nn = min(nrow, p.N - 1);
                    if (p.y_f32)
                    {
#pragma unroll
                        for (int jx = 0; jx < (GATED ? 32 : 1); jx++)
                            gb[jx] = static_cast<const uint32_t*>(p.y)[(size_t)min(m0 + col + jx, p.M - 1) * p.N + nn];
                    }
                    else
                    {
#pragma unroll
                        for (int jx = 0; jx < (GATED ? 32 : 1); jx++)
                            gb[jx] = static_cast<const unsigned short*>(p.y)[(size_t)min(m0 + col + jx, p.M - 1) * p.N + nn];
                    }
                }
            };
            if (!dep_waited)
            {
                asm volatile("griddepcontrol.wait;" ::: "memory"); // y, the addend and the workspace are touched from here on
                dep_waited = true;
            }
            if (has_piece)
                ask_gates(col0);
            // (a vote again: the tensor-memory loads below are warp-wide instructions)
            ok = __all_sync(0xffffffffu, ok && wait_or_abort(acc_full, si & 1u, abort_flag));
            si++;
            if (!ok)
                break;
            tcgen05_fence_after();
            if (sg.whole)
            {
                if constexpr (kWide)
                {
                    uint32_t d[32];
                    tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)col0, d);
                    tcgen05_wait_ld();
                    if (nrow < p.N)
                    {
    #pragma unroll
                        for (int jx = 0; jx < 32; jx++)
                            if (m0 + col0 + jx < p.M)
                                store_value(p, m0 + col0 + jx, nrow, __uint_as_float(d[jx]), gated, gate_value(p, gb[GATED ? jx : 0]), bias);
                    }
                    ask_gates(col1);
                    tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)col1, d);
                    tcgen05_wait_ld();
                    tcgen05_fence_before();
                    mbar_arrive(acc_empty); // this thread's last read of D: the next segment may overwrite it
                    if (nrow < p.N)
                    {
    #pragma unroll
                        for (int jx = 0; jx < 32; jx++)
                            if (m0 + col1 + jx < p.M)
                                store_value(p, m0 + col1 + jx, nrow, __uint_as_float(d[jx]), gated, gate_value(p, gb[GATED ? jx : 0]), bias);
                    }
                }
                else
                {
                    if (has_piece)
                    {
                        uint32_t d[32];
                        tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)col0, d);
                        tcgen05_wait_ld();
                        tcgen05_fence_before();
                        mbar_arrive(acc_empty);
                        if (nrow < p.N)
                        {
#pragma unroll
                            for (int jx = 0; jx < 32; jx++)
                                if (m0 + col0 + jx < p.M)
                                    store_value(p, m0 + col0 + jx, nrow, __uint_as_float(d[jx]), gated, gate_value(p, gb[GATED ? jx : 0]), bias);
                        }
                    }
                    else
                    {
                        tcgen05_fence_before();
                        mbar_arrive(acc_empty);
                    }
                }
            }
            else
            {
                const long long U = (long long)p.tiles * p.cpt;
                const int G = (int)gridDim.x;
                const int c_first = cta_of_unit((long long)sg.tile * p.cpt, U, G);
                const int c_last = cta_of_unit((long long)(sg.tile + 1) * p.cpt - 1, U, G);
                const uint32_t pieces = (uint32_t)(c_last - c_first + 1);
                float* mine = p.slots + (size_t)slot_of((int)blockIdx.x, sg.tile, U, G, p.cpt) * C::SLOT_FLOATS;
                if constexpr (kWide)
                {
                    uint32_t d[32];
                    tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)col0, d);
                    tcgen05_wait_ld();
#pragma unroll
                    for (int jx = 0; jx < 32; jx++)
                        mine[(size_t)(col0 + jx) * C::BN + r] = __uint_as_float(d[jx]);
                    tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)col1, d);
                    tcgen05_wait_ld();
                    tcgen05_fence_before();
                    mbar_arrive(acc_empty);
#pragma unroll
                    for (int jx = 0; jx < 32; jx++)
                        mine[(size_t)(col1 + jx) * C::BN + r] = __uint_as_float(d[jx]);
                }
                else if (has_piece)
                {
                    uint32_t d[32];
                    tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)col0, d);
                    tcgen05_wait_ld();
                    tcgen05_fence_before();
                    mbar_arrive(acc_empty);
#pragma unroll
                    for (int jx = 0; jx < 32; jx++)
                        mine[(size_t)(col0 + jx) * C::BN + r] = __uint_as_float(d[jx]);
                }
                else
                {
                    tcgen05_fence_before();
                    mbar_arrive(acc_empty);
                }
                __threadfence();
                mbar_arrive(part_done);
                if (warp == 0)
                {
                    // The whole warp waits (a lane spinning on its own while its warp-mates spin on another barrier
                    // starves), then one lane takes the ticket.
                    const bool landed = __all_sync(0xffffffffu, wait_or_abort(part_done, npart & 1u, abort_flag));
                    if (lane == 0 && landed)
                    {
                        __threadfence(); // the partial sums of all threads before the ticket
                        const uint32_t before = atomicAdd(p.counters + sg.tile, 1u);
                        __threadfence();
                        if (before == pieces - 1)
                            p.counters[sg.tile] = 0u; // leave the counter zeroed for the next call
                        *ticket_slot = before;
                        mbar_arrive(ticket_ready);
                    }
                    __syncwarp();
                }
                ok = wait_or_abort(ticket_ready, npart & 1u, abort_flag);
                npart++;
                if (!ok)
                    break;
                if (*ticket_slot == pieces - 1)
                {
                    // Last to arrive: add the tile's slots in the order of their K ranges and write y.  Nothing ties
                    // a thread to a tensor-memory lane here, so every thread takes four neighbouring weight rows of
                    // one batch row at a time (16-byte loads), four such positions and two slots per round trip
                    // to L2.
                    __threadfence();
                    constexpr int NT = C::DQ_WARPS * 32;        // threads at work
                    constexpr int Q = C::SLOT_FLOATS / 4;       // float4 per slot
                    static_assert(Q % (NT * 4) == 0, "four positions per thread and pass");
                    const bool vec = (p.N % 4 == 0) && !p.has_addend && !GATED &&
                                     (reinterpret_cast<uintptr_t>(p.y) & 15u) == 0;
                    for (int q0 = warp * 32 + lane; q0 < Q; q0 += NT * 4)
                    {
                        float4 v[4];
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                        for (int c = c_first; c <= c_last; c += 2) // fixed order: repeatable
                        {
                            const bool two = c + 1 <= c_last;
                            const float4* s0 = reinterpret_cast<const float4*>(
                                p.slots + (size_t)slot_of(c, sg.tile, U, G, p.cpt) * C::SLOT_FLOATS);
                            const float4* s1 = reinterpret_cast<const float4*>(
                                p.slots + (size_t)slot_of(two ? c + 1 : c, sg.tile, U, G, p.cpt) * C::SLOT_FLOATS);
                            float4 a0[4], a1[4];
#pragma unroll
                            for (int j = 0; j < 4; j++)
                            {
                                a0[j] = __ldcg(s0 + q0 + j * NT);
                                a1[j] = __ldcg(s1 + q0 + j * NT);
                            }
#pragma unroll
                            for (int j = 0; j < 4; j++)
                            {
                                v[j].x += a0[j].x, v[j].y += a0[j].y, v[j].z += a0[j].z, v[j].w += a0[j].w;
                                if (two)
                                    v[j].x += a1[j].x, v[j].y += a1[j].y, v[j].z += a1[j].z, v[j].w += a1[j].w;
                            }
                        }
#pragma unroll
                        for (int j = 0; j < 4; j++)
                        {
                            const int f = (q0 + j * NT) * 4;    // float index in the slot: [batch row][weight row]
                            const int m = m0 + f / C::BN, n4 = n_base + f % C::BN;
                            if (m >= p.M)
                                continue;
                            float o[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
                            if (vec && n4 + 3 < p.N)
                            {
                                if (p.has_bias)
                                {
#pragma unroll
                                    for (int e = 0; e < 4; e++)
                                        o[e] += __ldg(p.bias + n4 + e);
                                }
                                const size_t at = (size_t)m * p.N + n4;
                                if (p.y_f32)
                                    *reinterpret_cast<float4*>(static_cast<float*>(p.y) + at) = make_float4(o[0], o[1], o[2], o[3]);
                                else
                                {
                                    const __half2 h0 = __floats2half2_rn(o[0], o[1]), h1 = __floats2half2_rn(o[2], o[3]);
                                    uint2 pk;
                                    pk.x = *reinterpret_cast<const uint32_t*>(&h0), pk.y = *reinterpret_cast<const uint32_t*>(&h1);
                                    *reinterpret_cast<uint2*>(static_cast<__half*>(p.y) + at) = pk;
                                }
                            }
                            else
                            {
#pragma unroll
                                for (int e = 0; e < 4; e++)
                                    if (n4 + e < p.N)
                                        store_value(p, m, n4 + e, o[e], GATED,
                                                    GATED ? gate_value(p, gate_bits(p, m, n4 + e)) : 0.f,
                                                    p.has_bias ? __ldg(p.bias + n4 + e) : 0.f);
                            }
                        }
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------- tear-down
    tcgen05_fence_before();
    __syncthreads();
    if (warp == MMA_WARP)
    {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
    if (tid == 0 && *abort_flag)
        atomicExch(p.status, 1);
}

// Pre-pass for activations the tensor-core kernel does not take as they are: fp32 rows are rounded to fp16, and with
// the RMSNorm prologue every row is scaled by rsqrt(mean(x^2) + eps) * gain on the way (fp32 arithmetic, one
// rounding).  One CTA per row; the row is read twice when it has to be normalised (the second time from L2).
// Replaces the reference's Multiply -> Sum -> Divide -> Add -> Rsqrt -> Multiply chain in front of the Dot
// (reduce: src/nnfusion/core/kernels/cuda_gpu/kernels/reduce.hpp:18-600) and its Convert.
template <bool XF32>
__global__ void __launch_bounds__(256) prep_activations_kernel(const void* x, const float* gain, __half* out, int K,
                                                               float eps)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float part[8];
    const size_t row = blockIdx.x;
    auto load = [&](int k) -> float {
        return XF32 ? static_cast<const float*>(x)[row * K + k] : __half2float(static_cast<const __half*>(x)[row * K + k]);
    };
    float r = 1.f;
    if (gain != nullptr)
    {
        float ss = 0.f;
        for (int k = threadIdx.x; k < K; k += blockDim.x)
        {
            const float v = load(k);
            ss += v * v;
        }
        for (int o = 16; o > 0; o >>= 1)
            ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if ((threadIdx.x & 31) == 0)
            part[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) // fixed order: repeatable
            tot += part[w];
        r = 1.0f / sqrtf(tot / (float)K + eps);
    }
    for (int k = threadIdx.x; k < K; k += blockDim.x)
    {
        float v = load(k) * r;
        if (gain != nullptr)
            v *= gain[k];
        out[row * K + k] = __float2half_rn(v);
    }
}

template <int WBITS, bool GATED, int BXV>
cudaError_t launch(const GemmParams& p, const CUtensorMap& tx, const CUtensorMap& tw, int grid, cudaStream_t stream)
{
    using C = Cfg<WBITS, BXV>;
    static bool configured[nnf::kMaxDevices] = {}; // the attribute belongs to the device that is current
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        return e;
    if (dev < 0 || dev >= nnf::kMaxDevices)
        return cudaErrorInvalidDevice;
    if (!configured[dev])
    {
        e = cudaFuncSetAttribute(dq_gemm_kernel<WBITS, GATED, BXV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)C::SMEM_BYTES);
        if (e != cudaSuccess)
            return e;
        configured[dev] = true;
    }
    (void)cudaGetLastError();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(C::THREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, dq_gemm_kernel<WBITS, GATED, BXV>, p, tx, tw);
}
} // namespace

namespace nnf
{
int gemm_configure(nnf_b200_ctx*)
{
    return NNF_B200_OK;
}

// fp32 activations and the RMSNorm prologue go through a pre-pass that writes fp16 [M,K] into the workspace.
static bool needs_prepass(const nnf_b200_linear_desc& d)
{
    return d.x_dtype == NNF_B200_F32 || d.prologue == NNF_B200_PROLOGUE_RMSNORM;
}

// How a launch is laid out: persistent CTAs share tiles * chunks-per-tile units of work evenly; the workspace holds
// the arrival counters of the tiles, two partial-sum slots per CTA and, when needed, the fp16 copy of x.
struct GemmLayout
{
    int bx, m_tiles, n_tiles, tiles, cpt, grid, whole_tiles;
    size_t counter_bytes, slot_bytes, prepass_bytes;
    size_t total() const { return counter_bytes + slot_bytes + prepass_bytes; }
};

static GemmLayout gemm_layout(const nnf_b200_ctx* ctx, const nnf_b200_linear_desc& d)
{
    GemmLayout L{};
    L.bx = d.M <= 64 ? 64 : 256; // a narrow batch tile for small batches
    L.m_tiles = (d.M + L.bx - 1) / L.bx;
    L.n_tiles = (d.N + 127) / 128;
    L.tiles = L.m_tiles * L.n_tiles;
    const int kb_per_chunk = d.w_bits == 4 ? 4 : 2;
    L.cpt = (d.K / 64 + kb_per_chunk - 1) / kb_per_chunk;
    const long long units = (long long)L.tiles * L.cpt;
    const int sms = ctx ? ctx->sm_count : 148;
    // Shares cut anywhere (tiles at the seams cost a partial sum in the workspace, a ticket and a final addition:
    // about 30 k-blocks' worth of time on top of the 8 of an epilogue) or at tile boundaries only (the CTA with the
    // most tiles sets the time): whichever the estimate, in k-block times, favours.
    const double kb = d.K / 64.0;
    // (the same estimate serves the narrow tile: with a lower price for its smaller shared tiles the up projection
    // at 17 to 64 batch rows was cut across all SMs and took 24.9 us instead of 23.5)
    const double t_split = (double)L.tiles * kb / sms + 8.0 + 30.0;
    const double t_whole = (double)((L.tiles + sms - 1) / sms) * (kb + 8.0);
    L.whole_tiles = t_whole <= t_split;
    if (L.whole_tiles)
        L.grid = L.tiles < sms ? L.tiles : sms;
    else
        L.grid = (int)(units < sms ? units : sms);
    L.counter_bytes = ((size_t)L.tiles * sizeof(uint32_t) + 255) / 256 * 256;
    L.slot_bytes = (size_t)2 * L.grid * 128 * L.bx * sizeof(float); // two slots of one fp32 tile per CTA
    L.prepass_bytes = needs_prepass(d) ? ((size_t)d.M * d.K * sizeof(__half) + 255) / 256 * 256 : 0;
    return L;
}

size_t gemm_workspace_bytes(const nnf_b200_ctx* ctx, const nnf_b200_linear_desc& d)
{
    return gemm_layout(ctx, d).total();
}

int gemm_supported(const nnf_b200_ctx*, const nnf_b200_linear_desc& d, std::string* why)
{
    const int group = d.group_size > 0 ? d.group_size : d.K;
    if (d.K % 64 != 0 || group % 64 != 0 || d.K % group != 0)
    {
        *why = "K and group_size must be multiples of 64 and K a multiple of group_size";
        return NNF_B200_ENOTSUP;
    }
    if ((d.w_bits == 4 ? d.K / 2 : d.K) % 16 != 0)
    {
        *why = "weight rows must be a multiple of 16 bytes";
        return NNF_B200_ENOTSUP;
    }
    // the kernel counts its units of work (tiles x raw chunks of K) in 32-bit integers
    const long long tiles = (long long)((d.M + 255) / 256) * ((d.N + 127) / 128);
    const long long chunks = (d.K / 64 + (d.w_bits == 4 ? 3 : 1)) / (d.w_bits == 4 ? 4 : 2);
    if (tiles * chunks >= (1ll << 31) || tiles >= (1ll << 30))
    {
        *why = "M * N * K is beyond what one launch counts";
        return NNF_B200_ENOTSUP;
    }
    return NNF_B200_OK;
}

int gemm_launch(nnf_b200_ctx* ctx, cudaStream_t stream, const nnf_b200_linear_desc& d, const void* x,
                const nnf_b200_qweight* w, const nnf_b200_qweight* w2, const void* gain, const void* bias, void* y,
                void* workspace, size_t workspace_bytes)
{
    const GemmLayout L = gemm_layout(ctx, d);
    if (!workspace || workspace_bytes < L.total())
        return set_error(ctx, NNF_B200_EWORKSPACE,
                         "workspace of " + std::to_string(L.total()) +
                             " bytes required (tile counters, partial sums of shared tiles, fp16 copy of the activations)");
    if (reinterpret_cast<uintptr_t>(workspace) & 15u)
        return set_error(ctx, NNF_B200_EALIGN, "the workspace must be 16-byte aligned");
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    if (needs_prepass(d))
    {
        __half* xh = reinterpret_cast<__half*>(ws + L.counter_bytes + L.slot_bytes);
        const float* g = d.prologue == NNF_B200_PROLOGUE_RMSNORM ? static_cast<const float*>(gain) : nullptr;
        (void)cudaGetLastError();
        if (d.x_dtype == NNF_B200_F32)
            prep_activations_kernel<true><<<d.M, 256, 0, stream>>>(x, g, xh, d.K, d.rms_eps);
        else
            prep_activations_kernel<false><<<d.M, 256, 0, stream>>>(x, g, xh, d.K, d.rms_eps);
        cudaError_t pe = cudaGetLastError();
        if (pe != cudaSuccess)
            return set_error(ctx, NNF_B200_ECUDA, std::string("prep_activations launch: ") + cudaGetErrorString(pe));
        ctx->launches++;
        x = xh;
    }
    const bool silu_mul = d.epilogue == NNF_B200_EPILOGUE_SILU_MUL;
    const int row_bytes = d.w_bits == 4 ? d.K / 2 : d.K;
    GemmParams p{};
    p.y = y;
    p.status = ctx->dev_status;
    p.M = d.M, p.N = d.N, p.K = d.K;
    p.group = d.group_size > 0 ? d.group_size : d.K;
    p.G = d.K / p.group;
    p.zp_row_bytes = d.w_bits == 4 ? (p.G + 1) / 2 : p.G;
    p.y_f32 = d.y_dtype == NNF_B200_F32;
    p.scale_f32 = d.scale_dtype == NNF_B200_F32;
    p.m_tiles = L.m_tiles;
    p.tiles = L.tiles;
    p.cpt = L.cpt;
    p.whole_tiles = L.whole_tiles;
    p.kbpg_shift = -1;
    for (int sh = 0; sh < 31; sh++)
        if ((p.group / 64) == (1 << sh))
            p.kbpg_shift = sh;
    p.counters = reinterpret_cast<uint32_t*>(ws);
    p.slots = reinterpret_cast<float*>(ws + L.counter_bytes);

    // x: fp16 [M][K], boxes of 256 rows x 64 elements (the tensor map is not cached: x moves between calls)
    alignas(64) CUtensorMap tx;
    if (!encode_tensor_map_2d(ctx->encode_tiled, &tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x, (uint64_t)d.K,
                              (uint64_t)d.M, (uint64_t)d.K * 2, 64, (uint32_t)L.bx, CU_TENSOR_MAP_SWIZZLE_128B))
        return set_error(ctx, NNF_B200_ECUDA, "cuTensorMapEncodeTiled failed for the activations");

    // SiLU(x . Wg^T) * (x . Wu^T): the gate products go to y first, the second launch folds them in.
    const int passes = silu_mul ? 2 : 1;
    for (int pass = 0; pass < passes; pass++)
    {
        const nnf_b200_qweight* wp = (silu_mul && pass == 1) ? w2 : w;
        p.scale = wp->scale;
        p.zp = static_cast<const uint8_t*>(wp->zp);
        p.has_addend = d.epilogue == NNF_B200_EPILOGUE_ADD;
        p.has_bias = bias != nullptr && !p.has_addend && !silu_mul;
        p.bias = static_cast<const float*>(bias);
        // copied by value at once: a later lookup may empty the context's cache
        alignas(64) CUtensorMap twv;
        const CUtensorMap* tw = weight_tensor_map(ctx, wp->wq, d.N, row_bytes, 128, 128);
        if (!tw)
            return set_error(ctx, NNF_B200_ECUDA, "cuTensorMapEncodeTiled failed for the weight tensor");
        twv = *tw;
        const bool gated = silu_mul && pass == 1;
        cudaError_t e;
        if (L.bx == 256)
            e = d.w_bits == 4
                    ? (gated ? launch<4, true, 256>(p, tx, twv, L.grid, stream) : launch<4, false, 256>(p, tx, twv, L.grid, stream))
                    : (gated ? launch<8, true, 256>(p, tx, twv, L.grid, stream) : launch<8, false, 256>(p, tx, twv, L.grid, stream));
        else
            e = d.w_bits == 4
                    ? (gated ? launch<4, true, 64>(p, tx, twv, L.grid, stream) : launch<4, false, 64>(p, tx, twv, L.grid, stream))
                    : (gated ? launch<8, true, 64>(p, tx, twv, L.grid, stream) : launch<8, false, 64>(p, tx, twv, L.grid, stream));
        if (e != cudaSuccess)
            return set_error(ctx, NNF_B200_ECUDA, std::string("dq_gemm launch: ") + cudaGetErrorString(e));
        ctx->launches++;
    }
    return NNF_B200_OK;
}
} // namespace nnf
