// Large-M (prefill) dequantize-fused linear for sm_100a on the 5th-generation tensor cores.
//
//   y[M,N] = epi( x[M,K] . dequant(W)[N,K]^T )        x fp16, W uint4 / uint8 with group scales and zero-points
//
// Fused replacement of the reference's Convert -> Subtract -> Multiply element-wise kernels that materialise the
// dequantised weights (src/nnfusion/core/kernels/cuda_gpu/kernels/elementwise.hpp:33-157,
// elementwise_fused.cpp:42-189) followed by cublasHgemm / cublasSgemm behind cuda::Dot
// (src/nnfusion/core/kernels/cuda_gpu/kernels/dot.cpp:103-125,264-363).
//
// The CTA computes a transposed output tile  D[128 weight rows, BX batch rows] = Wdq[128, K] . X[BX, K]^T  so
// that the dequantised weights are the MMA's A operand and can be handed to the tensor core through TENSOR MEMORY
// instead of shared memory:
//   * warps "TMA" : one thread streams x tiles (BX rows x 64 fp16, 128-byte swizzle, the MMA's B operand), another
//                   raw packed-weight chunks (128 rows x 128 bytes, 128-byte swizzle), into shared-memory rings;
//   * warps "DQ"  : thread r owns weight row r of the tile = TMEM lane r.  Per 64-element k-block it reads its 32
//                   (uint4) or 64 (uint8) bytes from the raw ring, turns them into fp16 (q - zp) * scale with the
//                   exponent trick (PRMT + LOP3 + HSUB2 + HMUL2 per pair, exact integer before the scale), and
//                   writes the 32 packed registers into the A stage in TMEM with tcgen05.st.  Two groups of four
//                   warps alternate k-blocks so that the conversion keeps ahead of the tensor core;
//   * warp "MMA"  : one thread issues tcgen05.mma.kind::f16 (A from TMEM, B from the shared-memory descriptor,
//                   fp32 accumulator D in TMEM, 128 x BX x 16 per instruction) and releases stages with
//                   tcgen05.commit;
//   * epilogue    : the DQ warps read D with tcgen05.ld, apply bias or SiLU(gate) * up, convert and store y.
// With the SiLU * mul epilogue the CTA carries two weight sets (gate, up), two accumulators of 128 columns each
// and BX = 128.  Every mbarrier wait is bounded; on a time-out the CTA raises a status flag, skips its remaining
// work, and still frees its tensor memory.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "nnf_internal.h"
#include "sm100_ptx.cuh"

namespace
{
using namespace nnf::ptx;

template <int WBITS, bool DUAL>
struct Cfg
{
    static constexpr int SETS = DUAL ? 2 : 1;
    static constexpr int BN = 128;              // weight rows per CTA  (UMMA M, TMEM lanes)
    static constexpr int BX = DUAL ? 128 : 256; // batch rows per CTA   (UMMA N, accumulator columns per set)
    static constexpr int BK = 64;               // k-block: one 128-byte swizzle row of fp16
    // One ring index for the x tile in shared memory and the converted weights in tensor memory: the MMA thread
    // then has a single barrier to wait for and a single one to release per k-block.
    static constexpr int STAGES = DUAL ? 4 : 5;
    static constexpr int XSTAGES = STAGES;
    static constexpr int WSTAGES = 3;
    static constexpr int ASTAGES = STAGES;
    static constexpr int KB_PER_CHUNK = (WBITS == 4) ? 4 : 2; // k-blocks per 128-byte raw chunk
    static constexpr int RAW_BYTES = (WBITS == 4) ? 32 : 64;  // raw bytes per row and k-block
    static constexpr int DQ_GROUPS = 2;                       // groups of 4 warps alternating k-blocks
    static constexpr int DQ_WARPS = 4 * DQ_GROUPS * SETS;
    static constexpr int THREADS = (DQ_WARPS + 3) * 32;
    static constexpr int X_STAGE_BYTES = BX * 128;
    static constexpr int W_STAGE_BYTES = BN * 128;
    static constexpr int A_COL0 = SETS * BX;     // first TMEM column of the A stages
    static constexpr int A_STAGE_COLS = BK / 2;  // 64 fp16 per lane = 32 columns
    static constexpr int TMEM_COLS = 512;
    static constexpr int NUM_BARRIERS = 2 * STAGES + 2 * SETS * WSTAGES + 1;
    static constexpr size_t SMEM_BYTES =
        1024 + (size_t)XSTAGES * X_STAGE_BYTES + (size_t)SETS * WSTAGES * W_STAGE_BYTES + NUM_BARRIERS * 8 + 64;
    static_assert(A_COL0 + SETS * ASTAGES * A_STAGE_COLS <= TMEM_COLS, "tensor memory budget");
    static_assert(KB_PER_CHUNK % DQ_GROUPS == 0, "every group must touch every raw chunk");
};

struct GemmParams
{
    const void* scale[2];
    const uint8_t* zp[2];
    const float* bias;
    void* y;
    int* status;
    int M, N, K;
    int group, G, zp_row_bytes;
    int y_f32, scale_f32, has_bias;
    int has_addend; // bias points at an [M,N] tensor of y's type instead of fp32 [N]
    int m_tiles;
    int fast_store; // fp16 y, N a multiple of 8, y 16-byte aligned: the tile is written in 16-byte pieces
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

template <int WBITS, bool DUAL>
__global__ void __launch_bounds__(Cfg<WBITS, DUAL>::THREADS, 1)
    dq_gemm_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap_x,
                   const __grid_constant__ CUtensorMap tmap_w0, const __grid_constant__ CUtensorMap tmap_w1)
{
    using C = Cfg<WBITS, DUAL>;
    constexpr int SETS = C::SETS;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* xs = base;                                             // [XSTAGES][BX][128 B]
    uint8_t* wsm = xs + (size_t)C::XSTAGES * C::X_STAGE_BYTES;      // [SETS][WSTAGES][128][128 B]
    uint64_t* bars = reinterpret_cast<uint64_t*>(wsm + (size_t)SETS * C::WSTAGES * C::W_STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::NUM_BARRIERS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const uint32_t bar0 = smem_u32(bars);
    // full(s): the x tile has landed (TMA transaction bytes) and every conversion thread has stored its row of
    // the stage (SETS * 128 arrivals); empty(s): the MMAs that read the stage have completed (tcgen05.commit).
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (C::STAGES + s); };
    auto full_w = [&](int set, int s) { return bar0 + 8u * (2 * C::STAGES + set * C::WSTAGES + s); };
    auto empty_w = [&](int set, int s) { return bar0 + 8u * (2 * C::STAGES + SETS * C::WSTAGES + set * C::WSTAGES + s); };
    const uint32_t acc_full = bar0 + 8u * (C::NUM_BARRIERS - 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m_tile = blockIdx.x % p.m_tiles, n_tile = blockIdx.x / p.m_tiles;
    const int m0 = m_tile * C::BX, n0 = n_tile * C::BN;
    const int KB = p.K / C::BK;
    constexpr int TMA_WARP = C::DQ_WARPS, MMA_WARP = C::DQ_WARPS + 1, TMAW_WARP = C::DQ_WARPS + 2;

    // ---------------------------------------------------------------- set-up
    if (tid == 0)
    {
        for (int s = 0; s < C::STAGES; s++)
        {
            mbar_init(full(s), SETS * 128 + 1);
            mbar_init(empty(s), 1);
        }
        for (int set = 0; set < SETS; set++)
            for (int s = 0; s < C::WSTAGES; s++)
            {
                mbar_init(full_w(set, s), 1);
                mbar_init(empty_w(set, s), 4 * C::DQ_GROUPS * 32);
            }
        mbar_init(acc_full, 1);
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

    if (warp == TMA_WARP)
    {
        // ------------------------------------------------------------ TMA producer: activation tiles
        if (lane == 0)
        {
            bool ok = true;
            for (int kb = 0; kb < KB && ok; kb++)
            {
                const int s = kb % C::XSTAGES;
                const uint32_t ph = (uint32_t)(kb / C::XSTAGES) & 1u;
                ok = wait_or_abort(empty(s), ph ^ 1u, abort_flag);
                if (!ok)
                    break;
                mbar_arrive_expect_tx(full(s), C::X_STAGE_BYTES);
                tma_load_2d(smem_u32(xs + (size_t)s * C::X_STAGE_BYTES), &tmap_x, full(s), kb * C::BK, m0);
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
            const int chunks = (KB + C::KB_PER_CHUNK - 1) / C::KB_PER_CHUNK;
            for (int chunk = 0; chunk < chunks && ok; chunk++)
            {
                const int s = chunk % C::WSTAGES;
                const uint32_t ph = (uint32_t)(chunk / C::WSTAGES) & 1u;
                for (int set = 0; set < SETS && ok; set++)
                {
                    ok = wait_or_abort(empty_w(set, s), ph ^ 1u, abort_flag);
                    if (!ok)
                        break;
                    mbar_arrive_expect_tx(full_w(set, s), C::W_STAGE_BYTES);
                    tma_load_2d(smem_u32(wsm + (size_t)(set * C::WSTAGES + s) * C::W_STAGE_BYTES),
                                set == 0 ? &tmap_w0 : &tmap_w1, full_w(set, s), chunk * 128, n0);
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
            for (int kb = 0; kb < KB && ok; kb++)
            {
                const int sx = kb % C::STAGES, sa = sx;
                ok = wait_hot(full(sx), (uint32_t)(kb / C::STAGES) & 1u, abort_flag);
                if (!ok)
                    break;
                tcgen05_fence_after();
                const uint32_t xaddr = smem_u32(xs + (size_t)sx * C::X_STAGE_BYTES);
#pragma unroll
                for (int set = 0; set < SETS; set++)
                {
                    const uint32_t d_tmem = tmem_base + (uint32_t)(set * C::BX);
                    const uint32_t a_tmem = tmem_base + (uint32_t)(C::A_COL0 + (set * C::ASTAGES + sa) * C::A_STAGE_COLS);
#pragma unroll
                    for (int kk = 0; kk < C::BK / 16; kk++)
                        tcgen05_mma_ts(d_tmem, a_tmem + kk * 8, smem_desc_k_sw128(xaddr + kk * 32), idesc,
                                       (kb | kk) != 0 ? 1u : 0u);
                }
                tcgen05_commit(empty(sx)); // arrives when the MMAs above have consumed the stage
            }
            tcgen05_commit(acc_full);
        }
    }
    else
    {
        // ------------------------------------------------------------ dequantise into tensor memory
        const int set = DUAL ? warp / (4 * C::DQ_GROUPS) : 0;
        const int grp = (warp >> 2) % C::DQ_GROUPS;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;           // row of the tile = TMEM lane
        const int n = min(n0 + r, p.N - 1);          // rows past N read the last row's parameters, never stored
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int kb_per_group = p.group / C::BK;
        const uint32_t wsm_s = smem_u32(wsm), xs_s = smem_u32(xs);
        bool ok = true;

        auto load_scale = [&](int gidx) -> float {
            const size_t i = (size_t)n * p.G + gidx;
            return p.scale_f32 ? __ldg(static_cast<const float*>(p.scale[set]) + i)
                               : __half2float(__ldg(static_cast<const __half*>(p.scale[set]) + i));
        };
        auto load_zp = [&](int gidx) -> uint32_t {
            if (WBITS == 4)
                return (__ldg(p.zp[set] + (size_t)n * p.zp_row_bytes + (gidx >> 1)) >> (4 * (gidx & 1))) & 0xF;
            return __ldg(p.zp[set] + (size_t)n * p.G + gidx);
        };
        // (scale, zero-point) of the k-block in hand and, prefetched one iteration ahead, of the next one: the
        // loads complete while the current k-block is converted.
        float sc = 0.f, sc_next = 0.f;
        uint32_t zq = 0, zq_next = 0;
        if (grp < KB)
        {
            sc_next = load_scale(grp / kb_per_group);
            zq_next = load_zp(grp / kb_per_group);
        }

        // Raw bytes of k-block kb -> 64 fp16 (q - zp) * scale in k order: register i holds k = 2i (low half) and
        // k = 2i + 1 (high half).  Returns false if the wait for the raw chunk was aborted.
        auto convert = [&](int kb, uint32_t (&a)[32]) -> bool {
            const int chunk = kb / C::KB_PER_CHUNK, j = kb % C::KB_PER_CHUNK, sw = chunk % C::WSTAGES;
            sc = sc_next, zq = zq_next;
            {
                const int kb_n = kb + C::DQ_GROUPS;
                if (kb_n < KB && kb_n / kb_per_group != kb / kb_per_group)
                {
                    sc_next = load_scale(kb_n / kb_per_group);
                    zq_next = load_zp(kb_n / kb_per_group);
                }
            }
            if (j < C::DQ_GROUPS) // first k-block of this chunk for this thread
                if (!wait_or_abort(full_w(set, sw), (uint32_t)(chunk / C::WSTAGES) & 1u, abort_flag))
                    return false;
            // this row's raw bytes: 16-byte chunk c of row r is stored at chunk c ^ (r & 7)
            const uint32_t row = wsm_s + (uint32_t)((set * C::WSTAGES + sw) * C::W_STAGE_BYTES + r * 128);
            constexpr int NV = C::RAW_BYTES / 16;
            uint4 raw[NV];
#pragma unroll
            for (int v = 0; v < NV; v++)
                raw[v] = lds128(row + (uint32_t)(((j * NV + v) ^ (r & 7)) * 16));
            if (j + C::DQ_GROUPS >= C::KB_PER_CHUNK || kb + C::DQ_GROUPS >= KB)
                mbar_arrive(empty_w(set, sw)); // last read of this chunk by this thread

            const __half2 s2 = __float2half2_rn(sc);
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
            return true;
        };
        // Hand the converted k-block to the tensor core: wait for the A stage, store to tensor memory.
        auto stage = [&](int kb, const uint32_t (&a)[32]) -> bool {
            const int sa = kb % C::ASTAGES;
            if (!wait_or_abort(empty(sa), ((uint32_t)(kb / C::ASTAGES) & 1u) ^ 1u, abort_flag))
                return false;
            tcgen05_fence_after();
            tmem_st_32x32(tmem_base + lane_addr + (uint32_t)(C::A_COL0 + (set * C::ASTAGES + sa) * C::A_STAGE_COLS), a);
            return true;
        };
        auto publish = [&](int kb) {
            tcgen05_wait_st();
            tcgen05_fence_before();
            mbar_arrive(full(kb % C::ASTAGES));
        };
        // Two register buffers: while the tensor-memory store of one k-block drains, the next one is converted.
        uint32_t a0[32], a1[32];
        int kb = grp;
        if (kb < KB)
            ok = convert(kb, a0);
        while (ok && kb < KB)
        {
            const int kb1 = kb + C::DQ_GROUPS, kb2 = kb1 + C::DQ_GROUPS;
            if (!(ok = stage(kb, a0)))
                break;
            if (kb1 < KB && !(ok = convert(kb1, a1)))
                break;
            publish(kb);
            if (kb1 >= KB)
                break;
            if (!(ok = stage(kb1, a1)))
                break;
            if (kb2 < KB && !(ok = convert(kb2, a0)))
                break;
            publish(kb1);
            kb = kb2;
        }

        // ------------------------------------------------------------ epilogue
        // D holds y transposed (lane = weight row n, column = batch row m).  With fp16 output the tile is turned
        // around through shared memory (the x ring is idle by now) so that y is written in 16-byte pieces along n;
        // otherwise every value is stored on its own.
        if (ok)
            ok = wait_or_abort(acc_full, 0u, abort_flag);
        if (ok)
            tcgen05_fence_after();
        {
            constexpr int PEERS = C::DQ_WARPS / 4;   // warps per TMEM lane quarter
            const int peer = warp >> 2;              // 0 .. PEERS-1
            const int nrow = n0 + r;
            const float bias = (p.has_bias && nrow < p.N) ? __ldg(p.bias + nrow) : 0.f;
            // the tile is staged in the x ring as [BX][128] halves, row m = 256 bytes
            if (ok)
            {
                for (int cb = peer; cb < C::BX / 32; cb += PEERS)
                {
                    uint32_t d0[32], d1[32];
                    tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(cb * 32), d0);
                    if (DUAL)
                        tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(C::BX + cb * 32), d1);
                    tcgen05_wait_ld();
#pragma unroll
                    for (int jx = 0; jx < 32; jx++)
                    {
                        const int ml = cb * 32 + jx, m = m0 + ml;
                        float v = __uint_as_float(d0[jx]);
                        if (DUAL)
                        {
                            const float u = __uint_as_float(d1[jx]);
                            v = v * (1.0f / (1.0f + expf(-v))) * u;
                        }
                        v += bias;
                        if (p.has_addend && m < p.M && nrow < p.N)
                            v += p.y_f32 ? reinterpret_cast<const float*>(p.bias)[(size_t)m * p.N + nrow]
                                         : __half2float(reinterpret_cast<const __half*>(p.bias)[(size_t)m * p.N + nrow]);
                        if (p.fast_store)
                            sts16(xs_s + (uint32_t)((ml * 128 + r) * 2), __half_as_ushort(__float2half_rn(v)));
                        else if (m < p.M && nrow < p.N)
                        {
                            if (p.y_f32)
                                static_cast<float*>(p.y)[(size_t)m * p.N + nrow] = v;
                            else
                                static_cast<__half*>(p.y)[(size_t)m * p.N + nrow] = __float2half_rn(v);
                        }
                    }
                }
            }
            if (p.fast_store)
            {
                // all conversion warps (and only they) meet here, whether or not they got this far unharmed
                asm volatile("bar.sync 1, %0;" ::"n"(C::DQ_WARPS * 32) : "memory");
                if (!*abort_flag)
                {
                    const int t = warp * 32 + lane; // 0 .. DQ_WARPS*32-1
                    for (int c = t; c < C::BX * 16; c += C::DQ_WARPS * 32)
                    {
                        const int ml = c >> 4, nc = (c & 15) * 8;
                        const int m = m0 + ml, n = n0 + nc;
                        if (m < p.M && n < p.N)
                            *reinterpret_cast<uint4*>(static_cast<__half*>(p.y) + (size_t)m * p.N + n) =
                                lds128(xs_s + (uint32_t)((ml * 128 + nc) * 2));
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

template <int WBITS, bool DUAL>
cudaError_t launch(const GemmParams& p, const CUtensorMap& tx, const CUtensorMap& tw0, const CUtensorMap& tw1,
                   int grid, cudaStream_t stream)
{
    using C = Cfg<WBITS, DUAL>;
    static bool configured[nnf::kMaxDevices] = {}; // the attribute belongs to the device that is current
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        return e;
    if (dev < 0 || dev >= nnf::kMaxDevices)
        return cudaErrorInvalidDevice;
    if (!configured[dev])
    {
        e = cudaFuncSetAttribute(dq_gemm_kernel<WBITS, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)C::SMEM_BYTES);
        if (e != cudaSuccess)
            return e;
        configured[dev] = true;
    }
    (void)cudaGetLastError();
    dq_gemm_kernel<WBITS, DUAL><<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(p, tx, tw0, tw1);
    return cudaGetLastError();
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

size_t gemm_workspace_bytes(const nnf_b200_ctx*, const nnf_b200_linear_desc& d)
{
    return needs_prepass(d) ? ((size_t)d.M * d.K * sizeof(__half) + 255) / 256 * 256 : 0;
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
    return NNF_B200_OK;
}

int gemm_launch(nnf_b200_ctx* ctx, cudaStream_t stream, const nnf_b200_linear_desc& d, const void* x,
                const nnf_b200_qweight* w, const nnf_b200_qweight* w2, const void* gain, const void* bias, void* y,
                void* workspace, size_t workspace_bytes)
{
    if (needs_prepass(d))
    {
        const size_t need = gemm_workspace_bytes(ctx, d);
        if (!workspace || workspace_bytes < need)
            return set_error(ctx, NNF_B200_EWORKSPACE,
                             "workspace of " + std::to_string(need) + " bytes required (fp16 copy of the activations)");
        __half* xh = static_cast<__half*>(workspace);
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
    const bool dual = d.epilogue == NNF_B200_EPILOGUE_SILU_MUL;
    const int bx = dual ? 128 : 256;
    const int row_bytes = d.w_bits == 4 ? d.K / 2 : d.K;
    GemmParams p{};
    p.scale[0] = w->scale;
    p.zp[0] = static_cast<const uint8_t*>(w->zp);
    if (dual)
    {
        p.scale[1] = w2->scale;
        p.zp[1] = static_cast<const uint8_t*>(w2->zp);
    }
    p.bias = static_cast<const float*>(bias);
    p.y = y;
    p.status = ctx->dev_status;
    p.M = d.M, p.N = d.N, p.K = d.K;
    p.group = d.group_size > 0 ? d.group_size : d.K;
    p.G = d.K / p.group;
    p.zp_row_bytes = d.w_bits == 4 ? (p.G + 1) / 2 : p.G;
    p.y_f32 = d.y_dtype == NNF_B200_F32;
    p.scale_f32 = d.scale_dtype == NNF_B200_F32;
    p.has_addend = d.epilogue == NNF_B200_EPILOGUE_ADD;
    p.has_bias = bias != nullptr && !p.has_addend;
    p.m_tiles = (d.M + bx - 1) / bx;
    p.fast_store = !p.y_f32 && d.N % 8 == 0 && (reinterpret_cast<uintptr_t>(y) & 15u) == 0;
    const int n_tiles = (d.N + 127) / 128;

    // x: fp16 [M][K], boxes of BX rows x 64 elements (the tensor map is not cached: x moves between calls)
    alignas(64) CUtensorMap tx;
    if (!encode_tensor_map_2d(ctx->encode_tiled, &tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x, (uint64_t)d.K,
                              (uint64_t)d.M, (uint64_t)d.K * 2, 64, (uint32_t)bx, CU_TENSOR_MAP_SWIZZLE_128B))
        return set_error(ctx, NNF_B200_ECUDA, "cuTensorMapEncodeTiled failed for the activations");
    // copied by value at once: a later lookup may empty the context's cache
    alignas(64) CUtensorMap tw0v, tw1v;
    const CUtensorMap* tw0 = weight_tensor_map(ctx, w->wq, d.N, row_bytes, 128, 128);
    if (tw0)
        tw0v = *tw0;
    const CUtensorMap* tw1 = dual ? weight_tensor_map(ctx, w2->wq, d.N, row_bytes, 128, 128) : tw0;
    if (tw1)
        tw1v = *tw1;
    if (!tw0 || !tw1)
        return set_error(ctx, NNF_B200_ECUDA, "cuTensorMapEncodeTiled failed for the weight tensor");

    const int grid = p.m_tiles * n_tiles;
    cudaError_t e;
    if (d.w_bits == 4)
        e = dual ? launch<4, true>(p, tx, tw0v, tw1v, grid, stream) : launch<4, false>(p, tx, tw0v, tw1v, grid, stream);
    else
        e = dual ? launch<8, true>(p, tx, tw0v, tw1v, grid, stream) : launch<8, false>(p, tx, tw0v, tw1v, grid, stream);
    if (e != cudaSuccess)
        return set_error(ctx, NNF_B200_ECUDA, std::string("dq_gemm launch: ") + cudaGetErrorString(e));
    ctx->launches++;
    return NNF_B200_OK;
}
} // namespace nnf
