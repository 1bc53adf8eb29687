/*
 * nnf_b200 -- C ABI of the hand-written sm_100a kernels for NNFusion's
 * dequantize-fused low-bit linear path.
 *
 * The library is what the generated `cuda_codegen` runtime links instead of
 * (a) the element-wise Convert / Subtract / Multiply kernels that materialise
 * dequantised weights and (b) the cuBLAS call behind `Dot`; for a whole decoder
 * layer at decode time also instead of (c) the rotary / BatchMatMul / Softmax
 * chain of one attention step and (d) the NCCL all-reduce at the shard boundary
 * of a tensor-parallel layer.  All entry points are stream-ordered, take plain
 * device pointers, and never allocate device memory: like every kernel of the
 * generated runtime they receive tensors that live in the runtime's own memory
 * pool.  Kernels are launched as programmatic dependents of whatever precedes
 * them on the stream (they wait for it before touching anything it may have
 * written).
 *
 * Each declaration names the reference interface it stands in for (paths are
 * relative to the reference project root).
 */
#ifndef NNF_B200_H_
#define NNF_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NNF_B200_VERSION 1

#if defined(__GNUC__)
#define NNF_B200_API __attribute__((visibility("default")))
#else
#define NNF_B200_API
#endif

/* Status codes.  The generated code wraps calls in a macro that throws
 * std::runtime_error on non-zero, shaped like CUDA_SAFE_CALL / CUBLAS_SAFE_CALL
 * (src/nnfusion/core/kernels/cuda_gpu/cuda_langunit.cpp:47-62,115-129). */
enum
{
    NNF_B200_OK = 0,
    NNF_B200_EINVAL = 1,     /* malformed descriptor or null pointer            */
    NNF_B200_ENOTSUP = 2,    /* shape / type combination not implemented         */
    NNF_B200_ECUDA = 3,      /* a CUDA runtime or driver call failed             */
    NNF_B200_EWORKSPACE = 4, /* workspace too small or missing                   */
    NNF_B200_ETIMEDOUT = 5,  /* a bounded device-side wait gave up               */
    NNF_B200_EALIGN = 6      /* a pointer or leading dimension is misaligned     */
};

/* Element types of activations, scales and outputs (the reference's
 * element::f32 / element::f16, src/nnfusion/common/type/element_type.hpp:41-55). */
enum
{
    NNF_B200_F32 = 0,
    NNF_B200_F16 = 1
};

enum
{
    NNF_B200_PROLOGUE_NONE = 0,
    /* x <- x * rsqrt(mean(x^2) + eps) * gain, row-wise, before the contraction.
     * Replaces the Multiply -> Sum -> Divide -> Add -> Rsqrt -> Multiply chain
     * (reduce: src/nnfusion/core/kernels/cuda_gpu/kernels/reduce.hpp:18-600). */
    NNF_B200_PROLOGUE_RMSNORM = 1
};

enum
{
    NNF_B200_EPILOGUE_NONE = 0,
    /* y += bias[n].  Replaces cuda::MatMulAdd's separate add kernel
     * (src/nnfusion/core/kernels/cuda_gpu/kernels/matmuladd.cpp:43-71,145-217). */
    NNF_B200_EPILOGUE_BIAS = 1,
    /* y = SiLU(x.W^T) * (x.W2^T) with a second weight set; replaces the fused
     * Sigmoid -> Multiply -> Multiply element-wise kernel
     * (src/nnfusion/core/kernels/cuda_gpu/kernels/elementwise_fused.cpp:42-189). */
    NNF_B200_EPILOGUE_SILU_MUL = 2,
    /* y = x.W^T + c with c an [M,N] tensor of y's element type, passed in the `bias`
     * argument (it may be y itself).  cuda::MatMulAdd with its full-size addend
     * (src/nnfusion/core/kernels/cuda_gpu/kernels/matmuladd.cpp:29-93; the operator's C is
     * already broadcast to [M,N], src/nnfusion/core/operators/generic_op/generic_op_define/MatMulAdd.cpp:6-35):
     * the residual connection of a decoder layer. */
    NNF_B200_EPILOGUE_ADD = 3
};

enum
{
    NNF_B200_KERNEL_AUTO = 0,
    NNF_B200_KERNEL_GEMV = 1, /* small-M, HBM-bound: M <= 16                         */
    NNF_B200_KERNEL_GEMM = 2  /* large-M, tensor-bound: TMA + tcgen05 + TMEM          */
};

/* Descriptor flags. */
enum
{
    /* Small-M kernel: subtract the zero-point from the fp16 integers before the
     * tensor-core multiply (bit-exact integer operands) instead of taking
     * sum((offset + zp) * x) out of the fp32 accumulator afterwards.  Slower;
     * the default differs from it by fp32 rounding only. */
    NNF_B200_FLAG_EXACT_ZP = 1
};

/* One quantised weight matrix W[N, K] as the kernels read it.
 *   bits 8: wq is uint8 [N, K]; zp is uint8 [N, K/group].
 *   bits 4: wq is [N, K/2] bytes, element k in bits 0-3 of byte k/2 for even k
 *           and in bits 4-7 for odd k; zp is packed the same way along the
 *           group axis, [N, ceil(K/group / 2)] bytes.
 *   scale is fp32 or fp16 [N, K/group] (descriptor field scale_dtype).
 * dequant(W)[n,k] = (float(q[n,k]) - float(zp[n,k/group])) * scale[n,k/group],
 * i.e. the Cast -> Sub -> Mul chain of the imported graph
 * (src/nnfusion/core/kernels/cuda_gpu/kernels/elementwise.hpp:33-157, op table
 * src/nnfusion/core/kernels/cuda_gpu/cuda_common_ops.hpp:28-97). */
typedef struct
{
    const void* wq;
    const void* scale;
    const void* zp;
} nnf_b200_qweight;

/* Descriptor of y[M,N] = epilogue(prologue(x)[M,K] . dequant(W)[N,K]^T), the
 * fused replacement of op::Dot with transpose_B
 * (src/nnfusion/core/operators/op_define/dot.cpp:43-135) fed by the dequant chain.
 * x and y are dense row-major (leading dimensions K and N). */
typedef struct
{
    int32_t M, N, K;
    int32_t w_bits;      /* 8 or 4                                                  */
    int32_t group_size;  /* K elements sharing one (scale, zp); 0 = per row (= K)   */
    int32_t x_dtype;     /* NNF_B200_F32 / NNF_B200_F16                             */
    int32_t y_dtype;
    int32_t scale_dtype;
    int32_t prologue;
    int32_t epilogue;
    float rms_eps;
    int32_t kernel;      /* NNF_B200_KERNEL_*                                       */
    int32_t split_k;     /* 0 = chosen by the library                               */
    int32_t flags;       /* NNF_B200_FLAG_*                                         */
    int32_t reserved[2]; /* must be zero                                            */
} nnf_b200_linear_desc;

typedef struct nnf_b200_ctx nnf_b200_ctx;

/* Per-device set-up, called from the generated runtime's cuda_init() next to
 * cublasCreate (src/nnfusion/engine/pass/codegen/cuda_codegen_pass.cpp:117-168);
 * reads device properties and raises the kernels' shared-memory limits. */
NNF_B200_API int nnf_b200_init(int device, nnf_b200_ctx** ctx);

/* Called from cuda_free() (same file, :194-211). */
NNF_B200_API int nnf_b200_free(nnf_b200_ctx* ctx);

NNF_B200_API const char* nnf_b200_strerror(int status);

/* Text of the last failure on this context ("" if none). */
NNF_B200_API const char* nnf_b200_last_error(const nnf_b200_ctx* ctx);

/* Number of SMs the context's device reports. */
NNF_B200_API int nnf_b200_sm_count(const nnf_b200_ctx* ctx);

/* Bytes of scratch the described call needs (0 if none).  The emitter requests
 * it with KernelEmitter::allocate_tensor so that it is planned into the static
 * pool (src/nnfusion/core/kernels/kernel_emitter.cpp:282-319).  It holds arrival
 * counters in front of partial sums (K split over CTAs at M <= 16; output tiles
 * shared by persistent CTAs above that, where it also holds the fp16 copy of fp32
 * or RMS-normalised activations).  The scratch must be zero-filled once before
 * its first use (nnf_b200_workspace_reset); every call leaves its counters zeroed
 * again, so calls of one descriptor can follow one another on the same buffer;
 * zero-fill it again before it serves another descriptor.  Calls that share one
 * scratch buffer must not overlap on the device.  ctx may be NULL (a 148-SM device
 * is assumed), for sizing at code-generation time. */
NNF_B200_API size_t nnf_b200_linear_workspace_bytes(const nnf_b200_ctx* ctx, const nnf_b200_linear_desc* desc);

/* Launch shape the library would use for a descriptor, for tuning and reporting:
 * out[0] kernel (NNF_B200_KERNEL_*), out[1] warps per CTA, out[2] split-K factor,
 * out[3] load-ring depth, out[4] CTAs, out[5] dynamic shared memory in bytes,
 * out[6] row tiles between two meetings of a CTA's warps, out[7] bits: 1 the CTAs
 * that share a tile ask to be launched as a thread-block cluster (their sums then
 * meet in shared memory; the launch falls back to the workspace when the device
 * cannot hold every cluster at once), 2 weight loads take lines in L1, 4 only the
 * scale / zero-point columns of a CTA's own K range are kept in shared memory,
 * 8 one batch holds every tile of a CTA.  out[6..7] are zero for the tensor-core
 * kernel.  ctx may be NULL (a 148-SM device is assumed).  No reference
 * counterpart: the reference leaves such choices to cuBLAS. */
NNF_B200_API int nnf_b200_linear_plan(const nnf_b200_ctx* ctx, const nnf_b200_linear_desc* desc, int32_t out[8]);

/* Stream-ordered zero fill of a workspace (cudaMemsetAsync). */
NNF_B200_API int nnf_b200_workspace_reset(nnf_b200_ctx* ctx, void* stream, void* workspace, size_t bytes);

/* The fused linear.  Stands in for the kernel sequence
 *   Convert_* -> FusedKernel_*Subtract*Multiply* -> Dot_*_cuda_lib (cuBLAS)
 * that the reference emits into kernel_entry (cuda::Dot:
 * src/nnfusion/core/kernels/cuda_gpu/kernels/dot.cpp:27-372; cuda::ElementWiseFused:
 * .../elementwise_fused.cpp:42-189).
 *   stream     cudaStream_t the emitted call site passes
 *              (src/nnfusion/core/kernels/kernel_emitter.cpp:160-181)
 *   x          [M,K] activations, x_dtype
 *   w          weight set; w2 second set for NNF_B200_EPILOGUE_SILU_MUL, else NULL
 *   gain       [K] fp32 RMSNorm gain, or NULL without that prologue
 *   bias       [N] fp32 bias, or NULL without that epilogue
 *   y          [M,N] output, y_dtype
 * Accumulation is fp32.  Returns a status code; failures are also kept as text
 * for nnf_b200_last_error. */
NNF_B200_API int nnf_b200_linear(nnf_b200_ctx* ctx, void* stream, const nnf_b200_linear_desc* desc, const void* x,
                    const nnf_b200_qweight* w, const nnf_b200_qweight* w2, const void* gain,
                    const void* bias, void* y, void* workspace, size_t workspace_bytes);

/* Size of the scratch array built into the library for nnf_b200_linear_static_scratch. */
#define NNF_B200_STATIC_SCRATCH_BYTES (4 * 1024 * 1024)

/* nnf_b200_linear for callers that cannot hand over a workspace because they cannot
 * allocate device memory any more: loops whose memory budget is frozen after
 * start-up, processes held to a fixed GPU quota.  It has no
 * counterpart in the reference (whose kernels get their scratch planned into the
 * generated runtime's pool).  It serves the small-M kernel (M <= 16), the one whose
 * split-K path needs scratch, and takes that scratch from an array of
 * NNF_B200_STATIC_SCRATCH_BYTES that is part of the library's device image: every GPU
 * that loads the library holds it until the process ends.  It needs no context and
 * calls no allocator.  Shapes whose split-K scratch exceeds the array are refused with
 * NNF_B200_EWORKSPACE (the text in errbuf names both sizes).
 * The first call made while a given device is current fetches the array's device
 * address and reads the device's attributes, and the first call of each kernel variant
 * on a device raises that kernel's shared-memory limit: make those calls outside of
 * any stream capture.  Host threads may call concurrently (the set-up is guarded); the
 * calls themselves still share the one array.  Every call uses the same array and
 * finds in it what the previous call left; the counters that must start at zero are
 * cleared on `stream` by each call.  Two calls that overlap on the GPU (for instance
 * on two streams of one process) race on the array: serialise them.  Each process
 * has its own copy of the array.
 * errbuf (may be NULL) receives a message of at most errbuf_len bytes on failure. */
NNF_B200_API int nnf_b200_linear_static_scratch(void* stream, const nnf_b200_linear_desc* desc, const void* x,
                                                const nnf_b200_qweight* w, const nnf_b200_qweight* w2,
                                                const void* gain, const void* bias, void* y, char* errbuf,
                                                size_t errbuf_len);

/* Companion of nnf_b200_linear_static_scratch (like it, without a counterpart in the
 * reference): reads and clears the status word that kernels launched through that entry
 * point raise when a bounded device-side wait gives up, for the device that is current.
 * Returns NNF_B200_OK, NNF_B200_ETIMEDOUT, or NNF_B200_ECUDA.  Synchronises `stream`,
 * allocates nothing; meant for tests and for a check outside the hot loop. */
NNF_B200_API int nnf_b200_static_scratch_status(void* stream);

/* ---- single-token (decode) attention over a key/value cache ---------------------------------------------
 *
 * out[h] = softmax(rot(q[h]) . K[kv(h)]^T * scale) . V[kv(h)] over cache rows 0 .. position, where row
 * `position` is the new token: its key (through the rotary embedding) and value are written into the caches by
 * the same call.  Stands in for the chain the reference runs for one decoding step of an attention layer:
 * Slice / Negative / Concat / Multiply / Add (rotary embedding; element-wise emitters,
 * src/nnfusion/core/kernels/cuda_gpu/kernels/elementwise.hpp:33-157), BatchMatMul with adj_y
 * (src/nnfusion/core/kernels/cuda_gpu/kernels/batch_matmul.cpp:49-144; operator definition
 * src/nnfusion/core/operators/generic_op/generic_op_define/BatchMatMul.cpp:6-50), Softmax
 * (src/nnfusion/core/kernels/cuda_gpu/kernels/softmax.cpp:78-122) and a second BatchMatMul.
 * Rotary embedding: element pairs (i, i + head_dim/2) of a head are rotated by position * base^(-2i/head_dim)
 * ("rotate half": x*cos + concat(-x[half:], x[:half])*sin). */
typedef struct nnf_b200_attn_desc
{
    int32_t heads;       /* query heads                                                     */
    int32_t kv_heads;    /* key/value heads; heads must be a multiple (grouped queries)      */
    int32_t head_dim;    /* 128                                                             */
    int32_t capacity;    /* rows per head the caches can hold; position < capacity          */
    int32_t position;    /* index of the new token = number of rows already in the caches   */
    int32_t rotary;      /* non-zero: rotate q and the new key                              */
    float rotary_base;   /* 0 -> 10000                                                      */
    float softmax_scale; /* 0 -> 1/sqrt(head_dim)                                           */
    int32_t splits;      /* ranges per head; 0 -> chosen by the library                     */
    int32_t dtype;       /* NNF_B200_F16: q, k, v, caches and out                           */
    int32_t reserved[4]; /* must be zero                                                    */
} nnf_b200_attn_desc;

/* Bytes of scratch the call needs (0 if none); zero-filled once before first use, left zeroed by every call.
 * ctx may be NULL (a 148-SM device is assumed). */
NNF_B200_API size_t nnf_b200_decode_attention_workspace_bytes(const nnf_b200_ctx* ctx, const nnf_b200_attn_desc* desc);

/* q [heads][head_dim], k_new / v_new [kv_heads][head_dim], caches [kv_heads][capacity][head_dim],
 * out [heads][head_dim]; all device pointers, 16-byte aligned.  Stream-ordered, never allocates. */
NNF_B200_API int nnf_b200_decode_attention(nnf_b200_ctx* ctx, void* stream, const nnf_b200_attn_desc* desc,
                                           const void* q, const void* k_new, const void* v_new, void* k_cache,
                                           void* v_cache, void* out, void* workspace, size_t workspace_bytes);

/* ---- one-shot sum all-reduce of a small fp16 tensor over peer memory -------------------------------------
 *
 * out = sum over ranks of bufs[r], added in rank order in fp32 and rounded once, so that every rank gets the
 * same bits.  Stands in for the NCCL call behind cuda::SuperScalerAllReduce
 * (src/nnfusion/core/kernels/cuda_gpu/kernels/allreduce.cpp:18-98;
 * src/tools/nnfusion/templates/super_scaler/super_scaler.cu:244-277) at the shard boundary of a tensor-parallel
 * layer, where the tensor is a few KB per rank and a ring is all latency.
 *
 * bufs[r] / flags[r] (host arrays of `world` entries, world <= 8): rank r's addend buffer and flag words as mapped
 * into THIS process (peer pointers for r != rank; memory every rank has mapped, e.g. from cuMemMap or CUDA IPC).
 * A buffer has two halves, half_stride_bytes apart; call number e reads half (e & 1) of every rank, so a rank may
 * be one call ahead of a peer that is still reading.  epoch: the call number, starting at 1 and growing by one per
 * call, the same on every rank -- or 0 to let the kernel count calls itself in words kept after the flags (then a
 * captured sequence with an even number of calls can be replayed).  Other rules for the caller: the flag words
 * (nnf_b200_allreduce_flag_bytes of them) start zeroed and are never written by anyone else; the addend of this
 * call must be complete in its half, in stream order, before the call.  A flag area sized for `count` elements
 * serves every call of up to that many elements (its layout does not depend on the size of a call), as long as
 * all ranks make the same sequence of calls on it.  count: fp16 elements, a multiple of 8;
 * bufs 16-byte aligned.
 * A rank whose peers never call gives up after about 0.4 s, writes nothing, and nnf_b200_device_status then
 * reports NNF_B200_ETIMEDOUT. */
NNF_B200_API size_t nnf_b200_allreduce_flag_bytes(size_t count);
NNF_B200_API int nnf_b200_allreduce_oneshot(nnf_b200_ctx* ctx, void* stream, int rank, int world,
                                            const void* const* bufs, void* const* flags, size_t count,
                                            size_t half_stride_bytes, void* out, uint32_t epoch);

/* ---- small-M linear whose result is summed over the ranks of a tensor-parallel group in the same launch ----
 *
 * y = sum over ranks r of x_r . dequant(W_r)^T (+ bias or addend, applied once, on the sum): the row-parallel
 * linear of a sharded layer and the all-reduce that follows it, as one kernel.  In the reference these are a Dot
 * kernel and cuda::SuperScalerAllReduce (src/nnfusion/core/kernels/cuda_gpu/kernels/allreduce.cpp:18-98).
 * The CTA that finishes a 16-row tile of the output writes its fp32 sums into every rank's buffer (plain stores,
 * over NVLink for the peers'), announces the tile to every peer, waits (bounded) for their announcements of the
 * same tile, finds everybody's sums in its own memory and adds them in rank order, so every rank stores the same
 * bits and the exchange of early tiles overlaps the arithmetic of later ones.
 *
 * peers->bufs[r] / flags[r]: rank r's buffer (two halves of world * M * N floats, one M * N block per sender,
 * half_stride_bytes apart) and flag words
 * (nnf_b200_linear_allreduce_flag_bytes(desc) bytes, zeroed once, never written by anyone else) as mapped into
 * this process.  peers->epoch: call number, from 1, +1 per call, the same on every rank -- or 0 to count on the
 * device (then a captured sequence with an even number of calls can be replayed).  Every rank calls with the same
 * descriptor.  Restrictions: M <= 16, fp16 output, no RMSNorm prologue, no SiLU*mul epilogue. */
typedef struct nnf_b200_peers
{
    int32_t rank, world;
    void* const* bufs;
    void* const* flags;
    size_t half_stride_bytes;
    uint32_t epoch;
} nnf_b200_peers;

NNF_B200_API size_t nnf_b200_linear_allreduce_flag_bytes(const nnf_b200_linear_desc* desc);
NNF_B200_API int nnf_b200_linear_allreduce(nnf_b200_ctx* ctx, void* stream, const nnf_b200_linear_desc* desc,
                                           const void* x, const nnf_b200_qweight* w, const void* bias, void* y,
                                           void* workspace, size_t workspace_bytes, const nnf_b200_peers* peers);

/* Reads (and clears) the device-side status word: 0, or NNF_B200_ETIMEDOUT when a
 * bounded wait inside a kernel gave up since the last query.  Synchronises the
 * stream; meant for tests and debugging, not for the hot path. */
NNF_B200_API int nnf_b200_device_status(nnf_b200_ctx* ctx, void* stream);

/* Number of kernels the library has launched on this context since init
 * (a counter for benchmarks; reset by passing reset != 0). */
NNF_B200_API uint64_t nnf_b200_launch_count(nnf_b200_ctx* ctx, int reset);

/* Host helper: pack `rows` x `cols` uint4 values (one per byte) two per byte,
 * low nibble first, into rows x ceil(cols/2) bytes.  Used when constants are
 * written at compile time (src/nnfusion/core/kernels/cuda_gpu/kernels/constant.cpp:34-61). */
NNF_B200_API int nnf_b200_pack_u4(const uint8_t* vals, size_t rows, size_t cols, uint8_t* out);

#ifdef __cplusplus
}
#endif
#endif /* NNF_B200_H_ */
