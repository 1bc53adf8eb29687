// Internal declarations shared by the C-ABI translation unit and the kernel launchers.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <map>
#include <string>
#include <tuple>

#include "nnf_b200.h"

struct nnf_b200_ctx
{
    int device = 0;
    int sm_count = 0;
    int smem_optin = 0;          // max dynamic shared memory per block (opt-in)
    int cc_major = 0, cc_minor = 0;
    uint64_t launches = 0;
    std::string last_error;
    void* encode_tiled = nullptr; // cuTensorMapEncodeTiled entry point (driver)
    int* dev_status = nullptr;    // device word set to non-zero when a bounded device-side wait gave up
    // Tensor maps of weight tensors, keyed by (address, rows, row bytes, box bytes, box rows, swizzle).
    std::map<std::tuple<const void*, int, int, int, int, int>, CUtensorMap> tensor_maps;
};

namespace nnf
{
constexpr int kMaxDevices = 64; // per-device bookkeeping (shared-memory opt-ins) is kept in arrays of this size

// Launch plan of the small-M kernel, shared by workspace sizing and launch.
struct GemvPlan
{
    int mb = 1;          // 8-row batches of x (1: M <= 8, 2: M <= 16)
    int warps = 8;       // warps per CTA = K slices per split
    int splits = 1;      // split-K factor
    int depth = 4;       // tiles in the shared-memory load ring
    int ctas_per_split = 1;
    int row_tiles = 0;   // ceil(N / 16)
    int slices = 0;      // 128-byte weight-row slices along K
    bool dual = false;
    bool xsplit = false; // activations carried as fp16 hi + lo
    bool exact = false;  // remove zero-points before the multiply instead of correcting the fp32 sum
    size_t slot_floats = 0;     // floats per (split, row tile) partial slot
    size_t workspace_bytes = 0; // 0 when splits == 1
    size_t smem_bytes = 0;      // dynamic shared memory of the launch
    int batch = 1;              // row tiles between two reductions over the CTA's warps
    int tq = 4;                 // accumulator column pairs that carry batch rows
    int scale_tile_bytes = 0;   // scales of one 16-row tile
    int zp_tile_bytes = 0;      // zero-points of one 16-row tile
    int pset_bytes = 0;         // shared memory per ring slot and weight set for both (0: plain loads)
    int lsu_weights = 0;        // weights by per-thread cp.async instead of bulk copies
    int xfrag_bytes = 0;        // shared memory per warp for the activation fragments of batch rows 8..15
    int direct = 0;             // served by the register-pipeline kernel (dq_gemv_direct.cu) instead of the ring kernel
    int prefetch_tiles = 0;     // register-pipeline kernel: L2 prefetch window in row tiles
    int l1_lines = 0;           // register-pipeline kernel: weight loads take lines in L1
    int sm_sc_row = 0;          // register-pipeline kernel: bytes of a row of scales in shared memory
    int sm_zp_row = 0;          // ... and of a row of zero-points
    int range_layout = 0;       // ... which hold only the columns of a CTA's own K range
    int pset_sm = 0;            // ... shared memory per tile and weight set for both
    int cluster = 0;            // ... the splits of a tile form a thread-block cluster (sums meet in shared memory)
    int param_bufs = 2;         // ... and the number of batches of parameters held at a time (1: one batch is all)
};

int set_error(nnf_b200_ctx* ctx, int status, const std::string& msg);
// Descriptor and operand checks of a linear call that need no context; *why receives the reason on failure.
int check_linear_call(const nnf_b200_linear_desc* d, const void* x, const nnf_b200_qweight* w,
                      const nnf_b200_qweight* w2, const void* gain, const void* bias, const void* y,
                      const void* workspace, std::string* why);

// Launch attribute that lets a kernel start while the launch before it on the stream is finishing (programmatic
// dependent launch); every kernel launched with it executes griddepcontrol.wait before it touches anything that
// launch may have written.
void overlap_attribute(cudaLaunchAttribute* attr, unsigned* count);

// Cached 2-D byte tensor map [rows][row_bytes] with a box of box_rows x box_bytes (128-byte swizzle when
// box_bytes == 128, none otherwise); nullptr if the driver refuses it.
const CUtensorMap* weight_tensor_map(nnf_b200_ctx* ctx, const void* base, int rows, int row_bytes, int box_bytes,
                                     int box_rows);

// allow_direct = false keeps the plan on the ring kernel (the one that takes the zero-points out before the multiply).
int gemv_plan(const nnf_b200_ctx* ctx, const nnf_b200_linear_desc& d, GemvPlan* plan, std::string* why,
              bool allow_direct = true);
bool gemv_direct_plan(const nnf_b200_ctx* ctx, const nnf_b200_linear_desc& d, GemvPlan* plan);
cudaError_t gemv_direct_dispatch(const nnf_b200_linear_desc& d, const GemvPlan& plan, const void* x,
                                 const nnf_b200_qweight* w, const nnf_b200_qweight* w2, const void* gain,
                                 const void* bias, void* y, int* status, void* workspace, cudaStream_t stream,
                                 const nnf_b200_peers* peers = nullptr);
int gemv_launch(nnf_b200_ctx* ctx, cudaStream_t stream, const nnf_b200_linear_desc& d, const GemvPlan& plan,
                const void* x, const nnf_b200_qweight* w, const nnf_b200_qweight* w2, const void* gain,
                const void* bias, void* y, void* workspace, const nnf_b200_peers* peers = nullptr);
int gemv_configure(nnf_b200_ctx* ctx);

size_t gemm_workspace_bytes(const nnf_b200_ctx* ctx, const nnf_b200_linear_desc& d);
int gemm_supported(const nnf_b200_ctx* ctx, const nnf_b200_linear_desc& d, std::string* why);
int gemm_launch(nnf_b200_ctx* ctx, cudaStream_t stream, const nnf_b200_linear_desc& d, const void* x,
                const nnf_b200_qweight* w, const nnf_b200_qweight* w2, const void* gain, const void* bias,
                void* y, void* workspace, size_t workspace_bytes);
int gemm_configure(nnf_b200_ctx* ctx);

size_t allreduce_flag_bytes(size_t count);
int allreduce_launch(nnf_b200_ctx* ctx, cudaStream_t stream, int rank, int world, const void* const* bufs,
                     void* const* flags, size_t count, size_t half_stride, void* out, uint32_t epoch);

int attn_check(const nnf_b200_attn_desc& d, std::string* why);
size_t attn_workspace_bytes(const nnf_b200_ctx* ctx, const nnf_b200_attn_desc& d);
int attn_launch(nnf_b200_ctx* ctx, cudaStream_t stream, const nnf_b200_attn_desc& d, const void* q, const void* k_new,
                const void* v_new, void* k_cache, void* v_cache, void* out, void* workspace);
} // namespace nnf
