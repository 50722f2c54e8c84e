// Shared device helpers and internal structures of the sm_100a MoE library.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cfloat>
#include <cstddef>
#include <cstdint>

#include "p92b_moe.h"

namespace p92b {

constexpr int kExperts = P92B_ROUTED_EXPERTS;
constexpr int kTop = P92B_TOP_K;

// Error words a kernel can record in p92b_plan::status instead of faulting.
enum : int {
    kStatusOk = 0,
    kStatusBadExpertId = 1,   // an expert id outside the bank's range was clamped
    kStatusWaitExpired = 2,   // a bounded mbarrier wait gave up
    kStatusBadPointer = 3,    // a matrix of a caller's projection table is not 16-byte aligned
};

__device__ __forceinline__ float bf16_bits_to_float(std::uint16_t bits) {
    return __uint_as_float(static_cast<std::uint32_t>(bits) << 16);
}

__device__ __forceinline__ std::uint16_t float_to_bf16_bits(float value) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(value));
}

__device__ __forceinline__ float decode_e4m3(std::uint8_t bits) {
    __nv_fp8_e4m3 value;
    value.__x = bits;
    return static_cast<float>(value);
}

// Two E2M1 values (low nibble first) -> packed f16x2, exact.
__device__ __forceinline__ std::uint32_t e2m1x2_to_f16x2(std::uint32_t byte) {
    std::uint32_t out;
    asm("{ .reg .b8 lo, hi; .reg .b16 t;\n"
        "  cvt.u16.u32 t, %1;\n"
        "  mov.b16 {lo, hi}, t;\n"
        "  cvt.rn.f16x2.e2m1x2 %0, lo; }\n"
        : "=r"(out)
        : "r"(byte));
    return out;
}

// One 16-element NVFP4 block from 16 floats, the arithmetic of the reference
// quantiser (amax -> E4M3 scale of amax*gs/6 -> values * gs/scale -> E2M1,
// round-to-nearest-even).  Returns the 8 packed bytes; *scale_bits gets the scale.
__device__ __forceinline__ uint2 quantize_block16(const float (&v)[16], float global_scale,
                                                  std::uint8_t* scale_bits) {
    float maximum = 0.0F;
#pragma unroll
    for (int i = 0; i < 16; ++i) maximum = fmaxf(maximum, fabsf(v[i]));
    const __nv_fp8_e4m3 scale(maximum * (global_scale / 6.0F));
    *scale_bits = scale.__x;
    const float decoded = static_cast<float>(scale);
    const float multiplier = decoded == 0.0F ? 0.0F : global_scale / decoded;
    std::uint32_t words[2] = {0U, 0U};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 pair = make_float2(v[2 * i] * multiplier, v[2 * i + 1] * multiplier);
        const std::uint32_t byte = __nv_fp4x2_e2m1(pair).__x;
        words[i >> 2] |= byte << ((i & 3) * 8);
    }
    return make_uint2(words[0], words[1]);
}

// Top-8 of one token by one warp: lane l holds experts l, l+32, ..., l+224 in registers.
// Eight rounds of (local best, warp butterfly arg-max) with the reference's total order: higher
// corrected score first, equal scores -> lower id (cuda/nvfp4_ops.cu:391-392,411-412).  Weights
// are the uncorrected sigmoid of the winners, summed in slot order and scaled by
// routed_scale/total (:420,425-432).  The score is written exactly as the reference writes it and
// every file using this is compiled with --use_fast_math like the reference, so expf and the
// divisions lower to the same hardware approximations.  lg/ids/weights point at this token's row.
__device__ __forceinline__ void warp_top8(const float* __restrict__ lg, const float* __restrict__ bias,
                                          std::int32_t* __restrict__ ids, float* __restrict__ weights,
                                          float routed_scale) {
    const int lane = threadIdx.x & 31;
    // One 64-bit word per candidate: the high half is an order-preserving integer image of the corrected score (0 for
    // a NaN: a comparison-based scan never picks it), the low half is ~id, so that "greater" means higher score, then
    // lower id - the reference's total order (cuda/nvfp4_ops.cu:391-392,411-412) in one unsigned comparison.
    unsigned long long cand[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        const float raw = 1.0F / (1.0F + expf(-lg[e]));
        const float corrected = raw + bias[e];
        const std::uint32_t bits = __float_as_uint(corrected);
        const std::uint32_t key = corrected != corrected ? 0U : (bits & 0x80000000U ? ~bits : bits | 0x80000000U);
        cand[i] = (static_cast<unsigned long long>(key) << 32) | static_cast<std::uint32_t>(~e);
    }
    // Each lane first orders its own eight candidates, best first: a 19-comparator network on registers.  A round of
    // the selection then only looks at the head of each lane's list.
#define P92B_ORDER(a, b)                                                       \
    {                                                                          \
        const unsigned long long hi = cand[a] > cand[b] ? cand[a] : cand[b];   \
        const unsigned long long lo = cand[a] > cand[b] ? cand[b] : cand[a];   \
        cand[a] = hi; cand[b] = lo;                                            \
    }
    P92B_ORDER(0, 1) P92B_ORDER(2, 3) P92B_ORDER(4, 5) P92B_ORDER(6, 7)
    P92B_ORDER(0, 2) P92B_ORDER(1, 3) P92B_ORDER(4, 6) P92B_ORDER(5, 7)
    P92B_ORDER(1, 2) P92B_ORDER(5, 6)
    P92B_ORDER(0, 4) P92B_ORDER(1, 5) P92B_ORDER(2, 6) P92B_ORDER(3, 7)
    P92B_ORDER(2, 4) P92B_ORDER(3, 5)
    P92B_ORDER(1, 2) P92B_ORDER(3, 4) P92B_ORDER(5, 6)
#undef P92B_ORDER
    int chosen_id = 0;            // lane k keeps slot k's expert
    // The eight rounds stay a loop: unrolled they are a few thousand instructions, and a block that
    // runs this alone (the routing block of the fused kernels) then waits on instruction fetches.
#pragma unroll 1
    for (int slot = 0; slot < 8; ++slot) {
        // warp arg-max over the heads, two reductions one after the other: the maximum of the score images, then the
        // lowest id among the lanes that hold it (one lane, unless two scores are exactly equal or every list is down
        // to NaNs).  A vote for the holder and a shuffle of its id instead of the second reduction is three dependent
        // warp-wide steps and a branch: 200 cycles per round against the 120 of this form.
        const std::uint32_t key = static_cast<std::uint32_t>(cand[0] >> 32);
        const std::uint32_t my_id = ~static_cast<std::uint32_t>(cand[0]);       // an exhausted list reads 0xffffffff
        const std::uint32_t top = __reduce_max_sync(0xffffffffU, key);
        const int winner = static_cast<int>(__reduce_min_sync(0xffffffffU, key == top ? my_id : 0xffffffffU));
        if ((winner & 31) == lane && static_cast<std::uint32_t>(winner) == my_id) {
#pragma unroll
            for (int i = 0; i < 7; ++i) cand[i] = cand[i + 1];
            cand[7] = 0ULL;                                    // exhausted: image 0, id 0xffffffff
        }
        if (lane == slot) chosen_id = winner;
    }
    // weights: the uncorrected sigmoid of the winners (the same expression as above, so the same bits), summed in slot
    // order and scaled by routed_scale / total (:420,425-432)
    const float chosen_weight = lane < 8 ? 1.0F / (1.0F + expf(-lg[chosen_id & (kExperts - 1)])) : 0.0F;
    float total = 0.0F;
#pragma unroll
    for (int slot = 0; slot < 8; ++slot) total += __shfl_sync(0xffffffffU, chosen_weight, slot);
    const float multiplier = routed_scale / total;
    if (lane < 8) {
        ids[lane] = chosen_id;
        weights[lane] = chosen_weight * multiplier;
    }
}

// Layout of one layer's expert weights inside the library (device memory).
// Entry e = local expert index, entry local_experts = the shared expert.
//
// The tensor-core kernels read the weights as a pure stream: for every 128-row tile and K block the
// bytes of one pipeline stage are contiguous in memory, already in the shared-memory image the MMA
// descriptors expect, so a stage is ONE bulk copy and an expert's tiles are one sequential read.
//   chunk (36,864 B) = box0 (16 KB) | box1 (16 KB) | scales0 (2 KB) | scales1 (2 KB)
//   box    = 128 rows x 128 bytes (256 E2M1 values of one K block), 16-byte pieces XOR-swizzled by
//            (row & 7): the 128-byte swizzle a TMA tile load would have produced
//   scales = the matching four 512-byte tiles of the 128x4-tiled E4M3 layout
//   g13: [entry][row tile of I][K block of H]    box0/1 = gate/up rows of the same K block
//   g2:  [entry][row tile of H][pair of K blocks] box0/1 = K blocks 2s, 2s+1 of the down matrix
constexpr int kChunkBytes = 36864;
constexpr int kChunkBox = 16384;
constexpr int kChunkScaleOffset = 32768;
constexpr int kChunkScaleBytes = 2048;

struct BankView {
    const std::uint8_t* g13;
    const std::uint8_t* g2;
    const float* alpha;         // [entries][3]
    int first_expert;
    int local_experts;
    int hidden;
    int intermediate;
};

// Routing products of one call, all in device memory owned by the plan.
// "Position" space: routed assignments sorted by expert (stable), followed by
// one row per token for the shared expert.
struct RouteView {
    const std::int32_t* counts;      // [257]  rows per entry (entry 256 = shared = rows)
    const std::int32_t* offsets;     // [258]  exclusive prefix in position space
    const std::int32_t* row_token;   // [9*rows] token of each position
    const std::int32_t* active;      // [257]  entries with rows, shared expert first
    const std::int32_t* active_count;
};

}  // namespace p92b

struct p92b_bank {
    p92b::BankView view {};
    void* storage = nullptr;
    std::size_t bytes = 0;
    bool tc_ready = true;       // the tiled stream is always built
};

struct p92b_plan {
    int max_rows = 0;
    int hidden = 0;
    int intermediate = 0;
    int sm_count = 0;
    int last_launches = 0;
    void* storage = nullptr;
    std::size_t bytes = 0;
    // device scratch (carved out of storage)
    float* logits = nullptr;              // [max_rows][256]
    std::int32_t* ids = nullptr;          // [max_rows][8]
    float* route_weights = nullptr;       // [max_rows][8]
    std::int32_t* order = nullptr;        // [8*max_rows]
    std::int32_t* position = nullptr;     // [8*max_rows]
    std::int32_t* counts = nullptr;       // [257]
    std::int32_t* offsets = nullptr;      // [258]
    std::int32_t* row_token = nullptr;    // [9*max_rows]
    std::int32_t* active = nullptr;       // [257]
    std::int32_t* active_count = nullptr; // [1]
    std::int32_t* pp_off = nullptr;       // [258] padded offsets (tensor-core path)
    std::int32_t* tile_prefix = nullptr;  // [258]
    std::int32_t* tile_prefix_wide = nullptr;   // [258] the same prefix for token tiles twice as wide (down product)
    int wide_rows = 0;                    // token tile tile_prefix_wide was last built for (0: not built)
    std::int32_t* pp_of_flat = nullptr;   // [9*max_rows] padded position of (row, slot), shared rows last
    std::int32_t* chunk_hist = nullptr;   // [chunks][256]
    unsigned* scan_blocks_done = nullptr; // [1] blocks of the permutation's scan kernel that have finished (zero between calls)
    int chunks = 0;
    std::uint8_t* xq = nullptr;           // [max_rows][H/2]
    std::uint8_t* xs = nullptr;           // [max_rows][H/16]
    std::uint16_t* stage_in = nullptr;    // [max_rows][H]  host-call staging
    std::uint16_t* stage_out = nullptr;   // [max_rows][H]
    // pipelined host calls: second pair of staging rows, copy streams and the events between the three streams
    std::uint16_t* stage_in_b = nullptr;
    std::uint16_t* stage_out_b = nullptr;
    cudaStream_t copy_in_stream = nullptr;
    cudaStream_t copy_out_stream = nullptr;
    cudaEvent_t in_ready[2] = {};
    cudaEvent_t block_done[2] = {};
    cudaEvent_t out_done[2] = {};
    unsigned host_calls = 0;
    std::int32_t* status = nullptr;       // [1]
    // tensor-core path: operands in the padded position space (every expert's rows start on a
    // multiple of 32 or 128), scales in the 128x4-tiled layout
    int last_path = 2;                    // path the last forward took
    int path = 0;                         // 0 auto, 2 tcgen05 kernels one launch per stage, 3 fused tcgen05 decode kernel
    bool tc_ready = false;
    std::size_t pp_rows = 0;              // rows of the padded buffers
    std::uint8_t* xq_pp = nullptr;        // [pp_rows][H/2]
    std::uint8_t* xs_sw = nullptr;        // tiled scales of xq_pp
    std::uint8_t* hq_pp = nullptr;        // [pp_rows][I/2]
    std::uint8_t* hs_sw = nullptr;        // tiled scales of hq_pp
    std::uint16_t* mixed_pp = nullptr;    // [pp_rows][H]
    CUtensorMap map_x[4] = {};            // token boxes of 16/32/64/128 rows over xq_pp
    CUtensorMap map_h[4] = {};            // same over hq_pp
    // fused decode kernel (rows <= 8)
    std::uint8_t* xq_tok = nullptr;       // [16][H/2] token-order NVFP4 rows
    std::uint8_t* xs_tok = nullptr;       // [H/64][512] their scales, one 128-row tile per 4 scale columns
    unsigned* mega_sync = nullptr;        // [2] arrival counters (monotonic across launches)
    std::int32_t* gu_done = nullptr;      // [2][264] per launch parity: gate/up tiles finished per active slot, [257] the tile counter
    std::int32_t* ep_gu_done = nullptr;   // [2][264] the same for the fused expert-parallel kernel
    unsigned long long* ep_logits = nullptr;    // [8][256] its router logits as tagged words
    unsigned long long* mega_logits = nullptr;  // [8][256] router logits as {value, launch number} words
    unsigned long long* mega_ret = nullptr;     // [8][9][1280] down rows as {two BF16, launch number} words
    float* w_norms = nullptr;                   // [2][256] norms of the router rows (tensor-core router), alternating by call
    int norms_parity = 0;
    float* logit_partials = nullptr;            // [kRouterSplits][min(max_rows, kRouterSplitRows)][256] partial logits of the K splits
    int* router_stats = nullptr;                // [2] large-batch router: logits recomputed exactly so far, tokens that took a whole row
    unsigned long long* mega_hidden = nullptr;  // [8][H/2] un-normalised output rows as tagged words (fused post-norm)
    std::uint16_t* normed = nullptr;            // [max_rows][H] pre-normalised rows of the multi-kernel path
    unsigned mega_epoch = 0;
    unsigned ep_epoch = 0;                // launches of the fused expert-parallel kernel (counters mega_sync[2..3])
    unsigned long long* mega_trace = nullptr;   // [sm_count][64] timer stamps of the last fused launch (P92B_TRACE=1)
    bool trace_on = false;
    CUtensorMap map_x_tok {};
    // expert-parallel scratch: per (source, local expert) padded base and arrival start
    std::int32_t* ep_src_base = nullptr;
    std::int32_t* ep_src_start = nullptr;
    std::int32_t* ep_zero_counts = nullptr;
    std::int32_t* epg_counts = nullptr;   // [257] histogram and [258] offsets of the whole gathered batch
    std::int32_t* epg_offsets = nullptr;
    int ep_words = 0;
    // optional stage timing (host side)
    bool timing = false;
    cudaEvent_t stage_events[P92B_STAGES + 1] = {};
    float stage_ms[P92B_STAGES] = {};
    int timed_calls = 0;
};

// Exchange memory of one GPU for the kernels that do their own expert-parallel exchanges
// (decode_ep.cu, ep_gathered.cu): this GPU's window plus the mapped windows of its peers.
struct p92b_ep_window {
    int rank = 0, world = 1, rows_per_gpu = 0;
    std::uint8_t* local = nullptr;
    std::uint8_t* peers[16] = {};
    bool opened[16] = {};
    bool connected = false;
    bool fused_ok = false;                // small enough for the single-kernel path
    bool bulk = false;                    // a window of the large-batch path (p92b_ep_window_create_bulk): its own layout
    int bulk_hidden = 0;
    unsigned epoch = 0;                   // calls so far (the same number on every GPU)
    std::size_t bytes = 0;
    std::size_t gathered_base = 0;        // offset of the regions of the multi-kernel gathered path
    CUtensorMap map_tok[2] = {};
};

namespace p92b {

// Launch with or without programmatic dependent launch: with `pdl` the kernel may start while the
// previous kernel in the stream is still draining, and must call ptx::pdl_wait() before it touches
// anything that kernel writes.
template <class... KArgs, class... Args>
cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, std::size_t smem, cudaStream_t stream,
                          bool pdl, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

// Opt-in to more than 48 KB of dynamic shared memory.  The attribute belongs to the (kernel, device)
// pair, not to the process: a host that drives several GPUs from one process has to set it once on
// each of them, so the "already done" flag is kept per device (one table per kernel through the
// non-type template parameter).
constexpr int kMaxDevices = 64;
template <auto Kernel>
cudaError_t ensure_dynamic_smem(int bytes) {
    static bool configured[kMaxDevices] = {};
    int device = 0;
    cudaError_t st = cudaGetDevice(&device);
    if (st != cudaSuccess) return st;
    const bool tracked = device >= 0 && device < kMaxDevices;
    if (tracked && configured[device]) return cudaSuccess;
    st = cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (st == cudaSuccess && tracked) configured[device] = true;
    return st;
}

// kernel launchers (defined across the .cu files)
cudaError_t launch_router_logits(const std::uint16_t* x, const std::uint16_t* w, float* out,
                                 int batch_rows, int rows, int columns, bool gemv_order,
                                 cudaStream_t stream, bool pdl = false);
cudaError_t launch_router_top8(const float* logits, const float* bias, std::int32_t* ids,
                               float* weights, int rows, float routed_scale, cudaStream_t stream,
                               bool pdl = false);
// range_count >= 0 restricts the permutation to expert ids [range_first, range_first + range_count): other ids
// (another GPU's experts, -1 for an empty token slot) are skipped and get position -1.  shared_rows >= 0 overrides
// the shared expert's row count in the lists (default: assignments / 8).
cudaError_t launch_permute(p92b_plan* plan, const std::int32_t* ids, int assignments,
                           std::int32_t* order, std::int32_t* position, std::int32_t* counts,
                           std::int32_t* offsets, bool route_lists, int pad_align, int tile_rows,
                           cudaStream_t stream, bool pdl = false, int range_first = 0, int range_count = -1,
                           int shared_rows = -1);
int route_fused_max_rows();
cudaError_t launch_route_fused(p92b_plan* plan, const float* bias, float routed_scale, const std::uint16_t* x,
                               int rows, int pad_align, int tile_rows, cudaStream_t stream, bool pdl);
cudaError_t launch_quantize(const std::uint16_t* input, std::uint8_t* output, std::uint8_t* scales,
                            long groups, float global_scale, cudaStream_t stream);
// Writes the matrices of one kind (0/1/2 = gate/up/down) of all `entries` of a table of reference-format
// projections (device copy, entry * 3 + kind) into the chunk stream, and their alpha values.
// blocks_per_chunk 1: gate (slot 0) or up (slot 1) of a K block; 2: K blocks 2s, 2s+1 of a down matrix.
cudaError_t launch_retile_table(const p92b_expert_projection* device_table, int entries, int kind, std::uint8_t* chunks,
                                std::size_t entry_bytes, int rows, int k_bytes, int blocks_per_chunk, int slot,
                                float* alpha, cudaStream_t stream);
cudaError_t launch_combine_shared(const std::uint16_t* mixed, const std::int32_t* mixed_index,
                                  const float* route_weights, std::uint16_t* output, int rows,
                                  int hidden, cudaStream_t stream, bool pdl = false);
cudaError_t launch_rmsnorm(const std::uint16_t* input, const std::uint16_t* weight, std::uint16_t* output, int rows,
                           int elements, int input_stride, int output_stride, float epsilon, cudaStream_t stream,
                           bool pdl = false);
// Large-batch router (router_tc.cu): tensor-core logits + exact repair -> plan->logits, ids, route_weights.
// cudaErrorNotSupported when the batch is too small or a pointer is not 16-byte aligned: take the exact kernels then.
int router_fast_min_rows();
constexpr int kRouterSplits = 8;                // K splits of the tensor-core logits for small batches
constexpr int kRouterSplitRows = 256;           // ... used up to this many rows
cudaError_t launch_router_fast(p92b_plan* plan, const std::uint16_t* x, const std::uint16_t* router_w, const float* bias,
                               int rows, float routed_scale, cudaStream_t stream, bool pdl);
// tensor-core path (expert_tc.cu)
cudaError_t make_operand_map(CUtensorMap* map, const void* base, std::size_t rows, std::size_t row_bytes,
                             int box_rows);
int tc_tile_rows(int rows);
int tc_pad_align(int rows);
cudaError_t launch_quantize_padded(const p92b_plan* plan, const std::uint16_t* x, int rows, cudaStream_t stream,
                                   bool pdl = false);
cudaError_t launch_quantize_rows_to_pp(const std::uint16_t* x, const std::int32_t* index, std::uint8_t* xq,
                                       std::uint8_t* xs, int n, int width, cudaStream_t stream, bool pdl = false);
// Optional redirections of the grouped kernels' outputs (null members: the plan's own buffers).
struct TcIo {
    std::uint16_t* down_out = nullptr;      // single-matrix products: BF16 rows written here instead of mixed_pp
    const std::int32_t* out_row = nullptr;  // [dense position] -> output row (null: rows sit at their padded position)
    std::uint16_t* gate_out = nullptr;      // both set: gate and up rows stored un-fused (no SwiGLU, no re-quantisation)
    std::uint16_t* up_out = nullptr;
    const p92b_expert_projection* table = nullptr;   // weights read in place from this device table (expert * 3 + kind)
    int table_kind = 0;                     // with `table`, single-matrix products: which of the three matrices
    bool single_matrix = false;             // with `table`, token-row side: one matrix (gate or up alone), rows to down_out
    bool skip_shared = false;               // the call has no shared expert
    bool wait_upstream = false;             // down product: the kernel just upstream may still be waiting for ITS predecessor
                                            // when this one starts, so the routing lists may only be read after a wait
    std::uint16_t* const* row_dest = nullptr;   // down product of large batches only (down_slab_applies): [padded position] ->
                                            // where that row's `hidden` BF16 values go, this GPU's memory or a peer's
};
// True when launch_experts_tc(..., down = true) with the lists last built for `rows` runs the slab kernel, the one
// that honours TcIo::row_dest.
bool down_slab_applies(const p92b_plan* plan, int rows);
cudaError_t launch_gather_quantized_rows(const std::uint8_t* packed, const std::uint8_t* scales_swizzled,
                                         const std::int32_t* pp_of_flat, std::uint8_t* xq, std::uint8_t* xs, int assignments,
                                         int k_bytes, bool distinct_rows, cudaStream_t stream, bool pdl = false);
cudaError_t launch_experts_tc(const p92b_plan* plan, const p92b_bank* bank, int rows, bool down,
                              cudaStream_t stream, bool pdl = false, const TcIo* io = nullptr);
// Routing lists of a call in which every row goes to the bank's last entry only (the dense MLP).
cudaError_t launch_dense_lists(p92b_plan* plan, int rows, int tile_rows, cudaStream_t stream, bool pdl = false);
// Pipelined host-buffer calls (moe_api.cu).  Three streams: the caller's (the block), one for rows coming in, one
// for rows going out; two sets of staging rows used alternately.  begin: the copy-in of this call is enqueued on
// the plan's in-stream (after the block of call n-2 has read the set) and `stream` is made to wait for it and for
// the copy-out of call n-2; the caller then enqueues its block from *rows_in to *rows_out on `stream`; end: the
// copy-out is enqueued on the plan's out-stream behind the block.
cudaError_t host_pipeline_begin(p92b_plan* plan, const std::uint16_t* pinned_input, int rows, cudaStream_t stream,
                                std::uint16_t** rows_in, std::uint16_t** rows_out, int* set);
cudaError_t host_pipeline_end(p92b_plan* plan, std::uint16_t* pinned_output, int rows, cudaStream_t stream, int set);
// fused decode kernel (decode_mega.cu)
int decode_mega_max_rows();
cudaError_t launch_decode_mega(p92b_plan* plan, const p92b_bank* bank, const std::uint16_t* x,
                               const std::uint16_t* router_w, const float* bias, std::uint16_t* out, int rows,
                               float routed_scale, cudaStream_t stream, bool pdl, const std::uint16_t* pre_norm_w = nullptr,
                               const std::uint16_t* post_norm_w = nullptr, float norm_eps = 0.0F);

}  // namespace p92b
