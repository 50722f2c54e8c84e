// Token histogram and permutation into expert-contiguous order.
//
// Result contract (bit-exact with the reference): position of assignment
// (row, slot) = #{assignments with a smaller expert id}
//             + #{assignments with the same id and a smaller flat index row*8+slot},
// i.e. a STABLE counting sort of the flat index by expert id.  That is the
// order the reference's ranking loop produces per projection kind
// (cuda/nvfp4_grouped.cu:117-132) and the order its host-scheduled path walks
// rows in (src/model.cpp:1528-1540).  No atomics touch the ordering, so the
// result is deterministic: each warp owns a contiguous chunk of flat indices,
// ranks inside a 32-wide step come from __match_any_sync + popcount of the
// lower lanes, and chunk bases come from an exclusive scan over (expert, chunk).
#include "p92b_common.cuh"
#include "tc_ptx.cuh"

#include <cstdio>

namespace p92b {

using ptx::pdl_launch_dependents;
using ptx::pdl_wait;

namespace {

constexpr int kChunk = 256;          // flat indices per warp in the multi-block path
constexpr int kWarps = 8;

// Which expert ids take part.  The whole range by default; an expert-parallel GPU that holds the ids of the whole
// batch restricts the permutation to its own experts [first, first + count) - ids outside (other GPUs' experts, and
// -1 for an empty token slot) are then skipped, not clamped: they get no position and are not counted.
struct IdRange {
    int first = 0;
    int count = kExperts;
    int restricted = 0;
};

// Counts the experts of one chunk into hist[256] (owned by the calling warp).
// `cached` (optional): the chunk's ids already in shared memory, cached[i - begin].
__device__ __forceinline__ void warp_histogram(const std::int32_t* __restrict__ ids, int begin, int end,
                                               std::int32_t* hist, std::int32_t* status,
                                               const std::int16_t* cached = nullptr, IdRange range = IdRange()) {
    const int lane = threadIdx.x & 31;
    for (int e = lane; e < kExperts; e += 32) hist[e] = 0;
    __syncwarp();
    for (int base = begin; base < end; base += 32) {
        const int i = base + lane;
        bool valid = i < end;
        int e = valid ? (cached != nullptr ? static_cast<int>(cached[i - begin]) : ids[i]) : -1;
        if (range.restricted && (e < range.first || e >= range.first + range.count)) {
            valid = false;
            e = -1;
        }
        if (valid && (e < 0 || e >= kExperts)) {
            atomicCAS(status, kStatusOk, kStatusBadExpertId);
            e = e < 0 ? 0 : kExperts - 1;
        }
        const unsigned peers = __match_any_sync(0xffffffffU, e);
        if (valid && (peers & ((1U << lane) - 1U)) == 0U) hist[e] += __popc(peers);
        __syncwarp();
    }
}

// A warp's ids once into shared memory, all loads in flight together, clamped to -1 .. 256 so that they fit 16 bits
// and an id out of range stays out of range.
__device__ __forceinline__ void load_chunk_ids(const std::int32_t* __restrict__ ids, int begin, int end,
                                               std::int16_t* cached) {
    for (int i = begin + (threadIdx.x & 31); i < end; i += 32) {
        const int e = ids[i];
        cached[i - begin] = static_cast<std::int16_t>(e < -1 ? -1 : (e > kExperts ? kExperts : e));
    }
    __syncwarp();
}

// Scatters one chunk.  base[e] = first position of this chunk's rows of expert e; running[256] is warp-private
// scratch; pp_delta[e] (shared memory, read only with pp_of_flat) = padded offset - offset of expert e.  The steps
// of a chunk depend on one another through running[], so whatever a step reads has to be in shared memory or in
// registers already: a global load per step is a round trip to the L2 per step.
__device__ __forceinline__ void warp_scatter(const std::int32_t* __restrict__ ids, int begin, int end,
                                             const std::int32_t* base, std::int32_t* running,
                                             std::int32_t* __restrict__ order,
                                             std::int32_t* __restrict__ position,
                                             std::int32_t* __restrict__ row_token,
                                             const std::int32_t* pp_delta,
                                             std::int32_t* __restrict__ pp_of_flat,
                                             const std::int16_t* cached = nullptr, IdRange range = IdRange()) {
    const int lane = threadIdx.x & 31;
    for (int e = lane; e < kExperts; e += 32) running[e] = base[e];
    __syncwarp();
    for (int step = begin; step < end; step += 32) {
        const int i = step + lane;
        bool valid = i < end;
        int e = valid ? (cached != nullptr ? static_cast<int>(cached[i - begin]) : ids[i]) : -1;
        if (range.restricted && (e < range.first || e >= range.first + range.count)) {
            if (valid) {                      // skipped: no position
                if (position != nullptr) position[i] = -1;
                if (pp_of_flat != nullptr) pp_of_flat[i] = -1;
            }
            valid = false;
            e = -1;
        }
        if (valid) e = e < 0 ? 0 : (e >= kExperts ? kExperts - 1 : e);
        const unsigned peers = __match_any_sync(0xffffffffU, e);
        const int rank = __popc(peers & ((1U << lane) - 1U));
        int pos = 0;
        if (valid) {
            pos = running[e] + rank;
            if (order != nullptr) order[pos] = i;
            if (position != nullptr) position[i] = pos;
            if (row_token != nullptr) row_token[pos] = i / kTop;
            if (pp_of_flat != nullptr) pp_of_flat[i] = pp_delta[e] + pos;
        }
        __syncwarp();
        if (valid && rank == 0) running[e] += __popc(peers);
        __syncwarp();
    }
}

// Exclusive scan of 256 per-expert totals by one 256-thread block.
__device__ __forceinline__ int block_exclusive_scan_256(int value, std::int32_t* warp_totals) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    int inclusive = value;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
        const int other = __shfl_up_sync(0xffffffffU, inclusive, offset);
        if (lane >= offset) inclusive += other;
    }
    if (lane == 31) warp_totals[warp] = inclusive;
    __syncthreads();
    int before = 0;
    for (int wi = 0; wi < warp; ++wi) before += warp_totals[wi];
    __syncthreads();
    return before + inclusive - value;
}

// Lists written for the expert kernels: counts/offsets extended with the shared
// expert as entry 256 (rows = tokens, positions after the routed ones), the
// compact list of entries that have rows, shared expert first (it is the largest
// group, so the persistent kernels start it first), and - for the tensor-core
// kernels - a padded position space in which every entry's rows start on a
// multiple of `pad_align`, plus the prefix of token-tile counts over the active list.
struct RouteLists {
    std::int32_t* counts;        // [257]
    std::int32_t* offsets;       // [258]
    std::int32_t* active;        // [257]
    std::int32_t* active_count;  // [1]
    std::int32_t* pp_off;        // [258] padded offsets (null: not wanted)
    std::int32_t* tile_prefix;   // [258] exclusive prefix of token tiles over the active list, total last
    std::int32_t* tile_prefix_wide;   // the same for tiles of tile_rows_wide rows (null: not wanted)
    int pad_align;
    int tile_rows;
    int tile_rows_wide;
    bool enabled;
};

__device__ __forceinline__ void write_route_lists(int e, int count, int offset, int assignments, int rows,
                                                  const RouteLists& lists, std::int32_t* scan_scratch) {
    lists.counts[e] = count;
    lists.offsets[e] = offset;
    if (e == kExperts - 1) lists.offsets[kExperts] = assignments;
    if (!lists.enabled) return;
    const int slot = block_exclusive_scan_256(count > 0 ? 1 : 0, scan_scratch);
    if (count > 0) lists.active[1 + slot] = e;
    if (e == kExperts - 1) {
        lists.counts[kExperts] = rows;
        lists.offsets[kExperts + 1] = assignments + rows;
        lists.active[0] = kExperts;
        *lists.active_count = 1 + slot + (count > 0 ? 1 : 0);
    }
    if (lists.pp_off == nullptr) return;
    const int align = lists.pad_align;
    const int padded = (count + align - 1) / align * align;
    const int pp = block_exclusive_scan_256(padded, scan_scratch);
    lists.pp_off[e] = pp;
    const int tiles = (count + lists.tile_rows - 1) / lists.tile_rows;
    const int shared_tiles = (rows + lists.tile_rows - 1) / lists.tile_rows;
    const int before = block_exclusive_scan_256(tiles, scan_scratch);
    if (count > 0) lists.tile_prefix[1 + slot] = shared_tiles + before;
    if (e == kExperts - 1) {
        lists.pp_off[kExperts] = pp + padded;
        lists.pp_off[kExperts + 1] = pp + padded + (rows + align - 1) / align * align;
        lists.tile_prefix[0] = 0;
        lists.tile_prefix[1 + slot + (count > 0 ? 1 : 0)] = shared_tiles + before + tiles;   // total, after the last active
    }
    if (lists.tile_prefix_wide == nullptr) return;
    const int wide = lists.tile_rows_wide;
    const int tiles_w = (count + wide - 1) / wide;
    const int shared_w = (rows + wide - 1) / wide;
    const int before_w = block_exclusive_scan_256(tiles_w, scan_scratch);
    if (count > 0) lists.tile_prefix_wide[1 + slot] = shared_w + before_w;
    if (e == kExperts - 1) {
        lists.tile_prefix_wide[0] = 0;
        lists.tile_prefix_wide[1 + slot + (count > 0 ? 1 : 0)] = shared_w + before_w + tiles_w;
    }
}

// ---- single-block path (assignments <= 8 * 1024) ---------------------------
__global__ void __launch_bounds__(256) permute_small_kernel(
    const std::int32_t* __restrict__ ids, int assignments, std::int32_t* order,
    std::int32_t* position, RouteLists lists, std::int32_t* row_token, std::int32_t* pp_of_flat,
    std::int32_t* status, IdRange range, int shared_rows) {
    __shared__ std::int32_t hist[kWarps][kExperts];
    __shared__ std::int32_t running[kWarps][kExperts];
    __shared__ std::int32_t scan_scratch[kWarps];
    __shared__ std::int32_t pp_delta[kExperts];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5;
    const int per_warp = ((assignments + kWarps - 1) / kWarps + 31) / 32 * 32;
    const int begin = min(assignments, warp * per_warp);
    const int end = min(assignments, begin + per_warp);
    // the warp's ids once into shared memory, all loads in flight together: the two passes below are chains of
    // dependent 32-wide steps and would otherwise pay a global-memory round trip per step
    __shared__ std::int16_t cached_ids[kWarps][1024];
    load_chunk_ids(ids, begin, end, cached_ids[warp]);
    warp_histogram(ids, begin, end, hist[warp], status, cached_ids[warp], range);
    __syncthreads();
    const int e = threadIdx.x;
    int total = 0;
#pragma unroll
    for (int wi = 0; wi < kWarps; ++wi) {
        const int c = hist[wi][e];
        hist[wi][e] = total;      // exclusive prefix over chunks
        total += c;
    }
    const int offset = block_exclusive_scan_256(total, scan_scratch);
#pragma unroll
    for (int wi = 0; wi < kWarps; ++wi) hist[wi][e] += offset;
    const int rows = shared_rows >= 0 ? shared_rows : assignments / kTop;
    write_route_lists(e, total, offset, assignments, rows, lists, scan_scratch);
    pp_delta[e] = (pp_of_flat != nullptr && lists.pp_off != nullptr) ? lists.pp_off[e] - offset : 0;       // write_route_lists stored both just above
    __syncthreads();
    warp_scatter(ids, begin, end, hist[warp], running[warp], order, position, row_token, pp_delta, pp_of_flat,
                 cached_ids[warp], range);
    if (row_token != nullptr) {
        for (int t = threadIdx.x; t < rows; t += blockDim.x) {
            row_token[assignments + t] = t;
            if (pp_of_flat != nullptr) pp_of_flat[assignments + t] = lists.pp_off[kExperts] + t;
        }
    }
}

// ---- multi-block path -------------------------------------------------------
__global__ void __launch_bounds__(256) permute_hist_kernel(const std::int32_t* __restrict__ ids,
                                                           int assignments,
                                                           std::int32_t* __restrict__ chunk_hist,
                                                           std::int32_t* status, IdRange range) {
    __shared__ std::int32_t hist[kWarps][kExperts];
    __shared__ std::int16_t cached_ids[kWarps][kChunk];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int chunk = blockIdx.x * kWarps + warp;
    const int begin = min(assignments, chunk * kChunk);
    const int end = min(assignments, begin + kChunk);
    load_chunk_ids(ids, begin, end, cached_ids[warp]);
    warp_histogram(ids, begin, end, hist[warp], status, cached_ids[warp], range);
    if (begin < assignments) {
        for (int e = lane; e < kExperts; e += 32) chunk_hist[static_cast<std::size_t>(chunk) * kExperts + e] = hist[warp][e];
    }
}

// Exclusive prefix over the chunks, per expert, then the lists.  gridDim.x blocks of 1024 threads share the experts
// (256 / gridDim.x each); an expert has 1024 / that many threads, each owning a slice of the chunks: a sum pass, the
// slice bases through shared memory, then the pass that writes the prefixes.  The block that finishes last (a counter,
// reset by that block for the next call) adds the scan over the 256 expert totals and writes the lists.  One thread
// per expert walking 512 chunks took 60 µs at 131,072 assignments, one block with four threads per expert 22 µs.
constexpr int kScanThreads = 1024;
constexpr int kScanBlocksLarge = 8;
__global__ void __launch_bounds__(kScanThreads) permute_scan_kernel(std::int32_t* __restrict__ chunk_hist, int chunks,
                                                                    int assignments, RouteLists lists, int shared_rows,
                                                                    unsigned* __restrict__ blocks_done) {
    __shared__ std::int32_t scan_scratch[kWarps];
    __shared__ std::int32_t segment_total[kScanThreads];
    __shared__ int is_last;
    pdl_launch_dependents();
    pdl_wait();
    const int experts_here = kExperts / static_cast<int>(gridDim.x);          // 256 or 32
    const int segments = kScanThreads / experts_here;                        // 4 or 32
    const int e_local = threadIdx.x % experts_here;
    const int segment = threadIdx.x / experts_here;
    const int e = static_cast<int>(blockIdx.x) * experts_here + e_local;
    const int per_segment = (chunks + segments - 1) / segments;
    const int first = min(chunks, segment * per_segment);
    const int last = min(chunks, first + per_segment);
    int sum = 0;
#pragma unroll 16
    for (int c = first; c < last; ++c) sum += chunk_hist[static_cast<std::size_t>(c) * kExperts + e];
    segment_total[segment * experts_here + e_local] = sum;
    __syncthreads();
    int running = 0, total = 0;
    for (int s = 0; s < segments; ++s) {
        const int v = segment_total[s * experts_here + e_local];
        if (s < segment) running += v;
        total += v;
    }
#pragma unroll 16
    for (int c = first; c < last; ++c) {
        const std::size_t at = static_cast<std::size_t>(c) * kExperts + e;
        const int v = chunk_hist[at];
        chunk_hist[at] = running;
        running += v;
    }
    if (segment == 0) lists.counts[e] = total;
    // the last block to get here sees every block's totals
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned before = atomicAdd(blocks_done, 1U);
        is_last = before + 1U == gridDim.x ? 1 : 0;
        if (is_last) *blocks_done = 0U;
    }
    __syncthreads();
    if (!is_last || threadIdx.x >= kExperts) return;   // whole warps leave; the block-wide barriers below count the rest
    __threadfence();
    const int expert = threadIdx.x;
    const int expert_total = __ldcg(lists.counts + expert);
    const int offset = block_exclusive_scan_256(expert_total, scan_scratch);
    write_route_lists(expert, expert_total, offset, assignments, shared_rows >= 0 ? shared_rows : assignments / kTop, lists,
                      scan_scratch);
}

__global__ void __launch_bounds__(256) permute_scatter_kernel(
    const std::int32_t* __restrict__ ids, int assignments, const std::int32_t* __restrict__ chunk_hist,
    const std::int32_t* __restrict__ offsets, std::int32_t* order, std::int32_t* position,
    std::int32_t* row_token, const std::int32_t* __restrict__ pp_off, std::int32_t* pp_of_flat, IdRange range,
    int shared_rows) {
    __shared__ std::int32_t base[kWarps][kExperts];
    __shared__ std::int32_t running[kWarps][kExperts];
    __shared__ std::int32_t pp_delta[kExperts];
    __shared__ std::int16_t cached_ids[kWarps][kChunk];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int chunk = blockIdx.x * kWarps + warp;
    const int begin = min(assignments, chunk * kChunk);
    const int end = min(assignments, begin + kChunk);
    load_chunk_ids(ids, begin, end, cached_ids[warp]);
    pp_delta[threadIdx.x] = pp_of_flat != nullptr ? pp_off[threadIdx.x] - offsets[threadIdx.x] : 0;
    if (begin < assignments) {
        for (int e = lane; e < kExperts; e += 32) {
            base[warp][e] = offsets[e] + chunk_hist[static_cast<std::size_t>(chunk) * kExperts + e];
        }
    }
    __syncthreads();
    warp_scatter(ids, begin, end, base[warp], running[warp], order, position, row_token, pp_delta, pp_of_flat,
                 cached_ids[warp], range);
    if (row_token != nullptr) {
        const int rows = shared_rows >= 0 ? shared_rows : assignments / kTop;
        const int t = blockIdx.x * blockDim.x + threadIdx.x;
        if (t < rows) {
            row_token[assignments + t] = t;
            if (pp_of_flat != nullptr) pp_of_flat[assignments + t] = pp_off[kExperts] + t;
        }
    }
}

// ---- decode front end: top-8 + permutation + lists + NVFP4 token rows, one block ------------
// For up to 8 tokens the three routing stages are a few microseconds of work each, so they run as
// one 256-thread block instead of three launches: warp w ranks token w; thread e counts expert e
// (the ranking law of cuda/nvfp4_grouped.cu:117-132 evaluated directly: 64 assignments at most);
// then every thread quantises 16-element blocks of the token rows (cuda/nvfp4_ops.cu:818-841) and
// stores them once per destination row of the padded position space, scales in the 128x4 tiling.
constexpr int kFusedMaxRows = 8;

__global__ void __launch_bounds__(256) route_fused_kernel(
    const float* __restrict__ logits, const float* __restrict__ bias, std::int32_t* __restrict__ ids,
    float* __restrict__ weights, float routed_scale, int rows, std::int32_t* __restrict__ order,
    std::int32_t* __restrict__ position, RouteLists lists, std::int32_t* __restrict__ row_token,
    std::int32_t* __restrict__ pp_of_flat, const std::uint16_t* __restrict__ x, std::uint8_t* __restrict__ xq,
    std::uint8_t* __restrict__ xs, int hidden, float quant_scale) {
    __shared__ std::int32_t s_ids[kFusedMaxRows * kTop];
    __shared__ std::int32_t s_pp[kFusedMaxRows * (kTop + 1)];
    __shared__ std::int32_t scan_scratch[kWarps];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5;
    const int assignments = rows * kTop;
    if (warp < rows) {
        warp_top8(logits + static_cast<std::size_t>(warp) * kExperts, bias, ids + warp * kTop, weights + warp * kTop,
                  routed_scale);
    }
    __syncthreads();
    if (threadIdx.x < assignments) s_ids[threadIdx.x] = ids[threadIdx.x];
    __syncthreads();
    const int e = threadIdx.x;
    int count = 0;
    for (int j = 0; j < assignments; ++j) count += s_ids[j] == e;
    const int offset = block_exclusive_scan_256(count, scan_scratch);
    write_route_lists(e, count, offset, assignments, rows, lists, scan_scratch);
    __syncthreads();
    if (threadIdx.x < assignments) {
        const int i = threadIdx.x;
        const int mine = s_ids[i];
        int rank = 0;
        for (int j = 0; j < i; ++j) rank += s_ids[j] == mine;
        const int pos = lists.offsets[mine] + rank;
        order[pos] = i;
        position[i] = pos;
        row_token[pos] = i / kTop;
        const int pp = lists.pp_off[mine] + rank;
        pp_of_flat[i] = pp;
        s_pp[i] = pp;
    } else if (threadIdx.x < assignments + rows) {
        const int t = threadIdx.x - assignments;
        row_token[assignments + t] = t;
        const int pp = lists.pp_off[kExperts] + t;
        pp_of_flat[assignments + t] = pp;
        s_pp[assignments + t] = pp;
    }
    __syncthreads();
    const int blocks = hidden / 16;
    const int col_blocks = (blocks + 3) / 4;
    for (int idx = threadIdx.x; idx < rows * blocks; idx += blockDim.x) {
        const int token = idx / blocks;
        const int b = idx - token * blocks;
        const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<std::size_t>(token) * hidden + b * 16);
        const uint4 lo = __ldg(src);
        const uint4 hi = __ldg(src + 1);
        const std::uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        float v[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[2 * i] = __uint_as_float(words[i] << 16);
            v[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000U);
        }
        std::uint8_t scale_bits;
        const uint2 packed = quantize_block16(v, quant_scale, &scale_bits);
#pragma unroll
        for (int slot = 0; slot <= kTop; ++slot) {
            const std::size_t pp =
                static_cast<std::size_t>(s_pp[slot < kTop ? token * kTop + slot : assignments + token]);
            *reinterpret_cast<uint2*>(xq + pp * (hidden / 2) + b * 8) = packed;
            xs[((pp >> 7) * col_blocks + (b >> 2)) * 512 + (pp & 31) * 16 + ((pp >> 5) & 3) * 4 + (b & 3)] = scale_bits;
        }
    }
}

// Lists for a call without routing: all `rows` rows belong to entry 256 (the bank's last entry), which starts at
// padded position 0; no routed expert has rows.
__global__ void __launch_bounds__(256) dense_lists_kernel(RouteLists lists, int rows) {
    pdl_launch_dependents();
    pdl_wait();
    const int e = threadIdx.x;
    lists.counts[e] = 0;
    lists.offsets[e] = 0;
    lists.pp_off[e] = 0;
    if (e == 0) {
        lists.counts[kExperts] = rows;
        lists.offsets[kExperts] = 0;
        lists.offsets[kExperts + 1] = rows;
        lists.active[0] = kExperts;
        *lists.active_count = 1;
        lists.pp_off[kExperts] = 0;
        lists.pp_off[kExperts + 1] = (rows + lists.pad_align - 1) / lists.pad_align * lists.pad_align;
        lists.tile_prefix[0] = 0;
        lists.tile_prefix[1] = (rows + lists.tile_rows - 1) / lists.tile_rows;
        if (lists.tile_prefix_wide != nullptr) {
            lists.tile_prefix_wide[0] = 0;
            lists.tile_prefix_wide[1] = (rows + lists.tile_rows_wide - 1) / lists.tile_rows_wide;
        }
    }
}

}  // namespace

int route_fused_max_rows() { return kFusedMaxRows; }

cudaError_t launch_dense_lists(p92b_plan* plan, int rows, int tile_rows, cudaStream_t stream, bool pdl) {
    RouteLists lists {};
    lists.counts = plan->counts;
    lists.offsets = plan->offsets;
    lists.active = plan->active;
    lists.active_count = plan->active_count;
    lists.enabled = true;
    lists.pad_align = 128;
    lists.tile_rows = tile_rows;
    lists.pp_off = plan->pp_off;
    lists.tile_prefix = plan->tile_prefix;
    const bool wide = tile_rows == 64;
    lists.tile_rows_wide = wide ? 128 : tile_rows;
    lists.tile_prefix_wide = wide ? plan->tile_prefix_wide : nullptr;
    plan->wide_rows = wide ? 128 : 0;
    plan->last_launches += 1;
    return launch_kernel(dense_lists_kernel, dim3(1), dim3(256), 0, stream, pdl, lists, rows);
}

cudaError_t launch_route_fused(p92b_plan* plan, const float* bias, float routed_scale, const std::uint16_t* x,
                               int rows, int pad_align, int tile_rows, cudaStream_t stream, bool pdl) {
    if (rows <= 0 || rows > kFusedMaxRows) return cudaErrorInvalidValue;
    RouteLists lists {};
    lists.counts = plan->counts;
    lists.offsets = plan->offsets;
    lists.active = plan->active;
    lists.active_count = plan->active_count;
    lists.enabled = true;
    lists.pad_align = pad_align;
    lists.tile_rows = tile_rows;
    lists.pp_off = plan->pp_off;
    lists.tile_prefix = plan->tile_prefix;
    lists.tile_rows_wide = tile_rows;
    lists.tile_prefix_wide = nullptr;
    plan->wide_rows = 0;
    plan->last_launches += 1;
    return launch_kernel(route_fused_kernel, dim3(1), dim3(256), 0, stream, pdl, plan->logits, bias, plan->ids,
                         plan->route_weights, routed_scale, rows, plan->order, plan->position, lists, plan->row_token,
                         plan->pp_of_flat, x, plan->xq_pp, plan->xs_sw, plan->hidden, 1.0F);
}

cudaError_t launch_permute(p92b_plan* plan, const std::int32_t* ids, int assignments,
                           std::int32_t* order, std::int32_t* position, std::int32_t* counts,
                           std::int32_t* offsets, bool route_lists, int pad_align, int tile_rows,
                           cudaStream_t stream, bool pdl, int range_first, int range_count, int shared_rows) {
    IdRange range;
    if (range_count >= 0) {
        range.first = range_first;
        range.count = range_count;
        range.restricted = 1;
    }
    if (plan == nullptr || ids == nullptr || counts == nullptr || offsets == nullptr || assignments <= 0 ||
        assignments > plan->max_rows * kTop) {
        return cudaErrorInvalidValue;
    }
    RouteLists lists {};
    lists.counts = counts;
    lists.offsets = offsets;
    lists.active = plan->active;
    lists.active_count = plan->active_count;
    lists.enabled = route_lists;
    lists.pad_align = pad_align > 0 ? pad_align : 1;
    lists.tile_rows = tile_rows > 0 ? tile_rows : 1;
    const bool padded = route_lists && pad_align > 0;
    lists.pp_off = padded ? plan->pp_off : nullptr;
    lists.tile_prefix = padded ? plan->tile_prefix : nullptr;
    // large batches: the down product takes token tiles twice as wide as the gate/up product (one
    // accumulator per tile instead of two, so 128 columns still leave room for two buffers)
    const bool wide = padded && tile_rows == 64;
    lists.tile_rows_wide = wide ? 128 : lists.tile_rows;
    lists.tile_prefix_wide = wide ? plan->tile_prefix_wide : nullptr;
    plan->wide_rows = wide ? 128 : 0;
    std::int32_t* row_token = route_lists ? plan->row_token : nullptr;
    std::int32_t* pp_of_flat = padded ? plan->pp_of_flat : nullptr;
    // one block takes up to 8,192 assignments, but from 4,097 on the three-kernel form is quicker (33 against 22 µs at 8,192)
    if (assignments <= 4096) {
        plan->last_launches += 1;
        return launch_kernel(permute_small_kernel, dim3(1), dim3(256), 0, stream, pdl, ids, assignments, order, position,
                             lists, row_token, pp_of_flat, plan->status, range, shared_rows);
    }
    const int chunks = (assignments + kChunk - 1) / kChunk;
    if (chunks > plan->chunks) return cudaErrorInvalidValue;
    const int blocks = (chunks + kWarps - 1) / kWarps;
    plan->last_launches += 3;
    cudaError_t st = launch_kernel(permute_hist_kernel, dim3(blocks), dim3(256), 0, stream, pdl, ids, assignments,
                                   plan->chunk_hist, plan->status, range);
    if (st != cudaSuccess) return st;
    st = launch_kernel(permute_scan_kernel, dim3(chunks >= 64 ? kScanBlocksLarge : 1), dim3(kScanThreads), 0, stream, pdl,
                       plan->chunk_hist, chunks, assignments, lists, shared_rows, plan->scan_blocks_done);
    if (st != cudaSuccess) return st;
    return launch_kernel(permute_scatter_kernel, dim3(blocks), dim3(256), 0, stream, pdl,
                         static_cast<const std::int32_t*>(ids), assignments,
                         static_cast<const std::int32_t*>(plan->chunk_hist), static_cast<const std::int32_t*>(offsets),
                         order, position, row_token, static_cast<const std::int32_t*>(lists.pp_off), pp_of_flat, range,
                         shared_rows);
}

}  // namespace p92b

// ---------------------------------------------------------------------------
// Allocation-free permutation (p92b_moe_permute_static).
//
// For callers that cannot give the library a plan because they cannot allocate:
// the engine has already committed all device memory to its own arena, the host
// process forbids further CUDA allocations, or the call sits in a loop that must
// not run into the device-wide synchronisation cudaMalloc / cudaFree may cause.
// The scratch of the multi-block permutation lives in this file-scope device
// array instead.  Every GPU that loads the library carries its copy of the array
// (P92B_STATIC_PERMUTE_SCRATCH_BYTES) until the process exits.
//
// In host code the array's name is only a stand-in for the symbol, not a device
// address, so the address is fetched once per device with cudaGetSymbolAddress
// (that device current) and handed to the kernels as an ordinary pointer.
// Layout: [chunks][256] int32 chunk histograms, then the status word and the scan kernel's block counter.
//
// The address cache below is filled on first use per device.  Two host threads that make their
// first call on the same device at the same time both look the address up and both store the
// same value: harmless, but the kernels of their calls would still share the one array, so such
// calls have to be serialised by the caller for that reason anyway.
// ---------------------------------------------------------------------------
namespace {

constexpr int kStaticMaxAssignments = P92B_STATIC_PERMUTE_MAX_ASSIGNMENTS;
constexpr int kStaticChunks = kStaticMaxAssignments / p92b::kChunk;
constexpr int kStaticWords = kStaticChunks * p92b::kExperts + 64;
static_assert(kStaticWords * 4 == P92B_STATIC_PERMUTE_SCRATCH_BYTES, "header and array disagree");
constexpr int kStaticMaxDevices = 64;

static __device__ __align__(256) std::int32_t g_static_permute_scratch[kStaticWords];

std::int32_t* g_static_scratch_address[kStaticMaxDevices] = {};

// Device address of the array on the current device; looked up on first use.
cudaError_t static_scratch(std::int32_t** out) {
    int device = 0;
    cudaError_t st = cudaGetDevice(&device);
    if (st != cudaSuccess) return st;
    if (device < 0 || device >= kStaticMaxDevices) return cudaErrorNotSupported;
    if (g_static_scratch_address[device] == nullptr) {
        void* address = nullptr;
        st = cudaGetSymbolAddress(&address, g_static_permute_scratch);
        if (st != cudaSuccess) return st;
        g_static_scratch_address[device] = static_cast<std::int32_t*>(address);
    }
    *out = g_static_scratch_address[device];
    return cudaSuccess;
}

}  // namespace

extern "C" int p92b_moe_permute_static(const int32_t* expert_ids, int assignments, int32_t* order,
                                       int32_t* position, int32_t* counts, int32_t* offsets, void* stream_) {
    using namespace p92b;
    if (expert_ids == nullptr || counts == nullptr || offsets == nullptr || assignments <= 0) {
        return cudaErrorInvalidValue;
    }
    if (assignments > kStaticMaxAssignments) {
        std::fprintf(stderr,
                     "p92b_moe_permute_static: %d assignments exceed the built-in scratch (limit %d = %d rows x 8); "
                     "use p92b_moe_permute with a plan\n",
                     assignments, kStaticMaxAssignments, kStaticMaxAssignments / kTop);
        return cudaErrorInvalidValue;
    }
    std::int32_t* scratch = nullptr;
    cudaError_t st = static_scratch(&scratch);
    if (st != cudaSuccess) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    std::int32_t* chunk_hist = scratch;
    std::int32_t* status = scratch + kStaticChunks * kExperts;
    // the array still holds the previous call's words: the status word and the block counter must start at zero,
    // the histograms are fully rewritten by permute_hist_kernel before anything reads them
    st = cudaMemsetAsync(status, 0, 2 * sizeof(std::int32_t), stream);       // the status word and the scan's block counter
    if (st != cudaSuccess) return st;
    RouteLists lists {};
    lists.counts = counts;
    lists.offsets = offsets;
    lists.enabled = false;
    lists.pad_align = 1;
    lists.tile_rows = 1;
    lists.tile_rows_wide = 1;
    lists.tile_prefix_wide = nullptr;
    if (assignments <= kWarps * 1024) {
        permute_small_kernel<<<1, 256, 0, stream>>>(expert_ids, assignments, order, position, lists, nullptr, nullptr,
                                                    status, IdRange(), -1);
        return cudaGetLastError();
    }
    const int chunks = (assignments + kChunk - 1) / kChunk;
    const int blocks = (chunks + kWarps - 1) / kWarps;
    permute_hist_kernel<<<blocks, 256, 0, stream>>>(expert_ids, assignments, chunk_hist, status, IdRange());
    permute_scan_kernel<<<chunks >= 64 ? p92b::kScanBlocksLarge : 1, p92b::kScanThreads, 0, stream>>>(
        chunk_hist, chunks, assignments, lists, -1, reinterpret_cast<unsigned*>(status + 1));
    permute_scatter_kernel<<<blocks, 256, 0, stream>>>(expert_ids, assignments, chunk_hist, offsets, order, position,
                                                       nullptr, nullptr, nullptr, IdRange(), -1);
    return cudaGetLastError();
}

// The status word of the calls above lives in the same built-in array, where a caller cannot
// reach it; this copies it out.  Like the permutation itself it allocates nothing: one
// cudaMemcpyAsync into the caller's host word, then a synchronisation of `stream`.
extern "C" int p92b_moe_permute_static_status(int32_t* host_status, void* stream_) {
    using namespace p92b;
    if (host_status == nullptr) return cudaErrorInvalidValue;
    std::int32_t* scratch = nullptr;
    cudaError_t st = static_scratch(&scratch);
    if (st != cudaSuccess) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    st = cudaMemcpyAsync(host_status, scratch + kStaticChunks * kExperts, sizeof(std::int32_t), cudaMemcpyDeviceToHost,
                         stream);
    if (st != cudaSuccess) return st;
    return cudaStreamSynchronize(stream);
}
