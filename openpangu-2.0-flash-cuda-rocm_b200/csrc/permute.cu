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

namespace p92b {
namespace {

constexpr int kChunk = 256;          // flat indices per warp in the multi-block path
constexpr int kWarps = 8;

// Counts the experts of one chunk into hist[256] (owned by the calling warp).
__device__ __forceinline__ void warp_histogram(const std::int32_t* __restrict__ ids, int begin, int end,
                                               std::int32_t* hist, std::int32_t* status) {
    const int lane = threadIdx.x & 31;
    for (int e = lane; e < kExperts; e += 32) hist[e] = 0;
    __syncwarp();
    for (int base = begin; base < end; base += 32) {
        const int i = base + lane;
        const bool valid = i < end;
        int e = valid ? ids[i] : -1;
        if (valid && (e < 0 || e >= kExperts)) {
            atomicCAS(status, kStatusOk, kStatusBadExpertId);
            e = e < 0 ? 0 : kExperts - 1;
        }
        const unsigned peers = __match_any_sync(0xffffffffU, e);
        if (valid && (peers & ((1U << lane) - 1U)) == 0U) hist[e] += __popc(peers);
        __syncwarp();
    }
}

// Scatters one chunk.  base[e] = first position of this chunk's rows of expert e;
// running[256] is warp-private scratch.
__device__ __forceinline__ void warp_scatter(const std::int32_t* __restrict__ ids, int begin, int end,
                                             const std::int32_t* base, std::int32_t* running,
                                             std::int32_t* __restrict__ order,
                                             std::int32_t* __restrict__ position,
                                             std::int32_t* __restrict__ row_token) {
    const int lane = threadIdx.x & 31;
    for (int e = lane; e < kExperts; e += 32) running[e] = base[e];
    __syncwarp();
    for (int step = begin; step < end; step += 32) {
        const int i = step + lane;
        const bool valid = i < end;
        int e = valid ? ids[i] : -1;
        if (valid) e = e < 0 ? 0 : (e >= kExperts ? kExperts - 1 : e);
        const unsigned peers = __match_any_sync(0xffffffffU, e);
        const int rank = __popc(peers & ((1U << lane) - 1U));
        int pos = 0;
        if (valid) {
            pos = running[e] + rank;
            if (order != nullptr) order[pos] = i;
            if (position != nullptr) position[i] = pos;
            if (row_token != nullptr) row_token[pos] = i / kTop;
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
// expert as entry 256 (rows = tokens, positions after the routed ones), and the
// compact list of entries that have rows, shared expert first (it is the largest
// group, so the persistent kernels start it first).
__device__ __forceinline__ void write_route_lists(int e, int count, int offset, int assignments, int rows,
                                                  std::int32_t* counts, std::int32_t* offsets,
                                                  std::int32_t* active, std::int32_t* active_count,
                                                  bool route_lists, std::int32_t* scan_scratch) {
    counts[e] = count;
    offsets[e] = offset;
    if (e == kExperts - 1) offsets[kExperts] = assignments;
    if (!route_lists) return;
    const int slot = block_exclusive_scan_256(count > 0 ? 1 : 0, scan_scratch);
    if (count > 0) active[1 + slot] = e;
    if (e == kExperts - 1) {
        counts[kExperts] = rows;
        offsets[kExperts + 1] = assignments + rows;
        active[0] = kExperts;
        *active_count = 1 + slot + (count > 0 ? 1 : 0);
    }
}

// ---- single-block path (assignments <= 8 * 1024) ---------------------------
__global__ void __launch_bounds__(256) permute_small_kernel(
    const std::int32_t* __restrict__ ids, int assignments, std::int32_t* order,
    std::int32_t* position, std::int32_t* counts, std::int32_t* offsets, std::int32_t* row_token,
    std::int32_t* active, std::int32_t* active_count, bool route_lists, std::int32_t* status) {
    __shared__ std::int32_t hist[kWarps][kExperts];
    __shared__ std::int32_t running[kWarps][kExperts];
    __shared__ std::int32_t scan_scratch[kWarps];
    const int warp = threadIdx.x >> 5;
    const int per_warp = ((assignments + kWarps - 1) / kWarps + 31) / 32 * 32;
    const int begin = min(assignments, warp * per_warp);
    const int end = min(assignments, begin + per_warp);
    warp_histogram(ids, begin, end, hist[warp], status);
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
    const int rows = assignments / kTop;
    write_route_lists(e, total, offset, assignments, rows, counts, offsets, active, active_count, route_lists,
                      scan_scratch);
    __syncthreads();
    warp_scatter(ids, begin, end, hist[warp], running[warp], order, position, row_token);
    if (row_token != nullptr) {
        for (int t = threadIdx.x; t < rows; t += blockDim.x) row_token[assignments + t] = t;
    }
}

// ---- multi-block path -------------------------------------------------------
__global__ void __launch_bounds__(256) permute_hist_kernel(const std::int32_t* __restrict__ ids,
                                                           int assignments,
                                                           std::int32_t* __restrict__ chunk_hist,
                                                           std::int32_t* status) {
    __shared__ std::int32_t hist[kWarps][kExperts];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int chunk = blockIdx.x * kWarps + warp;
    const int begin = min(assignments, chunk * kChunk);
    const int end = min(assignments, begin + kChunk);
    warp_histogram(ids, begin, end, hist[warp], status);
    if (begin < assignments) {
        for (int e = lane; e < kExperts; e += 32) chunk_hist[static_cast<std::size_t>(chunk) * kExperts + e] = hist[warp][e];
    }
}

__global__ void __launch_bounds__(256) permute_scan_kernel(std::int32_t* __restrict__ chunk_hist, int chunks,
                                                           int assignments, std::int32_t* counts,
                                                           std::int32_t* offsets, std::int32_t* active,
                                                           std::int32_t* active_count, bool route_lists) {
    __shared__ std::int32_t scan_scratch[kWarps];
    const int e = threadIdx.x;
    int total = 0;
#pragma unroll 8
    for (int c = 0; c < chunks; ++c) {
        const std::size_t at = static_cast<std::size_t>(c) * kExperts + e;
        const int v = chunk_hist[at];
        chunk_hist[at] = total;
        total += v;
    }
    const int offset = block_exclusive_scan_256(total, scan_scratch);
    write_route_lists(e, total, offset, assignments, assignments / kTop, counts, offsets, active, active_count,
                      route_lists, scan_scratch);
}

__global__ void __launch_bounds__(256) permute_scatter_kernel(
    const std::int32_t* __restrict__ ids, int assignments, const std::int32_t* __restrict__ chunk_hist,
    const std::int32_t* __restrict__ offsets, std::int32_t* order, std::int32_t* position,
    std::int32_t* row_token) {
    __shared__ std::int32_t base[kWarps][kExperts];
    __shared__ std::int32_t running[kWarps][kExperts];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int chunk = blockIdx.x * kWarps + warp;
    const int begin = min(assignments, chunk * kChunk);
    const int end = min(assignments, begin + kChunk);
    if (begin < assignments) {
        for (int e = lane; e < kExperts; e += 32) {
            base[warp][e] = offsets[e] + chunk_hist[static_cast<std::size_t>(chunk) * kExperts + e];
        }
    }
    __syncwarp();
    warp_scatter(ids, begin, end, base[warp], running[warp], order, position, row_token);
    if (row_token != nullptr) {
        const int rows = assignments / kTop;
        const int t = blockIdx.x * blockDim.x + threadIdx.x;
        if (t < rows) row_token[assignments + t] = t;
    }
}

}  // namespace

cudaError_t launch_permute(p92b_plan* plan, const std::int32_t* ids, int assignments,
                           std::int32_t* order, std::int32_t* position, std::int32_t* counts,
                           std::int32_t* offsets, bool route_lists, int first_expert,
                           int local_experts, cudaStream_t stream) {
    (void)first_expert;
    (void)local_experts;
    if (plan == nullptr || ids == nullptr || counts == nullptr || offsets == nullptr || assignments <= 0 ||
        assignments > plan->max_rows * kTop) {
        return cudaErrorInvalidValue;
    }
    std::int32_t* row_token = route_lists ? plan->row_token : nullptr;
    if (assignments <= kWarps * 1024) {
        permute_small_kernel<<<1, 256, 0, stream>>>(ids, assignments, order, position, counts, offsets, row_token,
                                                    plan->active, plan->active_count, route_lists, plan->status);
        plan->last_launches += 1;
        return cudaGetLastError();
    }
    const int chunks = (assignments + kChunk - 1) / kChunk;
    if (chunks > plan->chunks) return cudaErrorInvalidValue;
    const int blocks = (chunks + kWarps - 1) / kWarps;
    permute_hist_kernel<<<blocks, 256, 0, stream>>>(ids, assignments, plan->chunk_hist, plan->status);
    permute_scan_kernel<<<1, 256, 0, stream>>>(plan->chunk_hist, chunks, assignments, counts, offsets, plan->active,
                                               plan->active_count, route_lists);
    permute_scatter_kernel<<<blocks, 256, 0, stream>>>(ids, assignments, plan->chunk_hist, offsets, order, position,
                                                       row_token);
    plan->last_launches += 3;
    return cudaGetLastError();
}

}  // namespace p92b
