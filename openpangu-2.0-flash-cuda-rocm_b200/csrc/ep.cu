// Expert-parallel split of the block: the pieces either side of the two all-to-all exchanges.
//
// 256 routed experts are sharded contiguously over G GPUs (128/64/32 per GPU); router and shared
// expert are replicated; every GPU is home to its own tokens.  Per layer:
//   home:    route (logits, top-8, stable permutation by expert id) -> since expert ranges per GPU
//            are contiguous, the permuted order is already grouped by destination GPU; the
//            quantised rows (1280 B E2M1 + 160 B E4M3 scales) are packed in that order
//            [exchange 1: rows + per-expert counts]
//   owner:   rows of one expert arrive as G runs (one per source, each in source order); placing
//            source s's run after the runs of sources < s reproduces the GLOBAL stable order
//            restricted to this GPU's experts, i.e. the same permutation a single GPU computes.
//            Rows go into the padded position space, the tensor-core expert kernels run on the
//            local shard, and the BF16 down rows are gathered back in arrival order
//            [exchange 2: BF16 rows]
//   home:    weighted combine in slot order + the shared expert computed locally.
// The exchanges themselves are issued by the host side (NCCL all-to-all); nothing here waits on
// another GPU.
#include "p92b_common.cuh"
#include "tc_ptx.cuh"

#include <algorithm>

namespace p92b {
namespace {


// send[pos] = quantised row of the token behind permuted position pos.  One warp per row.
__global__ void __launch_bounds__(256) ep_pack_kernel(const std::uint8_t* __restrict__ xq,
                                                      const std::uint8_t* __restrict__ xs,
                                                      const std::int32_t* __restrict__ order,
                                                      std::uint8_t* __restrict__ send, int assignments, int q_bytes,
                                                      int s_bytes) {
    const int lane = threadIdx.x & 31;
    const int pos = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pos >= assignments) return;
    const int token = order[pos] / kTop;
    const uint4* src_q = reinterpret_cast<const uint4*>(xq + static_cast<std::size_t>(token) * q_bytes);
    const uint4* src_s = reinterpret_cast<const uint4*>(xs + static_cast<std::size_t>(token) * s_bytes);
    uint4* dst = reinterpret_cast<uint4*>(send + static_cast<std::size_t>(pos) * (q_bytes + s_bytes));
    for (int i = lane; i < q_bytes / 16; i += 32) dst[i] = src_q[i];
    for (int i = lane; i < s_bytes / 16; i += 32) dst[q_bytes / 16 + i] = src_s[i];
}

// Lists for the expert kernels from the per-source counts of the local experts.
//   recv_counts [sources][count_stride >= local]   rows source s sends for local expert e
//   counts[257] (global expert ids; zero outside the shard), pp_off[258] (128-aligned), active,
//   active_count, tile_prefix as the expert kernels expect them (no shared expert unless shared_rows>0)
//   src_base [sources][local]      padded position of the first row of (s, e)
//   src_start [sources][local+1]   index of that row inside the arrival buffer
__global__ void __launch_bounds__(256) ep_lists_kernel(const std::int32_t* __restrict__ recv_counts, int count_stride,
                                                       int sources, int first_expert, int local, int shared_rows,
                                                       int tile_rows,
                                                       std::int32_t* counts, std::int32_t* pp_off,
                                                       std::int32_t* active, std::int32_t* active_count,
                                                       std::int32_t* tile_prefix, std::int32_t* src_base,
                                                       std::int32_t* src_start) {
    __shared__ std::int32_t s_total[kExperts];
    __shared__ std::int32_t s_scan[kExperts + 1];
    const int e = threadIdx.x;                     // global expert id
    const int le = e - first_expert;
    const bool mine = le >= 0 && le < local;
    int total = 0;
    if (mine) {
        for (int s = 0; s < sources; ++s) total += recv_counts[s * count_stride + le];
    }
    s_total[e] = total;
    counts[e] = total;
    __syncthreads();
    if (threadIdx.x == 0) {
        // 256 entries: a serial pass is a few microseconds and keeps the three prefixes in one place
        int pp = 0, slot = 0, tiles = 0;
        const int shared_tiles = (shared_rows + tile_rows - 1) / tile_rows;
        if (shared_rows > 0) {
            active[slot++] = kExperts;
            tile_prefix[0] = 0;
            tiles = shared_tiles;
        }
        for (int i = 0; i < kExperts; ++i) {
            s_scan[i] = pp;
            pp_off[i] = pp;
            const int c = s_total[i];
            if (c > 0) {
                active[slot] = i;
                tile_prefix[slot] = tiles;
                ++slot;
                tiles += (c + tile_rows - 1) / tile_rows;
                pp += (c + 127) / 128 * 128;
            }
        }
        pp_off[kExperts] = pp;
        pp_off[kExperts + 1] = pp + (shared_rows + 127) / 128 * 128;
        counts[kExperts] = shared_rows;
        tile_prefix[slot] = tiles;
        *active_count = slot;
    }
    __syncthreads();
    if (mine) {
        int base = s_scan[e];
        for (int s = 0; s < sources; ++s) {
            src_base[s * local + le] = base;
            base += recv_counts[s * count_stride + le];
        }
    }
    // arrival index of the first row of (s, e): sources are concatenated, experts ascending inside a source
    if (threadIdx.x < sources) {
        const int s = threadIdx.x;
        int start = 0;
        for (int t = 0; t < s; ++t)
            for (int k = 0; k < local; ++k) start += recv_counts[t * count_stride + k];
        for (int k = 0; k < local; ++k) {
            src_start[s * (local + 1) + k] = start;
            start += recv_counts[s * count_stride + k];
        }
        src_start[s * (local + 1) + local] = start;
    }
}

// Arrived row i -> its padded position: finds (source, expert) from the run starts, copies the packed
// values, writes the scales into the 128x4 tiling, remembers the position for the way back.
__global__ void __launch_bounds__(256) ep_scatter_kernel(const std::uint8_t* __restrict__ recv,
                                                         const std::int32_t* __restrict__ src_start,
                                                         const std::int32_t* __restrict__ src_base, int sources,
                                                         int local, int total_rows, std::uint8_t* __restrict__ xq_pp,
                                                         std::uint8_t* __restrict__ xs_sw,
                                                         std::int32_t* __restrict__ pp_of_recv, int q_bytes,
                                                         int s_bytes) {
    const int lane = threadIdx.x & 31;
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= total_rows) return;
    int s = 0;
    while (s + 1 < sources && src_start[(s + 1) * (local + 1)] <= i) ++s;
    const std::int32_t* starts = src_start + s * (local + 1);
    int lo = 0, hi = local;                       // largest k with starts[k] <= i
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (starts[mid] <= i) lo = mid; else hi = mid;
    }
    while (lo + 1 < local && starts[lo + 1] <= i) ++lo;      // skip empty experts
    const std::size_t pp = static_cast<std::size_t>(src_base[s * local + lo] + (i - starts[lo]));
    const uint4* src = reinterpret_cast<const uint4*>(recv + static_cast<std::size_t>(i) * (q_bytes + s_bytes));
    uint4* dst = reinterpret_cast<uint4*>(xq_pp + pp * q_bytes);
    for (int k = lane; k < q_bytes / 16; k += 32) dst[k] = src[k];
    const std::uint8_t* scales = recv + static_cast<std::size_t>(i) * (q_bytes + s_bytes) + q_bytes;
    const int col_blocks = (s_bytes + 3) / 4;
    for (int b = lane; b < s_bytes; b += 32) {
        xs_sw[((pp >> 7) * col_blocks + (b >> 2)) * 512 + (pp & 31) * 16 + ((pp >> 5) & 3) * 4 + (b & 3)] = scales[b];
    }
    if (lane == 0) pp_of_recv[i] = static_cast<std::int32_t>(pp);
}

// out[i] = rows[index[i]]  (BF16 rows of `hidden` values), one warp per row.
__global__ void __launch_bounds__(256) ep_gather_rows_kernel(const std::uint16_t* __restrict__ rows,
                                                             const std::int32_t* __restrict__ index,
                                                             std::uint16_t* __restrict__ out, int total_rows,
                                                             int hidden) {
    const int lane = threadIdx.x & 31;
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= total_rows) return;
    const uint4* src = reinterpret_cast<const uint4*>(rows + static_cast<std::size_t>(index[i]) * hidden);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<std::size_t>(i) * hidden);
    for (int k = lane; k < hidden / 8; k += 32) dst[k] = src[k];
}

// Token rows (token order) -> padded positions 0..rows-1 of the shared expert's slab.
__global__ void __launch_bounds__(256) ep_shared_rows_kernel(const std::uint8_t* __restrict__ xq,
                                                             const std::uint8_t* __restrict__ xs, int rows,
                                                             std::uint8_t* __restrict__ xq_pp,
                                                             std::uint8_t* __restrict__ xs_sw, int q_bytes,
                                                             int s_bytes) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= rows) return;
    const std::size_t pp = static_cast<std::size_t>(t);
    const uint4* src = reinterpret_cast<const uint4*>(xq + static_cast<std::size_t>(t) * q_bytes);
    uint4* dst = reinterpret_cast<uint4*>(xq_pp + pp * q_bytes);
    for (int k = lane; k < q_bytes / 16; k += 32) dst[k] = src[k];
    const int col_blocks = (s_bytes + 3) / 4;
    for (int b = lane; b < s_bytes; b += 32) {
        xs_sw[((pp >> 7) * col_blocks + (b >> 2)) * 512 + (pp & 31) * 16 + ((pp >> 5) & 3) * 4 + (b & 3)] =
            xs[static_cast<std::size_t>(t) * s_bytes + b];
    }
}

// Home-side tail: FP32 combine of the returned rows in slot order (cuda/nvfp4_ops.cu:124-142), BF16
// rounding, + the shared expert's BF16 row, BF16 rounding (cuda/nvfp4_ops.cu:92-95).
__global__ void __launch_bounds__(256) ep_combine_kernel(const std::uint16_t* __restrict__ returned,
                                                         const std::int32_t* __restrict__ position,
                                                         const float* __restrict__ route_weights,
                                                         const std::uint16_t* __restrict__ shared_rows,
                                                         std::uint16_t* __restrict__ output, int hidden) {
    const int row = blockIdx.y;
    const int c8 = blockIdx.x * blockDim.x + threadIdx.x;
    if (c8 * 8 >= hidden) return;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0F;
#pragma unroll
    for (int slot = 0; slot < kTop; ++slot) {
        const int pos = position[row * kTop + slot];
        const float w = route_weights[row * kTop + slot];
        const uint4 r = *reinterpret_cast<const uint4*>(returned + static_cast<std::size_t>(pos) * hidden + c8 * 8);
        const std::uint32_t words[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            acc[2 * k] = fmaf(__uint_as_float(words[k] << 16), w, acc[2 * k]);
            acc[2 * k + 1] = fmaf(__uint_as_float(words[k] & 0xffff0000U), w, acc[2 * k + 1]);
        }
    }
    const uint4 sh = *reinterpret_cast<const uint4*>(shared_rows + static_cast<std::size_t>(row) * hidden + c8 * 8);
    const std::uint32_t sw[4] = {sh.x, sh.y, sh.z, sh.w};
    std::uint32_t out_words[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float lo = bf16_bits_to_float(float_to_bf16_bits(acc[2 * k])) + __uint_as_float(sw[k] << 16);
        const float hi = bf16_bits_to_float(float_to_bf16_bits(acc[2 * k + 1])) + __uint_as_float(sw[k] & 0xffff0000U);
        out_words[k] = static_cast<std::uint32_t>(float_to_bf16_bits(lo)) |
                       (static_cast<std::uint32_t>(float_to_bf16_bits(hi)) << 16);
    }
    *reinterpret_cast<uint4*>(output + static_cast<std::size_t>(row) * hidden + c8 * 8) =
        make_uint4(out_words[0], out_words[1], out_words[2], out_words[3]);
}

// ---- fixed-capacity exchange (small batches): no split size ever crosses to the host ------------
// Every (source, destination) pair owns a block of `cap` row slots behind a header with the
// per-expert counts, so both all-to-alls have equal splits and the whole layer stays asynchronous.
//   block = [ header: local int32, padded to 16 bytes ][ cap rows ]

__host__ __device__ inline std::size_t ep_header_bytes(int local) { return (static_cast<std::size_t>(local) * 4 + 15) / 16 * 16; }

// Home side: rows into their destination's block (slot = rank among the rows for that destination),
// headers = this GPU's histogram of the destination's experts, and for the way back the slot of
// every (row, slot) assignment in the returned buffer.
__global__ void __launch_bounds__(256) ep_pack_fixed_kernel(const std::uint8_t* __restrict__ xq,
                                                            const std::uint8_t* __restrict__ xs,
                                                            const std::int32_t* __restrict__ order,
                                                            const std::int32_t* __restrict__ ids,
                                                            const std::int32_t* __restrict__ counts,
                                                            const std::int32_t* __restrict__ offsets,
                                                            std::uint8_t* __restrict__ send, std::int32_t* __restrict__ ret_index,
                                                            int assignments, int world, int local, int cap, int q_bytes,
                                                            int s_bytes) {
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const std::size_t header = ep_header_bytes(local);
    const std::size_t block_bytes = header + static_cast<std::size_t>(cap) * (q_bytes + s_bytes);
    if (unit < world) {                                   // headers
        std::int32_t* h = reinterpret_cast<std::int32_t*>(send + unit * block_bytes);
        for (int k = lane; k < local; k += 32) h[k] = counts[unit * local + k];
    }
    if (unit >= assignments) return;
    const int pos = unit;
    const int flat = order[pos];
    const int token = flat / kTop;
    const int dst = ids[flat] / local;
    const int slot = pos - offsets[dst * local];
    if (lane == 0) ret_index[flat] = dst * cap + slot;
    if (slot >= cap) return;                              // cannot happen when cap >= 8 * rows
    const uint4* src_q = reinterpret_cast<const uint4*>(xq + static_cast<std::size_t>(token) * q_bytes);
    const uint4* src_s = reinterpret_cast<const uint4*>(xs + static_cast<std::size_t>(token) * s_bytes);
    uint4* row = reinterpret_cast<uint4*>(send + dst * block_bytes + header + static_cast<std::size_t>(slot) * (q_bytes + s_bytes));
    for (int i = lane; i < q_bytes / 16; i += 32) row[i] = src_q[i];
    for (int i = lane; i < s_bytes / 16; i += 32) row[q_bytes / 16 + i] = src_s[i];
}

// Owner side: slot (s, j) of the arrival buffer -> padded position (or -1 for an empty slot).
__global__ void __launch_bounds__(256) ep_scatter_fixed_kernel(const std::uint8_t* __restrict__ recv,
                                                               const std::int32_t* __restrict__ src_start,
                                                               const std::int32_t* __restrict__ src_base, int sources,
                                                               int local, int cap, std::uint8_t* __restrict__ xq_pp,
                                                               std::uint8_t* __restrict__ xs_sw,
                                                               std::int32_t* __restrict__ pp_of_slot, int q_bytes,
                                                               int s_bytes) {
    const int lane = threadIdx.x & 31;
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= sources * cap) return;
    const int s = i / cap;
    const int j = i - s * cap;
    const std::int32_t* starts = src_start + s * (local + 1);
    const int first = starts[0];
    if (j >= starts[local] - first) {
        if (lane == 0) pp_of_slot[i] = -1;
        return;
    }
    int lo = 0, hi = local;                       // largest k with starts[k] - first <= j
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (starts[mid] - first <= j) lo = mid; else hi = mid;
    }
    const std::size_t pp = static_cast<std::size_t>(src_base[s * local + lo] + (j - (starts[lo] - first)));
    const std::size_t header = ep_header_bytes(local);
    const std::size_t block_bytes = header + static_cast<std::size_t>(cap) * (q_bytes + s_bytes);
    const std::uint8_t* row = recv + s * block_bytes + header + static_cast<std::size_t>(j) * (q_bytes + s_bytes);
    const uint4* src = reinterpret_cast<const uint4*>(row);
    uint4* dst = reinterpret_cast<uint4*>(xq_pp + pp * q_bytes);
    for (int k = lane; k < q_bytes / 16; k += 32) dst[k] = src[k];
    const int col_blocks = (s_bytes + 3) / 4;
    for (int b = lane; b < s_bytes; b += 32) {
        xs_sw[((pp >> 7) * col_blocks + (b >> 2)) * 512 + (pp & 31) * 16 + ((pp >> 5) & 3) * 4 + (b & 3)] = row[q_bytes + b];
    }
    if (lane == 0) pp_of_slot[i] = static_cast<std::int32_t>(pp);
}

// out[slot] = rows[pp_of_slot[slot]] for the filled slots.
__global__ void __launch_bounds__(256) ep_gather_fixed_kernel(const std::uint16_t* __restrict__ rows,
                                                              const std::int32_t* __restrict__ pp_of_slot,
                                                              std::uint16_t* __restrict__ out, int slots, int hidden) {
    const int lane = threadIdx.x & 31;
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= slots) return;
    const int pp = pp_of_slot[i];
    if (pp < 0) return;
    const uint4* src = reinterpret_cast<const uint4*>(rows + static_cast<std::size_t>(pp) * hidden);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<std::size_t>(i) * hidden);
    for (int k = lane; k < hidden / 8; k += 32) dst[k] = src[k];
}

}  // namespace

// Lists of a GPU's experts from per-source histograms, for callers in other files.
cudaError_t launch_ep_lists(const std::int32_t* recv_counts, int count_stride, int sources, int first_expert, int local,
                            int shared_rows, int tile_rows, p92b_plan* plan, cudaStream_t stream) {
    if (static_cast<std::size_t>(sources) * (local + 1) > static_cast<std::size_t>(plan->ep_words)) return cudaErrorInvalidValue;
    ep_lists_kernel<<<1, 256, 0, stream>>>(recv_counts, count_stride, sources, first_expert, local, shared_rows, tile_rows,
                                           plan->counts, plan->pp_off, plan->active, plan->active_count, plan->tile_prefix,
                                           plan->ep_src_base, plan->ep_src_start);
    return cudaGetLastError();
}

namespace {

inline unsigned warps_grid(int rows) { return static_cast<unsigned>((rows + 7) / 8); }

}  // namespace
}  // namespace p92b

using namespace p92b;

extern "C" {

size_t p92b_ep_row_bytes(int hidden) { return static_cast<size_t>(hidden / 2 + hidden / 16); }

int p92b_ep_route(p92b_plan* plan, const uint16_t* input, const uint16_t* router_weight,
                  const float* correction_bias, int rows, float routed_scale, uint8_t* send_rows, void* stream_) {
    if (plan == nullptr || input == nullptr || router_weight == nullptr || correction_bias == nullptr ||
        send_rows == nullptr || rows <= 0 || rows > plan->max_rows) {
        return cudaErrorInvalidValue;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int hidden = plan->hidden;
    plan->last_launches = 0;
    // large batches: tensor-core logits with exact repair (same ids and weights); otherwise the exact-order kernels
    cudaError_t st = rows >= router_fast_min_rows()
                         ? launch_router_fast(plan, input, router_weight, correction_bias, rows, routed_scale, stream, false)
                         : cudaErrorNotSupported;
    if (st == cudaErrorNotSupported) {
        st = launch_router_logits(input, router_weight, plan->logits, rows, kExperts, hidden, rows == 1, stream);
        if (st != cudaSuccess) return st;
        st = launch_router_top8(plan->logits, correction_bias, plan->ids, plan->route_weights, rows, routed_scale, stream);
    }
    if (st != cudaSuccess) return st;
    st = launch_permute(plan, plan->ids, rows * kTop, plan->order, plan->position, plan->counts, plan->offsets, true, 1,
                        1 << 30, stream);
    if (st != cudaSuccess) return st;
    st = launch_quantize(input, plan->xq, plan->xs, static_cast<long>(rows) * hidden / 16, 1.0F, stream);
    if (st != cudaSuccess) return st;
    ep_pack_kernel<<<warps_grid(rows * kTop), 256, 0, stream>>>(plan->xq, plan->xs, plan->order, send_rows, rows * kTop,
                                                                hidden / 2, hidden / 16);
    plan->last_launches += 4;
    plan->last_path = 1;
    return cudaGetLastError();
}

int p92b_ep_experts(p92b_plan* plan, const p92b_bank* bank, const uint8_t* recv_rows, const int32_t* recv_counts,
                    int sources, int total_rows, uint16_t* out_rows, void* stream_) {
    if (plan == nullptr || bank == nullptr || recv_counts == nullptr || sources <= 0 || sources > 16 || total_rows < 0 ||
        total_rows > plan->max_rows * kTop || !plan->tc_ready || plan->hidden != bank->view.hidden ||
        plan->intermediate != bank->view.intermediate || (total_rows > 0 && (recv_rows == nullptr || out_rows == nullptr))) {
        return cudaErrorInvalidValue;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int local = bank->view.local_experts;
    if (static_cast<std::size_t>(sources) * (local + 1) > static_cast<std::size_t>(plan->ep_words)) return cudaErrorInvalidValue;
    plan->last_launches = 0;
    // the row count per expert is only known on the device: use the large-batch tile
    const int tile_rows = tc_tile_rows(1 << 20);
    ep_lists_kernel<<<1, 256, 0, stream>>>(recv_counts, local, sources, bank->view.first_expert, local, 0, tile_rows,
                                           plan->counts, plan->pp_off, plan->active, plan->active_count,
                                           plan->tile_prefix, plan->ep_src_base, plan->ep_src_start);
    cudaError_t st = cudaGetLastError();
    if (st != cudaSuccess || total_rows == 0) return st;
    ep_scatter_kernel<<<warps_grid(total_rows), 256, 0, stream>>>(recv_rows, plan->ep_src_start, plan->ep_src_base,
                                                                  sources, local, total_rows, plan->xq_pp, plan->xs_sw,
                                                                  plan->pp_of_flat, plan->hidden / 2, plan->hidden / 16);
    if ((st = cudaGetLastError()) != cudaSuccess) return st;
    plan->wide_rows = 0;          // the lists above carry one tile prefix only
    if ((st = launch_experts_tc(plan, bank, 1 << 20, false, stream)) != cudaSuccess) return st;
    if ((st = launch_experts_tc(plan, bank, 1 << 20, true, stream)) != cudaSuccess) return st;
    ep_gather_rows_kernel<<<warps_grid(total_rows), 256, 0, stream>>>(plan->mixed_pp, plan->pp_of_flat, out_rows,
                                                                      total_rows, plan->hidden);
    plan->last_launches = 5;
    plan->last_path = 2;
    return cudaGetLastError();
}

static int ep_combine_impl(p92b_plan* home_plan, p92b_plan* shared_plan, const p92b_bank* bank, const uint16_t* input,
                           const uint16_t* returned_rows, uint16_t* output, int rows, bool fixed, void* stream_) {
    if (home_plan == nullptr || shared_plan == nullptr || bank == nullptr || input == nullptr ||
        returned_rows == nullptr || output == nullptr || rows <= 0 || rows > home_plan->max_rows ||
        rows > shared_plan->max_rows || !shared_plan->tc_ready) {
        return cudaErrorInvalidValue;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    p92b_plan* sp = shared_plan;
    // shared expert on the home GPU: the only active entry, rows = the local tokens, positions 0..rows-1
    const int tile_rows = tc_tile_rows(rows);
    ep_lists_kernel<<<1, 256, 0, stream>>>(sp->ep_zero_counts, 1, 1, 0, 0, rows, tile_rows, sp->counts, sp->pp_off,
                                           sp->active, sp->active_count, sp->tile_prefix, sp->ep_src_base,
                                           sp->ep_src_start);
    cudaError_t st = cudaGetLastError();
    if (st != cudaSuccess) return st;
    // the home plan still holds this call's quantised token rows (p92b_ep_route)
    ep_shared_rows_kernel<<<warps_grid(rows), 256, 0, stream>>>(home_plan->xq, home_plan->xs, rows, sp->xq_pp, sp->xs_sw,
                                                                sp->hidden / 2, sp->hidden / 16);
    if ((st = cudaGetLastError()) != cudaSuccess) return st;
    sp->wide_rows = 0;
    if ((st = launch_experts_tc(sp, bank, rows, false, stream)) != cudaSuccess) return st;
    if ((st = launch_experts_tc(sp, bank, rows, true, stream)) != cudaSuccess) return st;
    dim3 grid((home_plan->hidden / 8 + 255) / 256, rows);
    ep_combine_kernel<<<grid, 256, 0, stream>>>(returned_rows, fixed ? home_plan->pp_of_flat : home_plan->position,
                                                home_plan->route_weights, sp->mixed_pp,
                                                output, home_plan->hidden);
    return cudaGetLastError();
}

int p92b_ep_combine(p92b_plan* home_plan, p92b_plan* shared_plan, const p92b_bank* bank, const uint16_t* input,
                    const uint16_t* returned_rows, uint16_t* output, int rows, void* stream) {
    return ep_combine_impl(home_plan, shared_plan, bank, input, returned_rows, output, rows, false, stream);
}

size_t p92b_ep_fixed_block_bytes(int hidden, int local_experts, int cap_rows) {
    return ep_header_bytes(local_experts) + static_cast<size_t>(cap_rows) * p92b_ep_row_bytes(hidden);
}

int p92b_ep_route_fixed(p92b_plan* plan, const uint16_t* input, const uint16_t* router_weight,
                        const float* correction_bias, int rows, float routed_scale, uint8_t* send_blocks, int world,
                        int cap_rows, void* stream_) {
    if (plan == nullptr || input == nullptr || router_weight == nullptr || correction_bias == nullptr ||
        send_blocks == nullptr || rows <= 0 || rows > plan->max_rows || world <= 0 || kExperts % world != 0 ||
        cap_rows < rows * kTop) {
        return cudaErrorInvalidValue;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int hidden = plan->hidden;
    plan->last_launches = 0;
    // large batches: tensor-core logits with exact repair (same ids and weights); otherwise the exact-order kernels
    cudaError_t st = rows >= router_fast_min_rows()
                         ? launch_router_fast(plan, input, router_weight, correction_bias, rows, routed_scale, stream, false)
                         : cudaErrorNotSupported;
    if (st == cudaErrorNotSupported) {
        st = launch_router_logits(input, router_weight, plan->logits, rows, kExperts, hidden, rows == 1, stream);
        if (st != cudaSuccess) return st;
        st = launch_router_top8(plan->logits, correction_bias, plan->ids, plan->route_weights, rows, routed_scale, stream);
    }
    if (st != cudaSuccess) return st;
    st = launch_permute(plan, plan->ids, rows * kTop, plan->order, plan->position, plan->counts, plan->offsets, true, 1,
                        1 << 30, stream);
    if (st != cudaSuccess) return st;
    st = launch_quantize(input, plan->xq, plan->xs, static_cast<long>(rows) * hidden / 16, 1.0F, stream);
    if (st != cudaSuccess) return st;
    const int units = std::max(rows * kTop, world);
    ep_pack_fixed_kernel<<<warps_grid(units), 256, 0, stream>>>(plan->xq, plan->xs, plan->order, plan->ids, plan->counts,
                                                                plan->offsets, send_blocks, plan->pp_of_flat, rows * kTop,
                                                                world, kExperts / world, cap_rows, hidden / 2, hidden / 16);
    plan->last_launches += 4;
    plan->last_path = 1;
    return cudaGetLastError();
}

int p92b_ep_experts_fixed(p92b_plan* plan, const p92b_bank* bank, const uint8_t* recv_blocks, int sources, int cap_rows,
                          uint16_t* out_slots, void* stream_) {
    if (plan == nullptr || bank == nullptr || recv_blocks == nullptr || out_slots == nullptr || sources <= 0 ||
        sources > 16 || cap_rows <= 0 || static_cast<long>(sources) * cap_rows > static_cast<long>(plan->max_rows) * kTop ||
        !plan->tc_ready || plan->hidden != bank->view.hidden || plan->intermediate != bank->view.intermediate) {
        return cudaErrorInvalidValue;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int local = bank->view.local_experts;
    const std::size_t block_bytes = p92b_ep_fixed_block_bytes(plan->hidden, local, cap_rows);
    const int slots = sources * cap_rows;
    // a token picks an expert at most once, so one expert sees at most slots / 8 rows: that picks the tile
    const int expert_rows_bound = std::max(1, slots / kTop);
    const int tile_rows = tc_tile_rows(expert_rows_bound);
    ep_lists_kernel<<<1, 256, 0, stream>>>(reinterpret_cast<const std::int32_t*>(recv_blocks),
                                           static_cast<int>(block_bytes / 4), sources, bank->view.first_expert, local, 0,
                                           tile_rows, plan->counts, plan->pp_off, plan->active, plan->active_count,
                                           plan->tile_prefix, plan->ep_src_base, plan->ep_src_start);
    cudaError_t st = cudaGetLastError();
    if (st != cudaSuccess) return st;
    ep_scatter_fixed_kernel<<<warps_grid(slots), 256, 0, stream>>>(recv_blocks, plan->ep_src_start, plan->ep_src_base,
                                                                   sources, local, cap_rows, plan->xq_pp, plan->xs_sw,
                                                                   plan->pp_of_flat, plan->hidden / 2, plan->hidden / 16);
    if ((st = cudaGetLastError()) != cudaSuccess) return st;
    plan->wide_rows = 0;
    if ((st = launch_experts_tc(plan, bank, expert_rows_bound, false, stream)) != cudaSuccess) return st;
    if ((st = launch_experts_tc(plan, bank, expert_rows_bound, true, stream)) != cudaSuccess) return st;
    ep_gather_fixed_kernel<<<warps_grid(slots), 256, 0, stream>>>(plan->mixed_pp, plan->pp_of_flat, out_slots, slots,
                                                                  plan->hidden);
    plan->last_launches = 5;
    plan->last_path = 2;
    return cudaGetLastError();
}

int p92b_ep_combine_fixed(p92b_plan* home_plan, p92b_plan* shared_plan, const p92b_bank* bank, const uint16_t* input,
                          const uint16_t* returned_slots, uint16_t* output, int rows, void* stream) {
    return ep_combine_impl(home_plan, shared_plan, bank, input, returned_slots, output, rows, true, stream);
}

}  // extern "C"
