// Expert-parallel MoE block for large batches (thousands of tokens per GPU): both exchanges done by the library's
// own kernels with plain 16-byte stores into the peers' windows over NVLink - no collective library, no split sizes
// crossing to the host, no host synchronisation anywhere in the layer.
//
//   dispatch = all-gather.  Every GPU routes its home tokens, quantises them (cuda/nvfp4_ops.cu:818-841; a token's
//       row is quantised independently of the expert it goes to, src/executor.cpp:53-59) and stores the 1,440-byte
//       rows and the top-8 ids into every peer's window.  With top-8 routing over 2..8 GPUs that moves the same bytes
//       per GPU as an all-to-all of one row per assignment would, and every size is known in advance.
//   routing.  Every GPU then holds the ids of the whole batch in the order (home GPU, token, slot) and runs the
//       permutation restricted to its own experts: the global permutation law (cuda/nvfp4_grouped.cu:117-132)
//       restricted to a GPU's experts IS that GPU's order, so per expert the rows are ordered exactly as one GPU
//       would order them.
//   experts.  The grouped tcgen05 kernels on this GPU's shard and, for its home tokens, the shared expert.
//   combine = direct placement.  Every result row is stored into its home GPU's window at [token][slot] (5 KB
//       each, the volume of an all-to-all return); the home GPU sums the eight slots in slot order and adds its
//       shared expert (cuda/nvfp4_ops.cu:124-142,92-95): the single-device combine law, bit for bit.  At large
//       batches the down product's own epilogue does these stores (a table of one destination pointer per padded row,
//       TcIo::row_dest; 256-byte runs), so the return crosses NVLink while the product is still running and only a
//       one-warp launch that publishes the flags follows; at small batches a separate kernel copies the rows.
//
// Synchronisation: data crosses as ordinary stores; after its stores a kernel's blocks fence at system scope and
// count themselves, the last one publishes the call number in a flag word of every peer (release, system scope);
// the consumer side waits for the flag of every peer with a bounded poll (about a second, then status 2) before it
// reads.  One window per GPU serves any number of layers; all GPUs must make the same sequence of calls on it.
// A GPU cannot run ahead of a peer by more than the part of a call before its first wait, so nothing is double-buffered:
// a GPU's next dispatch is issued after its own combine, which needed every peer's results of this call.
#include "p92b_common.cuh"
#include "tc_ptx.cuh"

#include <cstdlib>
#include <cstring>
#include <new>

namespace p92b {

using namespace ptx;

namespace {

constexpr int kMaxWorld = 16;
constexpr int kFlagBytes = 512;                 // arrive_flag[16], result_flag[16], block counters

struct BulkLayout {
    std::size_t flags, ids, rows, results, dest, total;
    int row_bytes;
    __host__ __device__ BulkLayout(int world, int rows_per_gpu, int hidden) {
        row_bytes = hidden / 2 + hidden / 16;
        flags = 0;
        ids = kFlagBytes;
        rows = ids + static_cast<std::size_t>(world) * rows_per_gpu * kTop * 4;
        rows = (rows + 255) / 256 * 256;
        results = rows + static_cast<std::size_t>(world) * rows_per_gpu * row_bytes;
        results = (results + 255) / 256 * 256;
        dest = results + static_cast<std::size_t>(rows_per_gpu) * kTop * hidden * 2;      // local use: one pointer per padded row
        dest = (dest + 255) / 256 * 256;
        total = dest + dest_entries(world, rows_per_gpu) * sizeof(void*);
    }
    __host__ __device__ static std::size_t dest_entries(int world, int rows_per_gpu) {
        return (static_cast<std::size_t>(world) * rows_per_gpu * (kTop + 1) + (kExperts + 1) * 127 + 127) / 128 * 128;
    }
};

struct PeerBases {
    std::uint8_t* base[kMaxWorld];
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// After a block's stores into the peers' windows: fence, count; the last block of the grid publishes `epoch` in
// flag word `which` (0 arrive, 1 result) of every peer and resets the counter for the next kernel.
__device__ __forceinline__ void publish_when_grid_done(PeerBases peers, std::size_t bulk_base, unsigned* counter, int which,
                                                       int rank, int world, unsigned epoch) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned done = atomicAdd(counter, 1U) + 1U;
        if (done == gridDim.x * gridDim.y) {
            __threadfence_system();
            *counter = 0U;
            for (int d = 0; d < world; ++d) {
                st_release_sys(reinterpret_cast<unsigned*>(peers.base[d] + bulk_base) + which * kMaxWorld + rank, epoch);
            }
        }
    }
}

// ---- 1. quantise the home tokens, store rows and ids into every window ----------------------------------------
// One warp per token slot.  The row is assembled in shared memory (packed values, then the 160 scale bytes) and
// leaves as 16-byte stores, 90 per peer.  Slots beyond `rows` publish ids of -1.
__global__ void __launch_bounds__(256) bulk_push_kernel(const std::uint16_t* __restrict__ x, const std::int32_t* __restrict__ my_ids,
                                                        PeerBases peers, std::size_t bulk_base, BulkLayout layout,
                                                        unsigned* counter, int rank, int world, int rows, int rows_per_gpu,
                                                        int hidden, float quant_scale, unsigned epoch) {
    extern __shared__ __align__(16) std::uint8_t push_smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * 8 + warp;
    if (t < rows_per_gpu) {
        const std::size_t slot = static_cast<std::size_t>(rank) * rows_per_gpu + t;
        const int id = t < rows && lane < kTop ? my_ids[t * kTop + lane] : -1;
        if (lane < kTop) {
            for (int d = 0; d < world; ++d) {
                reinterpret_cast<std::int32_t*>(peers.base[d] + bulk_base + layout.ids)[slot * kTop + lane] = id;
            }
        }
        if (t < rows) {
            std::uint8_t* row = push_smem + warp * layout.row_bytes;
            const int blocks16 = hidden / 16;
            for (int b = lane; b < blocks16; b += 32) {
                const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<std::size_t>(t) * hidden + b * 16);
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
                *reinterpret_cast<uint2*>(row + b * 8) = packed;
                row[hidden / 2 + b] = scale_bits;
            }
            __syncwarp();
            const int pieces = layout.row_bytes / 16;
            for (int d = 0; d < world; ++d) {
                uint4* dst = reinterpret_cast<uint4*>(peers.base[d] + bulk_base + layout.rows + slot * layout.row_bytes);
                for (int v = lane; v < pieces; v += 32) dst[v] = reinterpret_cast<const uint4*>(row)[v];
            }
        }
    }
    publish_when_grid_done(peers, bulk_base, counter, 0, rank, world, epoch);
}

// ---- waits ----------------------------------------------------------------------------------------------------
// One warp: lane d waits (bounded) until peer d's flag word carries this call's number.
__global__ void bulk_wait_kernel(const unsigned* __restrict__ flags, int world, unsigned epoch, std::int32_t* status) {
    const int d = threadIdx.x;
    if (d >= world) return;
    const std::uint64_t start = global_timer_ns();
    while (static_cast<int>(ld_acquire_sys(flags + d) - epoch) < 0) {
        if (poll_expired(start)) {
            atomicCAS(status, kStatusOk, kStatusWaitExpired);
            return;
        }
    }
}

// ---- 2. rows of this GPU's experts (and its own shared-expert rows) into the padded position space -------------
__global__ void __launch_bounds__(256) bulk_scatter_kernel(const std::uint8_t* __restrict__ arrived, const std::int32_t* __restrict__ pp_of_flat,
                                                           const std::int32_t* __restrict__ order, const std::int32_t* __restrict__ counts,
                                                           const std::int32_t* __restrict__ offsets,
                                                           int assignments, int home_first_token, int home_rows, int row_bytes,
                                                           int k_bytes, std::uint8_t* __restrict__ xq, std::uint8_t* __restrict__ xs,
                                                           PeerBases peers, std::size_t results_base, int rows_per_gpu,
                                                           std::uint16_t* mixed_pp, std::uint16_t** row_dest) {
    // A fixed grid walks the rows this GPU computes: the sorted positions of its experts' assignments (order[] maps a
    // position back to the flat index; with 2..8 GPUs these are a half to an eighth of the batch, and a block per
    // eight flat indices would mostly launch blocks that leave at once), then its own shared-expert rows.
    const int lane = threadIdx.x & 31;
    const int local_total = offsets[kExperts - 1] + counts[kExperts - 1];
    for (int work = blockIdx.x * 8 + (threadIdx.x >> 5); work < local_total + home_rows; work += gridDim.x * 8) {
    const int unit = work < local_total ? order[work] : assignments + (work - local_total);
    const int pp_signed = pp_of_flat[unit];
    if (pp_signed < 0) continue;                                 // (cannot happen for a listed position)
    const std::size_t pp = static_cast<std::size_t>(pp_signed);
    const std::size_t token = unit < assignments ? unit / kTop : home_first_token + (unit - assignments);
    if (row_dest != nullptr && lane == 0) {
        // where the down product stores this row: slot [token][slot] of the results in its home GPU's window, or,
        // for a shared-expert row, its own padded position on this GPU
        const int hidden = k_bytes * 2;
        if (unit < assignments) {
            const int home = static_cast<int>(token) / rows_per_gpu;
            const std::size_t slot_row = (token - static_cast<std::size_t>(home) * rows_per_gpu) * kTop + (unit - token * kTop);
            row_dest[pp] = reinterpret_cast<std::uint16_t*>(peers.base[home] + results_base) + slot_row * hidden;
        } else {
            row_dest[pp] = mixed_pp + pp * hidden;
        }
    }
    // 1,280 + 160 bytes at hidden 2560: every lane's loads are issued before its first store; the scale bytes move as
    // 4-byte words (a row's four scales of one 64-element step are neighbours in both layouts)
    const std::uint8_t* src = arrived + token * row_bytes;
    uint4* to = reinterpret_cast<uint4*>(xq + pp * k_bytes);
    const int pieces = k_bytes / 16;
    constexpr int kMaxPerLane = 4;                              // hidden <= 4096
    uint4 held[kMaxPerLane];
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int v = lane + 32 * i;
        if (v < pieces) held[i] = __ldcs(reinterpret_cast<const uint4*>(src) + v);
    }
    const int scale_words = k_bytes / 32;                       // K / 16 scale bytes, four to a word
    const int col_blocks = scale_words;
    std::uint8_t* sf_to = xs + (pp >> 7) * col_blocks * 512 + (pp & 31) * 16 + ((pp >> 5) & 3) * 4;
    std::uint32_t scale_word[2] = {0U, 0U};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int c = lane + 32 * i;
        if (c < scale_words) scale_word[i] = __ldcs(reinterpret_cast<const std::uint32_t*>(src + k_bytes) + c);
    }
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int v = lane + 32 * i;
        if (v < pieces) to[v] = held[i];
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int c = lane + 32 * i;
        if (c < scale_words) *reinterpret_cast<std::uint32_t*>(sf_to + static_cast<std::size_t>(c) * 512) = scale_word[i];
    }
    }
}

// ---- 3. result rows to their home GPUs ------------------------------------------------------------------------
__global__ void __launch_bounds__(256) bulk_return_kernel(const std::uint16_t* __restrict__ mixed_pp, const std::int32_t* __restrict__ pp_of_flat,
                                                          PeerBases peers, std::size_t bulk_base, BulkLayout layout,
                                                          unsigned* counter, int assignments, int rank, int world,
                                                          int rows_per_gpu, int hidden, unsigned epoch) {
    const int lane = threadIdx.x & 31;
    const int a = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (a < assignments) {
        const int pp = pp_of_flat[a];
        if (pp >= 0) {
            const int token = a / kTop;
            const int home = token / rows_per_gpu;
            const std::size_t slot_row = static_cast<std::size_t>(token - home * rows_per_gpu) * kTop + (a - token * kTop);
            const uint4* src = reinterpret_cast<const uint4*>(mixed_pp + static_cast<std::size_t>(pp) * hidden);
            uint4* dst = reinterpret_cast<uint4*>(peers.base[home] + bulk_base + layout.results + slot_row * hidden * 2);
            for (int v = lane; v < hidden / 8; v += 32) dst[v] = __ldcg(src + v);
        }
    }
    publish_when_grid_done(peers, bulk_base, counter + 1, 1, rank, world, epoch);
}

// The down product stored its rows straight into the windows (TcIo::row_dest): this launch comes after it in the
// stream, so those stores are complete, and only has to tell every peer.
__global__ void bulk_publish_kernel(PeerBases peers, std::size_t bulk_base, int which, int rank, int world, unsigned epoch) {
    const int d = threadIdx.x;
    if (d >= world) return;
    __threadfence_system();
    st_release_sys(reinterpret_cast<unsigned*>(peers.base[d] + bulk_base) + which * kMaxWorld + rank, epoch);
}

// ---- 4. combine on the home GPU: eight slots in slot order, one rounding, then the shared expert ----------------
__global__ void __launch_bounds__(256) bulk_combine_kernel(const std::uint16_t* __restrict__ results, const float* __restrict__ route_weights,
                                                           const std::uint16_t* __restrict__ mixed_pp, const std::int32_t* __restrict__ pp_off,
                                                           std::uint16_t* __restrict__ out, int rows, int hidden) {
    const int row = blockIdx.y;
    const int c8 = blockIdx.x * blockDim.x + threadIdx.x;
    if (c8 * 8 >= hidden || row >= rows) return;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0F;
    uint4 slot_rows[kTop];
    float w[kTop];
#pragma unroll
    for (int slot = 0; slot < kTop; ++slot) {
        w[slot] = route_weights[row * kTop + slot];
        slot_rows[slot] = *reinterpret_cast<const uint4*>(results + (static_cast<std::size_t>(row) * kTop + slot) * hidden + c8 * 8);
    }
#pragma unroll
    for (int slot = 0; slot < kTop; ++slot) {
        const std::uint32_t words[4] = {slot_rows[slot].x, slot_rows[slot].y, slot_rows[slot].z, slot_rows[slot].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            acc[2 * k] = fmaf(__uint_as_float(words[k] << 16), w[slot], acc[2 * k]);
            acc[2 * k + 1] = fmaf(__uint_as_float(words[k] & 0xffff0000U), w[slot], acc[2 * k + 1]);
        }
    }
    const uint4 sh = *reinterpret_cast<const uint4*>(mixed_pp + static_cast<std::size_t>(pp_off[kExperts] + row) * hidden + c8 * 8);
    const std::uint32_t sw[4] = {sh.x, sh.y, sh.z, sh.w};
    std::uint32_t out_words[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float lo = bf16_bits_to_float(float_to_bf16_bits(acc[2 * k])) + __uint_as_float(sw[k] << 16);
        const float hi = bf16_bits_to_float(float_to_bf16_bits(acc[2 * k + 1])) + __uint_as_float(sw[k] & 0xffff0000U);
        out_words[k] = static_cast<std::uint32_t>(float_to_bf16_bits(lo)) | (static_cast<std::uint32_t>(float_to_bf16_bits(hi)) << 16);
    }
    *reinterpret_cast<uint4*>(out + static_cast<std::size_t>(row) * hidden + c8 * 8) =
        make_uint4(out_words[0], out_words[1], out_words[2], out_words[3]);
}

}  // namespace

}  // namespace p92b

extern "C" {

int p92b_ep_window_create_bulk(p92b_ep_window** out, int rank, int world, int rows_per_gpu, int hidden) {
    using namespace p92b;
    if (out == nullptr) return cudaErrorInvalidValue;
    *out = nullptr;
    if (world <= 0 || world > kMaxWorld || rank < 0 || rank >= world || kExperts % world != 0 || rows_per_gpu <= 0 ||
        rows_per_gpu > (1 << 16) || hidden <= 0 || hidden % 256 != 0 || hidden > 4096) {
        return cudaErrorInvalidValue;
    }
    p92b_ep_window* w = new (std::nothrow) p92b_ep_window();
    if (w == nullptr) return cudaErrorMemoryAllocation;
    w->rank = rank;
    w->world = world;
    w->rows_per_gpu = rows_per_gpu;
    w->fused_ok = false;
    w->bulk = true;
    w->bulk_hidden = hidden;
    const BulkLayout layout(world, rows_per_gpu, hidden);
    w->bytes = layout.total;
    cudaError_t st = cudaMalloc(reinterpret_cast<void**>(&w->local), w->bytes);
    if (st == cudaSuccess) st = cudaMemset(w->local, 0, kFlagBytes);
    if (st == cudaSuccess) st = cudaDeviceSynchronize();
    if (st != cudaSuccess) {
        if (w->local != nullptr) cudaFree(w->local);
        delete w;
        return st;
    }
    w->peers[rank] = w->local;
    w->connected = world == 1;
    *out = w;
    return cudaSuccess;
}

int p92b_ep_forward_bulk(p92b_plan* plan, const p92b_bank* bank, p92b_ep_window* window, const uint16_t* input,
                         const uint16_t* router_weight, const float* correction_bias, uint16_t* output, int rows,
                         float routed_scale, void* stream_) {
    using namespace p92b;
    if (plan == nullptr || bank == nullptr || window == nullptr || input == nullptr || router_weight == nullptr ||
        correction_bias == nullptr || output == nullptr || rows <= 0 || rows > window->rows_per_gpu) {
        return cudaErrorInvalidValue;
    }
    const int world = window->world;
    const int rpg = window->rows_per_gpu;
    const int local = kExperts / world;
    const int tokens = world * rpg;
    const int hidden = plan->hidden;
    if (!window->bulk || !window->connected || window->bulk_hidden != hidden || !plan->tc_ready || !bank->tc_ready ||
        bank->view.hidden != hidden || bank->view.intermediate != plan->intermediate || bank->view.local_experts != local ||
        bank->view.first_expert != window->rank * local || plan->max_rows < tokens) {
        return cudaErrorNotSupported;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const BulkLayout layout(world, rpg, hidden);
    const unsigned epoch = ++window->epoch;
    PeerBases peers {};
    for (int r = 0; r < world; ++r) peers.base[r] = window->peers[r];
    std::uint8_t* mine = window->local;
    unsigned* flags = reinterpret_cast<unsigned*>(mine + layout.flags);
    unsigned* counters = flags + 2 * kMaxWorld;
    const int assignments = tokens * kTop;
    plan->last_launches = 0;
    plan->last_path = 2;
    // optional stage timing (p92b_plan_stage_timing): 0 router, 1 dispatch (stores + wait for every peer's rows),
    // 2 permutation + placement, 3 unused, 4 gate/up, 5 down, 6 return (stores + wait for every peer's results) + combine
    int stage = 0;
    auto mark = [&]() -> cudaError_t {
        if (!plan->timing) return cudaSuccess;
        return cudaEventRecord(plan->stage_events[stage++], stream);
    };
    if (cudaError_t m = mark(); m != cudaSuccess) return m;

    // router of the home tokens: ids into plan->ids, weights stay in plan->route_weights for the combine
    cudaError_t st = rows >= router_fast_min_rows()
                         ? launch_router_fast(plan, input, router_weight, correction_bias, rows, routed_scale, stream, false)
                         : cudaErrorNotSupported;
    if (st == cudaErrorNotSupported) {
        st = launch_router_logits(input, router_weight, plan->logits, rows, kExperts, hidden, false, stream);
        if (st != cudaSuccess) return st;
        st = launch_router_top8(plan->logits, correction_bias, plan->ids, plan->route_weights, rows, routed_scale, stream);
        plan->last_launches += 2;
    }
    if (st != cudaSuccess) return st;
    if ((st = mark()) != cudaSuccess) return st;
    // dispatch
    if ((st = ensure_dynamic_smem<bulk_push_kernel>(8 * layout.row_bytes)) != cudaSuccess) return st;
    bulk_push_kernel<<<(rpg + 7) / 8, 256, 8 * layout.row_bytes, stream>>>(input, plan->ids, peers, 0, layout, counters, window->rank,
                                                                           world, rows, rpg, hidden, 1.0F, epoch);
    bulk_wait_kernel<<<1, 32, 0, stream>>>(flags, world, epoch, plan->status);
    if ((st = cudaGetLastError()) != cudaSuccess) return st;
    if ((st = mark()) != cudaSuccess) return st;
    // the permutation law over the whole batch, restricted to this GPU's experts; lists for the grouped kernels
    st = cudaMemsetAsync(plan->pp_of_flat, 0xff, static_cast<std::size_t>(assignments + rows) * sizeof(std::int32_t), stream);
    if (st != cudaSuccess) return st;
    const std::int32_t* all_ids = reinterpret_cast<const std::int32_t*>(mine + layout.ids);
    st = launch_permute(plan, all_ids, assignments, plan->order, plan->position, plan->counts, plan->offsets, true,
                        tc_pad_align(tokens), tc_tile_rows(tokens), stream, false, bank->view.first_expert, local, rows);
    if (st != cudaSuccess) return st;
    const int units = assignments + rows;
    // large batches: the down product stores every row where the combine wants it, over NVLink while it computes
    const bool direct = down_slab_applies(plan, tokens) && std::getenv("P92B_BULK_NO_DIRECT") == nullptr;
    std::uint16_t** row_dest = direct ? reinterpret_cast<std::uint16_t**>(mine + layout.dest) : nullptr;
    (void)units;
    bulk_scatter_kernel<<<plan->sm_count * 4, 256, 0, stream>>>(mine + layout.rows, plan->pp_of_flat, plan->order, plan->counts,
                                                                plan->offsets, assignments,
                                                             window->rank * rpg, rows, layout.row_bytes, hidden / 2, plan->xq_pp,
                                                             plan->xs_sw, peers, layout.results, rpg, plan->mixed_pp, row_dest);
    if ((st = cudaGetLastError()) != cudaSuccess) return st;
    if ((st = mark()) != cudaSuccess) return st;
    if ((st = mark()) != cudaSuccess) return st;
    if ((st = launch_experts_tc(plan, bank, tokens, false, stream, false)) != cudaSuccess) return st;
    if ((st = mark()) != cudaSuccess) return st;
    TcIo io {};
    io.row_dest = row_dest;
    if ((st = launch_experts_tc(plan, bank, tokens, true, stream, false, direct ? &io : nullptr)) != cudaSuccess) return st;
    if ((st = mark()) != cudaSuccess) return st;
    // combine
    if (direct) {
        bulk_publish_kernel<<<1, 32, 0, stream>>>(peers, 0, 1, window->rank, world, epoch);
    } else {
        bulk_return_kernel<<<(assignments + 7) / 8, 256, 0, stream>>>(plan->mixed_pp, plan->pp_of_flat, peers, 0, layout, counters,
                                                                      assignments, window->rank, world, rpg, hidden, epoch);
    }
    bulk_wait_kernel<<<1, 32, 0, stream>>>(flags + kMaxWorld, world, epoch, plan->status);
    dim3 grid((hidden / 8 + 255) / 256, rows);
    bulk_combine_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const std::uint16_t*>(mine + layout.results),
                                                  plan->route_weights, plan->mixed_pp, plan->pp_off, output, rows, hidden);
    plan->last_launches += 10;
    if ((st = cudaGetLastError()) != cudaSuccess) return st;
    if (plan->timing) {
        if ((st = mark()) != cudaSuccess) return st;
        if ((st = cudaStreamSynchronize(stream)) != cudaSuccess) return st;
        for (int i = 0; i < P92B_STAGES; ++i) {
            float ms = 0.0F;
            if ((st = cudaEventElapsedTime(&ms, plan->stage_events[i], plan->stage_events[i + 1])) != cudaSuccess) return st;
            plan->stage_ms[i] += ms;
        }
        plan->timed_calls += 1;
    }
    return cudaSuccess;
}

}  // extern "C"
