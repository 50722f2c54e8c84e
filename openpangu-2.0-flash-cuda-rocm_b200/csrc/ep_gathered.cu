// Expert-parallel MoE block for medium batches (tens of tokens per GPU, up to 1024 in flight): the
// exchanges are done by the library's own kernels with stores into the peers' windows over NVLink,
// like the single-kernel decode path (decode_ep.cu), but the block is a short sequence of launches
// and the expert products are the grouped tcgen05 kernels, so an expert may have any number of rows.
//
//   dispatch = all-gather.  Every GPU quantises its tokens and stores rows, scales and top-8 ids
//       into every peer's window (1.5 KB per token and peer: 0.75 MB per GPU for 512 tokens, a
//       microsecond of NVLink).  Every GPU then has the whole batch and ranks the rows of its own
//       experts by the reference's law (cuda/nvfp4_grouped.cu:117-132): per expert the rows are
//       ordered by (home GPU, token, slot), exactly as one GPU would order them.
//   combine = direct placement.  After the down product each result row is stored into its home
//       GPU's window at [token][slot]; the home GPU sums in slot order and adds its shared expert
//       (cuda/nvfp4_ops.cu:124-142,92-95), which it computed in the same grouped launches.
//
// As in decode_ep.cu every word that crosses NVLink is 8 bytes {payload, call number} and is polled
// by its reader: no fence, no flag, no collective library, no host synchronisation; windows are
// double-buffered by call parity.  All polls are bounded by wall time and end in the plan's status word.
#include "p92b_common.cuh"
#include "tc_ptx.cuh"

#include <algorithm>
#include <cstdlib>

namespace p92b {

using namespace ptx;

namespace {

constexpr int kTokIdWords = kTop, kTokRowWords = 320, kTokScaleWords = 40;
constexpr int kTokWords = kTokIdWords + kTokRowWords + kTokScaleWords;     // 368 tagged words per token
constexpr int kRetRowWords = 1280;                                         // two BF16 per tagged word

struct Regions {
    std::size_t arrive_parity, ret_parity, ret_base;
    __host__ __device__ Regions(int world, int rows_per_gpu) {
        arrive_parity = static_cast<std::size_t>(world) * rows_per_gpu * kTokWords * 8;
        ret_base = 2 * arrive_parity;
        ret_parity = static_cast<std::size_t>(rows_per_gpu) * kTop * kRetRowWords * 8;
    }
};

__device__ __forceinline__ bool expired(std::uint64_t start) { return poll_expired(start); }

struct Peers {
    std::uint8_t* base[16];        // every GPU's gathered regions
};

// ---- 1. quantise the home tokens and store them, with their ids, into every window -----------------
// One thread per 16-element block (cuda/nvfp4_ops.cu:818-841); 160 blocks per row, so whole warps.
__global__ void __launch_bounds__(256) epg_push_kernel(const std::uint16_t* __restrict__ x,
                                                       const std::int32_t* __restrict__ my_ids, Peers peers,
                                                       std::size_t arrive_offset, int rank, int world, int rows,
                                                       int rows_per_gpu, int hidden, float quant_scale, std::uint32_t tag) {
    pdl_wait();
    pdl_launch_dependents();
    const int blocks16 = hidden / 16;
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    const std::size_t first_word = static_cast<std::size_t>(rank) * rows_per_gpu * kTokWords;
    if (g < rows * blocks16) {
        const int t = g / blocks16;
        const int b = g - t * blocks16;
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
        std::uint32_t scales4 = scale_bits;
        scales4 |= __shfl_down_sync(0xffffffffU, static_cast<std::uint32_t>(scale_bits), 1) << 8;
        scales4 |= __shfl_down_sync(0xffffffffU, static_cast<std::uint32_t>(scale_bits), 2) << 16;
        scales4 |= __shfl_down_sync(0xffffffffU, static_cast<std::uint32_t>(scale_bits), 3) << 24;
        for (int d = 0; d < world; ++d) {
            std::uint64_t* dst = reinterpret_cast<std::uint64_t*>(peers.base[d] + arrive_offset) + first_word +
                                 static_cast<std::size_t>(t) * kTokWords + kTokIdWords;
            st_tagged(dst + 2 * b, packed.x, tag);
            st_tagged(dst + 2 * b + 1, packed.y, tag);
            if ((b & 3) == 0) st_tagged(dst + kTokRowWords + (b >> 2), scales4, tag);
        }
    }
    // ids of all token slots of this GPU (-1: slot not filled this time), by the first threads of the grid
    if (g < rows_per_gpu * kTop) {
        const int t = g / kTop;
        const std::uint32_t id = static_cast<std::uint32_t>(t < rows ? my_ids[g] : -1);
        for (int d = 0; d < world; ++d) {
            std::uint64_t* dst = reinterpret_cast<std::uint64_t*>(peers.base[d] + arrive_offset) + first_word +
                                 static_cast<std::size_t>(t) * kTokWords;
            st_tagged(dst + (g - t * kTop), id, tag);
        }
    }
}

// ---- 2. routing lists of this GPU's experts from the ids of the whole batch -------------------------
// One block.  A token picks an expert at most once, so per local expert a bit mask of tokens says
// everything: its popcount is the expert's row count, the popcount below a token's bit is that row's
// rank - the order of cuda/nvfp4_grouped.cu:117-132 (same expert: by flat index = by token), without
// sorting the assignments of other GPUs' experts.  Writes what the grouped expert kernels read
// (counts, 128-aligned padded offsets, active list with the shared expert first, token-tile prefix)
// and the padded position of every assignment (-1: not this GPU's expert, or an empty token slot).
constexpr int kRouteThreads = 1024;
constexpr int kMaskWords = 32;                       // up to 1024 tokens
constexpr int kRoutePerThread = 8;                   // up to 8192 assignments

__global__ void __launch_bounds__(kRouteThreads) epg_route_kernel(const std::uint64_t* __restrict__ arrive, int tokens,
                                                                  int first_expert, int local, int shared_rows,
                                                                  int tile_rows, std::uint32_t tag,
                                                                  std::int32_t* __restrict__ counts,
                                                                  std::int32_t* __restrict__ pp_off,
                                                                  std::int32_t* __restrict__ active,
                                                                  std::int32_t* __restrict__ active_count,
                                                                  std::int32_t* __restrict__ tile_prefix,
                                                                  std::int32_t* __restrict__ pp_of_assignment,
                                                                  std::int32_t* status) {
    extern __shared__ std::uint32_t route_smem[];
    std::uint32_t* mask = route_smem;                                   // [local][kMaskWords]
    std::int32_t* expert_pp = reinterpret_cast<std::int32_t*>(route_smem + local * kMaskWords);   // [local]
    std::int32_t* expert_rows = expert_pp + local;                                                  // [local]
    pdl_wait();
    pdl_launch_dependents();
    const int assignments = tokens * kTop;
    for (int i = threadIdx.x; i < local * kMaskWords; i += kRouteThreads) mask[i] = 0U;
    __syncthreads();
    std::int32_t mine[kRoutePerThread];
    {
        uint2 word[kRoutePerThread];
        const std::uint64_t start = global_timer_ns();
        while (true) {
            bool missing = false;
#pragma unroll
            for (int j = 0; j < kRoutePerThread; ++j) {
                const int a = threadIdx.x + j * kRouteThreads;
                if (a < assignments) {
                    const int g = a / kTop;
                    word[j] = ld_tagged(arrive + static_cast<std::size_t>(g) * kTokWords + (a - g * kTop));
                } else {
                    word[j] = make_uint2(0xffffffffU, tag);
                }
            }
#pragma unroll
            for (int j = 0; j < kRoutePerThread; ++j) {
                const int a = threadIdx.x + j * kRouteThreads;
                if (a < assignments && word[j].y != tag) missing = true;
            }
            if (!missing) break;
            if (expired(start)) {
                atomicCAS(status, kStatusOk, kStatusWaitExpired);
#pragma unroll
                for (int j = 0; j < kRoutePerThread; ++j) {
                    if (word[j].y != tag) word[j].x = 0xffffffffU;         // treated as an empty slot
                }
                break;
            }
        }
#pragma unroll
        for (int j = 0; j < kRoutePerThread; ++j) {
            const int a = threadIdx.x + j * kRouteThreads;
            mine[j] = -1;
            if (a < assignments) {
                const int le = static_cast<std::int32_t>(word[j].x) - first_expert;
                if (static_cast<std::int32_t>(word[j].x) >= 0 && le >= 0 && le < local) {
                    mine[j] = le;
                    const int g = a / kTop;
                    atomicOr(&mask[le * kMaskWords + (g >> 5)], 1U << (g & 31));
                }
            }
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < kExperts; e += kRouteThreads) {
        const int le = e - first_expert;
        int count = 0;
        if (le >= 0 && le < local) {
#pragma unroll 8
            for (int w = 0; w < kMaskWords; ++w) count += __popc(mask[le * kMaskWords + w]);
        }
        counts[e] = count;
        if (le >= 0 && le < local) expert_rows[le] = count;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // 256 entries: a serial pass keeps the three prefixes in one place
        int pp = 0, slot = 0, tiles = 0;
        if (shared_rows > 0) {
            active[slot++] = kExperts;
            tile_prefix[0] = 0;
            tiles = (shared_rows + tile_rows - 1) / tile_rows;
        }
        for (int e = 0; e < kExperts; ++e) {
            pp_off[e] = pp;
            const int le = e - first_expert;
            if (le < 0 || le >= local) continue;
            expert_pp[le] = pp;
            const int c = expert_rows[le];
            if (c > 0) {
                active[slot] = e;
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
#pragma unroll
    for (int j = 0; j < kRoutePerThread; ++j) {
        const int a = threadIdx.x + j * kRouteThreads;
        if (a >= assignments) continue;
        int pp = -1;
        if (mine[j] >= 0) {
            const int g = a / kTop;
            const std::uint32_t* m = mask + mine[j] * kMaskWords;
            int rank = __popc(m[g >> 5] & ((1U << (g & 31)) - 1U));
            for (int w = 0; w < (g >> 5); ++w) rank += __popc(m[w]);
            pp = expert_pp[mine[j]] + rank;
        }
        pp_of_assignment[a] = pp;
    }
}

// ---- 3. rows of this GPU's experts into the padded position space ---------------------------------
// One warp per assignment of the batch, then one per home token (the shared expert's rows).
__global__ void __launch_bounds__(256) epg_scatter_kernel(const std::uint64_t* __restrict__ arrive,
                                                          const std::int32_t* __restrict__ pp_of_assignment,
                                                          const std::int32_t* __restrict__ pp_off, int assignments,
                                                          int rank, int rows, int rows_per_gpu,
                                                          std::uint8_t* __restrict__ xq_pp, std::uint8_t* __restrict__ xs_sw,
                                                          std::uint32_t tag, std::int32_t* status) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= assignments + rows) return;
    int token, pp;
    if (unit < assignments) {
        pp = pp_of_assignment[unit];
        if (pp < 0) return;
        token = unit / kTop;
    } else {
        const int t = unit - assignments;
        token = rank * rows_per_gpu + t;
        pp = pp_off[kExperts] + t;
    }
    const std::uint64_t* src = arrive + static_cast<std::size_t>(token) * kTokWords + kTokIdWords;
    constexpr int kPerLane = (kTokRowWords + kTokScaleWords + 31) / 32;       // 12
    uint2 word[kPerLane];
    const std::uint64_t start = global_timer_ns();
    while (true) {
        bool missing = false;
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) {
            const int w = lane + 32 * j;
            word[j] = w < kTokRowWords + kTokScaleWords ? ld_tagged(src + w) : make_uint2(0U, tag);
        }
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) missing = missing || word[j].y != tag;
        if (!__any_sync(0xffffffffU, missing)) break;
        if (__any_sync(0xffffffffU, expired(start))) {          // one decision for the whole warp
            if (lane == 0) atomicCAS(status, kStatusOk, kStatusWaitExpired);
            return;
        }
    }
    std::uint32_t* row_out = reinterpret_cast<std::uint32_t*>(xq_pp + static_cast<std::size_t>(pp) * (kTokRowWords * 4));
    const std::size_t upp = static_cast<std::size_t>(pp);
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
        const int w = lane + 32 * j;
        if (w < kTokRowWords) {
            row_out[w] = word[j].x;
        } else if (w < kTokRowWords + kTokScaleWords) {
            const int c = w - kTokRowWords;                                   // four scale columns 4c .. 4c+3
            *reinterpret_cast<std::uint32_t*>(xs_sw + ((upp >> 7) * kTokScaleWords + c) * 512 + (upp & 31) * 16 +
                                              ((upp >> 5) & 3) * 4) = word[j].x;
        }
    }
}

// ---- 4. result rows to their home GPUs ----------------------------------------------------------------
__global__ void __launch_bounds__(256) epg_return_kernel(const std::uint16_t* __restrict__ mixed_pp,
                                                         const std::int32_t* __restrict__ pp_of_assignment, Peers peers,
                                                         std::size_t ret_offset, int assignments, int rows_per_gpu,
                                                         int hidden, std::uint32_t tag) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int a = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (a >= assignments) return;
    const int pp = pp_of_assignment[a];
    if (pp < 0) return;
    const int token = a / kTop;
    const int home = token / rows_per_gpu;
    const int slot_row = (token - home * rows_per_gpu) * kTop + (a - token * kTop);
    const std::uint32_t* src = reinterpret_cast<const std::uint32_t*>(mixed_pp + static_cast<std::size_t>(pp) * hidden);
    std::uint64_t* dst = reinterpret_cast<std::uint64_t*>(peers.base[home] + ret_offset) +
                         static_cast<std::size_t>(slot_row) * kRetRowWords;
    for (int w = lane; w < hidden / 2; w += 32) st_tagged(dst + w, __ldcg(src + w), tag);
}

// ---- 5. combine on the home GPU ----------------------------------------------------------------------
// One thread per four output features: eight routed slots in slot order (polled), then the shared expert.
__global__ void __launch_bounds__(256) epg_combine_kernel(const std::uint64_t* __restrict__ ret,
                                                          const float* __restrict__ route_weights,
                                                          const std::uint16_t* __restrict__ mixed_pp,
                                                          const std::int32_t* __restrict__ pp_off,
                                                          std::uint16_t* __restrict__ out, int rows, int hidden,
                                                          std::uint32_t tag, std::int32_t* status) {
    pdl_wait();
    pdl_launch_dependents();
    const int quads = hidden / 4;
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= rows * quads) return;
    const int row = v / quads;
    const int q = v - row * quads;
    const std::uint64_t* operand = ret + static_cast<std::size_t>(row) * kTop * kRetRowWords + 2 * q;
    uint4 got[kTop];
    const std::uint64_t start = global_timer_ns();
    while (true) {
        bool missing = false;
#pragma unroll
        for (int slot = 0; slot < kTop; ++slot) got[slot] = ld_tagged_pair(operand + static_cast<std::size_t>(slot) * kRetRowWords);
#pragma unroll
        for (int slot = 0; slot < kTop; ++slot) missing = missing || got[slot].y != tag || got[slot].w != tag;
        if (!missing) break;
        if (expired(start)) {
            atomicCAS(status, kStatusOk, kStatusWaitExpired);
            return;
        }
    }
    float acc[4] = {0.0F, 0.0F, 0.0F, 0.0F};
#pragma unroll
    for (int slot = 0; slot < kTop; ++slot) {
        const float w = route_weights[row * kTop + slot];
        acc[0] = fmaf(__uint_as_float(got[slot].x << 16), w, acc[0]);
        acc[1] = fmaf(__uint_as_float(got[slot].x & 0xffff0000U), w, acc[1]);
        acc[2] = fmaf(__uint_as_float(got[slot].z << 16), w, acc[2]);
        acc[3] = fmaf(__uint_as_float(got[slot].z & 0xffff0000U), w, acc[3]);
    }
    const uint2 sh = *reinterpret_cast<const uint2*>(mixed_pp + static_cast<std::size_t>(pp_off[kExperts] + row) * hidden + 4 * q);
    const float o0 = bf16_bits_to_float(float_to_bf16_bits(acc[0])) + __uint_as_float(sh.x << 16);
    const float o1 = bf16_bits_to_float(float_to_bf16_bits(acc[1])) + __uint_as_float(sh.x & 0xffff0000U);
    const float o2 = bf16_bits_to_float(float_to_bf16_bits(acc[2])) + __uint_as_float(sh.y << 16);
    const float o3 = bf16_bits_to_float(float_to_bf16_bits(acc[3])) + __uint_as_float(sh.y & 0xffff0000U);
    *reinterpret_cast<uint2*>(out + static_cast<std::size_t>(row) * hidden + 4 * q) =
        make_uint2(static_cast<std::uint32_t>(float_to_bf16_bits(o0)) | (static_cast<std::uint32_t>(float_to_bf16_bits(o1)) << 16),
                   static_cast<std::uint32_t>(float_to_bf16_bits(o2)) | (static_cast<std::uint32_t>(float_to_bf16_bits(o3)) << 16));
}

}  // namespace

std::size_t ep_gathered_bytes(int world, int rows_per_gpu) {
    const Regions r(world, rows_per_gpu);
    return r.ret_base + 2 * r.ret_parity;
}

cudaError_t launch_ep_lists(const std::int32_t* recv_counts, int count_stride, int sources, int first_expert, int local,
                            int shared_rows, int tile_rows, p92b_plan* plan, cudaStream_t stream);   // ep.cu

}  // namespace p92b

extern "C" {

int p92b_ep_forward_gathered(p92b_plan* plan, const p92b_bank* bank, p92b_ep_window* window, const uint16_t* input,
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
    // one source: its token count is the batch; several: every slot of every GPU, empty ones marked by their owner
    const int tokens = world == 1 ? rows : world * rpg;
    if (window->bulk) return cudaErrorNotSupported;     // a large-batch window has another layout
    if (!window->connected || !plan->tc_ready || !bank->tc_ready || plan->hidden != 2560 || plan->intermediate != 1024 ||
        bank->view.hidden != 2560 || bank->view.intermediate != 1024 || bank->view.local_experts != local ||
        bank->view.first_expert != window->rank * local || plan->max_rows < tokens) {
        return cudaErrorNotSupported;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const bool pdl = std::getenv("P92B_NO_PDL") == nullptr;
    const int hidden = plan->hidden;
    const int assignments = tokens * kTop;
    const Regions regions(world, rpg);
    const unsigned call = window->epoch++;
    const std::uint32_t tag = call + 1U;
    const int parity = static_cast<int>(call & 1U);
    const std::size_t arrive_offset = window->gathered_base + parity * regions.arrive_parity;
    const std::size_t ret_offset = window->gathered_base + regions.ret_base + parity * regions.ret_parity;
    Peers peers {};
    for (int r = 0; r < world; ++r) peers.base[r] = window->peers[r];
    const std::uint64_t* my_arrive = reinterpret_cast<const std::uint64_t*>(window->local + arrive_offset);
    const std::uint64_t* my_ret = reinterpret_cast<const std::uint64_t*>(window->local + ret_offset);
    plan->last_launches = 0;
    // optional stage timing (p92b_plan_stage_timing): 0 router, 1 push (quantise + stores to every window), 2 routing lists
    // (waits for the ids of the whole batch), 3 placement (waits for the rows), 4 gate/up, 5 down, 6 return + combine
    // (waits for every peer's result rows)
    int stage = 0;
    auto mark = [&]() -> cudaError_t {
        if (!plan->timing) return cudaSuccess;
        return cudaEventRecord(plan->stage_events[stage++], stream);
    };
    if (cudaError_t m = mark(); m != cudaSuccess) return m;

    // router of the home tokens (ids into plan->ids, weights stay in plan->route_weights for the combine)
    // (tensor-core logits with exact repair from 9 rows on: same ids and weights, 20 against 38 µs at 64 to 512 rows)
    cudaError_t st = rows >= router_fast_min_rows()
                         ? launch_router_fast(plan, input, router_weight, correction_bias, rows, routed_scale, stream, pdl)
                         : cudaErrorNotSupported;
    if (st == cudaErrorNotSupported) {
        st = launch_router_logits(input, router_weight, plan->logits, rows, kExperts, hidden, world == 1 && rows == 1, stream, pdl);
        if (st != cudaSuccess) return st;
        st = launch_router_top8(plan->logits, correction_bias, plan->ids, plan->route_weights, rows, routed_scale, stream, pdl);
        plan->last_launches += 2;
    }
    if (st != cudaSuccess) return st;
    if ((st = mark()) != cudaSuccess) return st;
    const int push_threads = std::max(rows * (hidden / 16), rpg * kTop);
    st = launch_kernel(epg_push_kernel, dim3((push_threads + 255) / 256), dim3(256), 0, stream, pdl, input,
                       static_cast<const std::int32_t*>(plan->ids), peers, arrive_offset, window->rank, world, rows, rpg,
                       hidden, 1.0F, tag);
    if (st != cudaSuccess) return st;
    if ((st = mark()) != cudaSuccess) return st;
    // routing lists of this GPU's experts (+ its shared-expert rows) from the ids of the whole batch; a token picks
    // an expert at most once, so no expert has more rows than there are tokens
    const int tile_rows = tc_tile_rows(tokens);
    const std::size_t route_smem = static_cast<std::size_t>(local) * (kMaskWords + 2) * 4;
    st = ensure_dynamic_smem<epg_route_kernel>(static_cast<int>(kExperts * (kMaskWords + 2) * 4));
    if (st != cudaSuccess) return st;
    st = launch_kernel(epg_route_kernel, dim3(1), dim3(kRouteThreads), route_smem, stream, pdl, my_arrive, tokens,
                       bank->view.first_expert, local, rows, tile_rows, tag, plan->counts, plan->pp_off, plan->active,
                       plan->active_count, plan->tile_prefix, plan->pp_of_flat, plan->status);
    if (st != cudaSuccess) return st;
    if ((st = mark()) != cudaSuccess) return st;
    plan->wide_rows = 0;
    const int units = assignments + rows;
    st = launch_kernel(epg_scatter_kernel, dim3((units + 7) / 8), dim3(256), 0, stream, pdl, my_arrive,
                       static_cast<const std::int32_t*>(plan->pp_of_flat), static_cast<const std::int32_t*>(plan->pp_off),
                       assignments, window->rank, rows, rpg, plan->xq_pp, plan->xs_sw, tag, plan->status);
    if (st != cudaSuccess) return st;
    // every kernel of the chain waits for its predecessor before it finishes, so the lists two launches up are
    // complete when the down product looks at them
    if ((st = mark()) != cudaSuccess) return st;
    if ((st = launch_experts_tc(plan, bank, tokens, false, stream, pdl)) != cudaSuccess) return st;
    if ((st = mark()) != cudaSuccess) return st;
    if ((st = launch_experts_tc(plan, bank, tokens, true, stream, pdl)) != cudaSuccess) return st;
    if ((st = mark()) != cudaSuccess) return st;
    st = launch_kernel(epg_return_kernel, dim3((assignments + 7) / 8), dim3(256), 0, stream, pdl,
                       static_cast<const std::uint16_t*>(plan->mixed_pp), static_cast<const std::int32_t*>(plan->pp_of_flat),
                       peers, ret_offset, assignments, rpg, hidden, tag);
    if (st != cudaSuccess) return st;
    st = launch_kernel(epg_combine_kernel, dim3((rows * (hidden / 4) + 255) / 256), dim3(256), 0, stream, pdl, my_ret,
                       static_cast<const float*>(plan->route_weights), static_cast<const std::uint16_t*>(plan->mixed_pp),
                       static_cast<const std::int32_t*>(plan->pp_off), output, rows, hidden, tag, plan->status);
    plan->last_launches += 7;           // behind the router's two or three
    plan->last_path = 2;
    if (st != cudaSuccess) return st;
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
    return st;
}

}  // extern "C"
