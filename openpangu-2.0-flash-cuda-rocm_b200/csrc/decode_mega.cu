// The whole MoE block for up to 16 tokens (decode, MTP verify, small decode batches) as ONE persistent kernel.
//
// At these sizes the block is a 120 MB weight stream (≈19 µs at HBM speed) wrapped in a
// few microseconds of routing, so kernel boundaries - five dependent launches - cost
// as much as the stream itself.  Here one block per SM walks the phases, and what a phase
// needs from other blocks it gets without a device-wide stop:
//
//   P0  every block: its one or two router rows (logits in the reference's exact FP32
//       order, cuda/nvfp4_ops.cu:161-207) and its slice of the token quantisation
//       (cuda/nvfp4_ops.cu:818-841, scales written 128x4-tiled).  Each logit is published
//       as an 8-byte word {value, launch number}; the quantised rows are covered by an
//       arrive-only counter that only the TMA producer lanes wait on, later;
//   P1  every block, redundantly and in shared memory: polls the logit words, top-8 of
//       every token (cuda/nvfp4_ops.cu:357-433), histogram, stable permutation
//       (cuda/nvfp4_grouped.cu:117-132), active-expert list; block 0 also writes the
//       routing products to global memory;
//   P2  gate/up tiles and P3 down tiles through ONE TMA ring and one tcgen05 pipeline
//       (same operand formats as expert_tc.cu).  The token side of gate/up is simply all
//       tokens in token order (N=16 columns cost nothing at M=128), so it does not depend
//       on routing; the epilogue keeps the columns routed to the tile's expert.  A down
//       tile needs the eight gate/up tiles of its expert: per-expert counters, no barrier,
//       and its weights are already in flight while the producer waits.  Tiles are handed
//       out dynamically from one device-wide counter, gate/up tiles first, both in expert
//       order: a block that falls behind simply takes fewer (a gate/up tile is 10 ring
//       stages, a down tile 2, so the tail is fine-grained);
//   P4  weighted combine in slot order + shared expert (cuda/nvfp4_ops.cu:124-142,92-95):
//       the down epilogue publishes its rows as {two BF16, launch number} words and the
//       combining threads poll the words they need, so the combine of a token starts when
//       its last row lands, not when the slowest block is done.
//
// All blocks are co-resident (one per SM, grid = SM count); every wait on a counter, a
// word or an mbarrier is bounded by wall time and ends in a status word, never a hang.
#include "decode_pipeline.cuh"

#include <cstdlib>

namespace p92b {

using namespace ptx;
using namespace decode;

namespace {

constexpr int kMegaThreads = 192;
constexpr int kMegaMaxRows = 16;                   // = kN: the token side of every MMA holds them all; the kernel is built
                                                   // for 8 (the decode sizes, leaner loops) and for 16 rows
constexpr int kN = 16;                             // token columns of every MMA
// a ring stage: the bank's chunk (decode_pipeline.cuh), then two token boxes and two token scale slabs
constexpr int kOffB1 = 38912, kOffSfB0 = 40960, kOffSfB1 = 43008;
constexpr int kStage = 45056;
constexpr int kWeightTx = kChunkBytes;

struct MegaParams {
    BankView bank;
    const std::uint16_t* x;
    const std::uint16_t* router_w;
    const float* bias;
    std::uint16_t* out;
    float* logits;
    std::int32_t* ids;
    float* route_weights;
    std::int32_t* order;
    std::int32_t* position;
    std::int32_t* counts;
    std::int32_t* offsets;
    std::int32_t* pp_of_flat;
    std::uint8_t* xq_tok;          // [16][H/2] token-order NVFP4 rows
    std::uint8_t* xs_tok;          // their scales: one 128-row tile per 4 scale columns
    std::uint8_t* hq;              // [PP][I/2]
    std::uint8_t* hs;              // tiled scales of hq
    std::uint16_t* mixed;          // [PP][H]
    unsigned long long* logits_tagged;   // [8][256] {value, launch number}
    unsigned long long* ret;             // [8][9][1280] {two BF16, launch number}
    unsigned* sync;                // [0]: blocks that have finished P0 (monotonic across launches)
    std::int32_t* gu_done;         // [2][264] by launch parity: gate/up tiles finished per active slot, [257] tile counter
    std::int32_t* status;
    const std::uint16_t* pre_norm_w;     // optional: RMSNorm weight applied to the token rows before anything else
    const std::uint16_t* post_norm_w;    // optional: RMSNorm weight applied to the block's output rows
    unsigned long long* hidden_tagged;   // [8][H/2] {two BF16 of the un-normalised output, launch number} (post-norm only)
    float norm_eps;
    unsigned long long* trace;     // optional [grid][64] %globaltimer stamps per block (null: off)
    unsigned epoch;                // launches of this kernel on the plan before this one
    float routed_scale;
    float quant_scale;
    int rows;
    int hidden;
    int inter;
};

template <int R>
struct Routing {                   // shared-memory copy, identical in every block; R = the build's row limit
    static constexpr int kMaxActive = R * kTop + 1;
    std::int32_t ids[R * kTop];
    float weights[R * kTop];
    std::int32_t rank[R * kTop];          // earlier assignments with the same expert
    std::int32_t less[R * kTop];          // assignments with a smaller expert id
    std::int32_t slot_a[R * kTop];        // active slot of the assignment's expert (1-based)
    std::int32_t active[kMaxActive];                 // expert of an active slot; slot 0 is the shared expert
    std::int32_t slot_rows[kMaxActive];              // rows of an active slot
    std::int32_t pp_tok[kMaxActive][R];   // padded position of (active slot, token), -1 if not routed
    std::int32_t n_active;
    std::uint32_t expert_mask[kExperts];             // tokens routed to each expert
    std::int32_t before[kExperts];                   // assignments with a smaller expert id
    std::int32_t slot_of[kExperts];                  // active slot an expert has (if any token picked it)
    float logits[R * kExperts];
    float bias[kExperts];
};

// One arrival per block on a device-wide counter; whoever needs all blocks to have arrived waits for
// the count itself (wait_counter).
__device__ __forceinline__ void grid_arrive(unsigned* counter) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        fence_proxy_async_all();          // what the block wrote is later read by TMA in other blocks
        atomicAdd(counter, 1U);
    }
}

template <int R>
__global__ void __launch_bounds__(kMegaThreads, 1) moe_decode_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                      const __grid_constant__ CUtensorMap map_h,
                                                                      const MegaParams p) {
    extern __shared__ std::uint8_t smem_raw[];
    __shared__ Routing<R> rt;
    constexpr int kMaxActive = Routing<R>::kMaxActive;
    __shared__ __align__(8) std::uint64_t barrier_words[3 * kStages + 2 * kAccumBuffers];
    __shared__ std::uint32_t tmem_slot_word;
    __shared__ volatile std::uint32_t abort_word;
    __shared__ volatile int tile_queue[kTileQueue];
    __shared__ volatile int first_tile_word;
    __shared__ volatile int rows_ready_word;
    __shared__ float norm_partial[R][8];
    __shared__ float norm_inverse[R];

    const std::uint32_t base = (smem_u32(smem_raw) + 1023U) & ~1023U;
    const std::uint32_t bars = smem_u32(barrier_words);
    auto weight_bar = [&](int s) { return bars + 8U * s; };
    auto token_bar = [&](int s) { return bars + 8U * (kStages + s); };
    auto empty_bar = [&](int s) { return bars + 8U * (2 * kStages + s); };
    auto accum_full = [&](int b) { return bars + 8U * (3 * kStages + b); };
    auto accum_empty = [&](int b) { return bars + 8U * (3 * kStages + kAccumBuffers + b); };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int rows = p.rows;
    const int hidden = p.hidden;
    const int inter = p.inter;
    const int assignments = rows * kTop;
    const int grid = gridDim.x;
    const int block = blockIdx.x;
    const std::uint32_t tag = p.epoch + 1U;                // never 0: fresh scratch reads as "not yet"
    // this launch's counters were zeroed by the launch before (or at plan creation); it zeroes the next one's
    std::int32_t* const done = p.gu_done + (p.epoch & 1U) * 264;
    std::int32_t* const done_next = p.gu_done + ((p.epoch + 1U) & 1U) * 264;
    unsigned* const tile_counter = reinterpret_cast<unsigned*>(done + kExperts + 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(weight_bar(s), 1);
            mbar_init(token_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < kAccumBuffers; ++b) {
            mbar_init(accum_full(b), 1);
            mbar_init(accum_empty(b), 4);
        }
        abort_word = 0;
        fence_mbar_init();
        prefetch_tensormap(&map_x);
        prefetch_tensormap(&map_h);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_slot_word), kTmemCols);
        tmem_relinquish();
    }
    // the router rows and the bias do not depend on the kernel upstream: fetch them before waiting for it
    const int my_experts = block + grid < kExperts ? 2 : (block < kExperts ? 1 : 0);
    std::uint16_t* w_rows = reinterpret_cast<std::uint16_t*>(smem_raw + (base - smem_u32(smem_raw)));
    std::uint16_t* x_rows = w_rows + 2 * hidden;
    const int vec_per_row = hidden / 8;
    // (asynchronous 16-byte copies: the token rows below are requested behind them without waiting for these, so the
    // block pays one round trip to the L2 for both, not two)
    for (int i = threadIdx.x; i < my_experts * vec_per_row; i += kMegaThreads) {
        const int r = i / vec_per_row;
        const int c = i - r * vec_per_row;
        async_copy16(reinterpret_cast<uint4*>(w_rows + r * hidden) + c,
                     reinterpret_cast<const uint4*>(p.router_w + static_cast<std::size_t>(block + r * grid) * hidden) + c);
    }
    for (int e = threadIdx.x; e < kExperts; e += kMegaThreads) async_copy4(&rt.bias[e], p.bias + e);
    pdl_wait();                       // the token rows come from the kernel before this one
    pdl_launch_dependents();
    for (int i = threadIdx.x; i < rows * vec_per_row; i += kMegaThreads) {
        const int r = i / vec_per_row;
        const int c = i - r * vec_per_row;
        async_copy16(reinterpret_cast<uint4*>(x_rows + r * hidden) + c,
                     reinterpret_cast<const uint4*>(p.x + static_cast<std::size_t>(r) * hidden) + c);
    }
    // the first tile number is asked for now and used after the routing, the atomic's latency in between; behind the
    // copies, because the store of its result makes the warp wait for the answer
    if (threadIdx.x == 0) first_tile_word = static_cast<int>(atomicAdd(tile_counter, 1U));
    async_copies_wait();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // RMSNorm, the reference operator's arithmetic (cuda/nvfp4_ops.cu:67-90): 256 chains per row (chain t: elements
    // t, t+256, ... with fmaf), a shuffle-down tree per 32 chains, a second tree over the eight results, then
    // rsqrtf(sum / H + eps).  Eight "virtual warps" of 32 chains per row are dealt to the block's six warps.
    auto row_sum_of_squares = [&](const std::uint16_t* rows_bf16, int n_rows) {
        for (int vw = warp; vw < n_rows * 8; vw += kMegaThreads / 32) {
            const int r = vw >> 3, w8 = vw & 7;
            const std::uint16_t* xr = rows_bf16 + r * hidden;
            float square_sum = 0.0F;
            for (int i = w8 * 32 + lane; i < hidden; i += 256) {
                const float value = bf16_bits_to_float(xr[i]);
                square_sum = fmaf(value, value, square_sum);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) square_sum += __shfl_down_sync(0xffffffffU, square_sum, off);
            if (lane == 0) norm_partial[r][w8] = square_sum;
        }
        __syncthreads();
        for (int r = warp; r < n_rows; r += kMegaThreads / 32) {
            float total = lane < 8 ? norm_partial[r][lane] : 0.0F;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) total += __shfl_down_sync(0xffffffffU, total, off);
            if (lane == 0) norm_inverse[r] = rsqrtf(total / static_cast<float>(hidden) + p.norm_eps);
        }
        __syncthreads();
    };
    if (p.pre_norm_w != nullptr) {
        // every block normalises all token rows for itself, in place in shared memory: from here on the kernel sees
        // the rows the reference's rmsnorm(pre_mlp_norm) would have written (src/model.cpp:211-212,1210-1211)
        row_sum_of_squares(x_rows, rows);
        for (int i = threadIdx.x; i < rows * hidden; i += kMegaThreads) {
            const int r = i / hidden;
            const int c = i - r * hidden;
            x_rows[i] = float_to_bf16_bits(bf16_bits_to_float(x_rows[i]) * norm_inverse[r] *
                                           bf16_bits_to_float(__ldg(p.pre_norm_w + c)));
        }
        __syncthreads();
    }
    const std::uint32_t tmem_base = tmem_slot_word;
    auto stamp = [&](int slot) {
        if (p.trace != nullptr) p.trace[static_cast<std::size_t>(block) * 64 + slot] = global_timer_ns();
    };
    if (threadIdx.x == 0) stamp(0);
    auto give_up = [&](int code) {
        abort_word = 1;
        atomicCAS(p.status, kStatusOk, code);
    };

    // ------------------------------------------------------------------ P0
    {
        if (rows == 1) {
            // T = 1 order: 256 partial chains (thread t: columns t, t+256, ...), a shuffle-down tree
            // per 32 of them, then a tree over the eight results (cuda/nvfp4_ops.cu:38-51,161-176)
            // The block's (router row, group of 32 chains) pairs are dealt to its six warps - one warp per row would walk
            // eight dependent rounds while four warps idle - and a warp per row then adds the eight group sums.
            for (int job = warp; job < my_experts * 8; job += kMegaThreads / 32) {
                const int q = job >> 3, v = job & 7;
                const std::uint16_t* wr = w_rows + q * hidden;
                float partial = 0.0F;
                for (int c = lane + 32 * v; c < hidden; c += 256) {
                    partial = fmaf(bf16_bits_to_float(x_rows[c]), bf16_bits_to_float(wr[c]), partial);
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) partial += __shfl_down_sync(0xffffffffU, partial, off);
                if (lane == 0) norm_partial[q][v] = partial;
            }
            __syncthreads();
            for (int q = warp; q < my_experts; q += kMegaThreads / 32) {
                float value = lane < 8 ? norm_partial[q][lane] : 0.0F;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) value += __shfl_down_sync(0xffffffffU, value, off);
                if (lane == 0) {
                    const int e = block + q * grid;
                    p.logits[e] = value;
                    st_tagged(p.logits_tagged + e, __float_as_uint(value), tag);
                }
            }
        } else {
            // T > 1 order: lane l sums columns l, l+32, ...; shuffle-down tree (cuda/nvfp4_ops.cu:178-207).
            // A warp runs the chains of two tokens against one router row side by side (same order within
            // each chain), so four tokens x two rows are one round of the six warps.
            const int token_pairs = (rows + 1) / 2;
            for (int q = warp; q < my_experts * token_pairs; q += kMegaThreads / 32) {
                const int r = q / token_pairs;
                const int t0 = 2 * (q - r * token_pairs);
                const bool second = t0 + 1 < rows;
                const std::uint16_t* wr = w_rows + r * hidden;
                const std::uint16_t* xa = x_rows + t0 * hidden;
                const std::uint16_t* xb = x_rows + (second ? t0 + 1 : t0) * hidden;
                float va = 0.0F, vb = 0.0F;
#pragma unroll 8
                for (int c = lane; c < hidden; c += 32) {
                    const float wv = bf16_bits_to_float(wr[c]);
                    va = fmaf(bf16_bits_to_float(xa[c]), wv, va);
                    vb = fmaf(bf16_bits_to_float(xb[c]), wv, vb);
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    va += __shfl_down_sync(0xffffffffU, va, off);
                    vb += __shfl_down_sync(0xffffffffU, vb, off);
                }
                if (lane == 0) {
                    const int e = block + r * grid;
                    p.logits[static_cast<std::size_t>(t0) * kExperts + e] = va;
                    st_tagged(p.logits_tagged + t0 * kExperts + e, __float_as_uint(va), tag);
                    if (second) {
                        p.logits[static_cast<std::size_t>(t0 + 1) * kExperts + e] = vb;
                        st_tagged(p.logits_tagged + (t0 + 1) * kExperts + e, __float_as_uint(vb), tag);
                    }
                }
            }
        }
        // token quantisation, one 16-element block per thread, by the blocks at the END of the grid: those
        // have one router row, the others two
        const int blocks16 = hidden / 16;
        const int g = (grid - 1 - block) * kMegaThreads + threadIdx.x;
        if (g < rows * blocks16) {
            const int t = g / blocks16;
            const int b = g - t * blocks16;
            const uint4* src = reinterpret_cast<const uint4*>(x_rows + t * hidden + b * 16);
            const uint4 lo = src[0];
            const uint4 hi = src[1];
            const std::uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            float v[16];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[2 * i] = __uint_as_float(words[i] << 16);
                v[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000U);
            }
            std::uint8_t scale_bits;
            const uint2 packed = quantize_block16(v, p.quant_scale, &scale_bits);
            *reinterpret_cast<uint2*>(p.xq_tok + static_cast<std::size_t>(t) * (hidden / 2) + b * 8) = packed;
            p.xs_tok[static_cast<std::size_t>(b >> 2) * 512 + t * 16 + (b & 3)] = scale_bits;
        }
        if (block == 0) {
            for (int i = threadIdx.x; i <= kExperts + 1; i += kMegaThreads) done_next[i] = 0;
        }
    }
    if (threadIdx.x == 0) stamp(1);
    grid_arrive(p.sync + 0);          // quantised rows and zeroed counters of this block are out

    // ------------------------------------------------------------------ P1
    {
        // logits come from all blocks of this launch: each word is polled until it carries this launch's
        // number.  All of a thread's words are requested before the first is looked at.
        constexpr int kPerThread = (R * kExperts + kMegaThreads - 1) / kMegaThreads;
        uint2 word[kPerThread];
        const std::uint64_t poll_start = global_timer_ns();
        while (true) {
            // every word still missing is requested again in one batch: one round trip per round, not per word
            bool missing = false;
#pragma unroll
            for (int j = 0; j < kPerThread; ++j) {
                const int i = threadIdx.x + j * kMegaThreads;
                if (i < rows * kExperts) word[j] = ld_tagged(p.logits_tagged + i);
            }
#pragma unroll
            for (int j = 0; j < kPerThread; ++j) {
                const int i = threadIdx.x + j * kMegaThreads;
                if (i < rows * kExperts) {
                    if (word[j].y == tag) {
                        rt.logits[i] = __uint_as_float(word[j].x);
                    } else {
                        missing = true;
                    }
                }
            }
            if (!missing) break;
            if (global_timer_ns() - poll_start > 1000000000ULL) {
                give_up(kStatusWaitExpired);
                break;
            }
        }
        // a thread of the last warp (free unless there are six or more tokens) makes sure every block's share of
        // the quantised rows is written before the producer lane asks the TMA for them
        if (threadIdx.x == kMegaThreads - 32) {
            const bool arrived = wait_counter(p.sync + 0, (p.epoch + 1U) * static_cast<unsigned>(grid));
            fence_proxy_async_all();      // ordinary stores of other blocks -> this block's TMA loads
            rows_ready_word = arrived ? 1 : 0;
        }
        for (int i = threadIdx.x; i < kMaxActive * R; i += kMegaThreads) (&rt.pp_tok[0][0])[i] = -1;
        for (int i = threadIdx.x; i < kExperts; i += kMegaThreads) rt.expert_mask[i] = 0U;
        __syncthreads();
    }
    if (threadIdx.x == 0) stamp(2);
    if (!abort_word) {
        for (int t = warp; t < rows; t += kMegaThreads / 32) {
            warp_top8(rt.logits + t * kExperts, rt.bias, rt.ids + t * kTop, rt.weights + t * kTop, p.routed_scale);
        }
        if (threadIdx.x == 0) stamp(13);
        __syncthreads();
        if (threadIdx.x == 0) stamp(14);
        // The ranking law of cuda/nvfp4_grouped.cu:117-132, position = #(smaller expert id) + #(same id,
        // smaller flat index), through one bit mask of tokens per expert (a token picks an expert at most
        // once): popcounts give the ranks, a scan over the 256 experts the offsets and the active slots.
        if (threadIdx.x < assignments) atomicOr(&rt.expert_mask[rt.ids[threadIdx.x]], 1U << (threadIdx.x / kTop));
        __syncthreads();
        if (warp == 0) {
            int count[8], nonempty[8];
            int count_sum = 0, nonempty_sum = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const std::uint32_t m = rt.expert_mask[lane * 8 + i];
                count[i] = __popc(m);
                nonempty[i] = m != 0U;
                count_sum += count[i];
                nonempty_sum += nonempty[i];
            }
            int count_before = count_sum, nonempty_before = nonempty_sum;       // inclusive scans over lanes
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int c = __shfl_up_sync(0xffffffffU, count_before, off);
                const int n = __shfl_up_sync(0xffffffffU, nonempty_before, off);
                if (lane >= off) {
                    count_before += c;
                    nonempty_before += n;
                }
            }
            if (lane == 31) rt.n_active = nonempty_before + 1;
            count_before -= count_sum;
            nonempty_before -= nonempty_sum;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                rt.before[lane * 8 + i] = count_before;
                rt.slot_of[lane * 8 + i] = 1 + nonempty_before;
                count_before += count[i];
                nonempty_before += nonempty[i];
            }
        }
        __syncthreads();
        if (threadIdx.x < assignments) {
            const int i = threadIdx.x;
            const int t = i / kTop;
            const int e = rt.ids[i];
            const std::uint32_t m = rt.expert_mask[e];
            const int my_rank = __popc(m & ((1U << t) - 1U));
            const int slot = rt.slot_of[e];
            rt.rank[i] = my_rank;
            rt.less[i] = rt.before[e];
            rt.slot_a[i] = slot;
            rt.pp_tok[slot][t] = (slot - 1) * kTile + my_rank;
            if (my_rank == 0) {
                rt.active[slot] = e;
                rt.slot_rows[slot] = __popc(m);
            }
        } else if (threadIdx.x == assignments) {
            const int distinct = rt.n_active - 1;
            rt.active[0] = kExperts;
            rt.slot_rows[0] = rows;
            for (int t = 0; t < rows; ++t) rt.pp_tok[0][t] = distinct * kTile + t;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) stamp(3);
    // ------------------------------------------------------------ P2 + P3
    const int gu_tiles = inter / kTile;          // 8
    const int dn_tiles = hidden / kTile;         // 20
    const int gu_kblocks = (hidden / 2) / kKB;   // 10 stages per gate/up tile
    const int dn_stages = (inter / 2) / kKB / 2; // 2 stages per down tile (two K blocks each)
    const int gu_items = abort_word ? 0 : rt.n_active * gu_tiles;
    const int total_items = abort_word ? 0 : rt.n_active * (gu_tiles + dn_tiles);

    if (warp == 0) {
        if (elect_one() && !abort_word) {
            int stage = 0;
            std::uint32_t phase = 0;
            int sequence = 0;
            if (rows_ready_word == 0) give_up(kStatusWaitExpired);
            const std::uint64_t stream_policy = l2_policy_evict_first();     // weights are read once per launch
            int current = first_tile_word;
            while (!abort_word) {
                if (current >= total_items) {
                    // end of work: an empty stage carries the closing entry to the MMA lane
                    if (!mbar_wait(empty_bar(stage), phase ^ 1U)) { give_up(kStatusWaitExpired); break; }
                    tile_queue[sequence % kTileQueue] = -1;
                    mbar_arrive(weight_bar(stage));
                    mbar_arrive(token_bar(stage));
                    break;
                }
                const int following = static_cast<int>(atomicAdd(tile_counter, 1U));
                int kind, slot, m_tile;
                if (current < gu_items) {
                    kind = 0; slot = current / gu_tiles; m_tile = current - slot * gu_tiles;
                } else {
                    const int d = current - gu_items;
                    kind = 1; slot = d / dn_tiles; m_tile = d - slot * dn_tiles;
                }
                const int expert = rt.active[slot];
                const int entry = expert == kExperts ? p.bank.local_experts : expert - p.bank.first_expert;
                const int n_stages = kind == 0 ? gu_kblocks : dn_stages;
                bool tokens_ready = kind == 0;
                bool ok = true;
                for (int s = 0; s < n_stages; ++s) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1U)) { give_up(kStatusWaitExpired); ok = false; break; }
                    const std::uint32_t st = base + stage * kStage;
                    if (s == 0) tile_queue[sequence % kTileQueue] = encode_tile(kind, slot, m_tile);
                    if (sequence == 0 && s < 10) stamp(16 + s);
                    mbar_arrive_expect_tx(weight_bar(stage), kWeightTx);
                    if (kind == 0) {
                        bulk_load_hint(st, p.bank.g13 + ((static_cast<std::size_t>(entry) * gu_tiles + m_tile) * gu_kblocks + s) *
                                                            kChunkBytes,
                                       kChunkBytes, weight_bar(stage), stream_policy);
                        mbar_arrive_expect_tx(token_bar(stage), 2 * kSlab);
                        tma_load_2d(st + kOffB0, &map_x, token_bar(stage), s * kKB, 0);
                        bulk_load(st + kOffSfB0, p.xs_tok + static_cast<std::size_t>(s * 4) * 512, kSlab, token_bar(stage));
                    } else {
                        bulk_load_hint(st, p.bank.g2 + ((static_cast<std::size_t>(entry) * dn_tiles + m_tile) * dn_stages + s) *
                                                           kChunkBytes,
                                       kChunkBytes, weight_bar(stage), stream_policy);
                        if (!tokens_ready) {
                            // the SwiGLU rows of this expert exist once its eight gate/up tiles are done
                            if (!wait_counter(reinterpret_cast<const unsigned*>(done + slot),
                                              static_cast<unsigned>(gu_tiles))) {
                                give_up(kStatusWaitExpired);
                                ok = false;
                                break;
                            }
                            fence_proxy_async_all();
                            tokens_ready = true;
                        }
                        const int pp0 = slab_of_slot(slot, rt.n_active);
                        mbar_arrive_expect_tx(token_bar(stage), 4 * kSlab);
                        tma_load_2d(st + kOffB0, &map_h, token_bar(stage), (2 * s) * kKB, pp0);
                        tma_load_2d(st + kOffB1, &map_h, token_bar(stage), (2 * s + 1) * kKB, pp0);
                        const std::uint8_t* bsf = p.hs + (static_cast<std::size_t>(pp0 >> 7) * (inter / 64) + (2 * s) * 4) * 512;
                        bulk_load(st + kOffSfB0, bsf, kSlab, token_bar(stage));
                        bulk_load(st + kOffSfB1, bsf + 4 * 512, kSlab, token_bar(stage));
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1U; }
                }
                if (!ok) break;
                if (current < gu_items && following >= gu_items) stamp(4);   // this block's last gate/up tile issued
                ++sequence;
                current = following;
            }
            stamp(5);                                        // all loads issued
        }
    } else if (warp == 1) {
        if (elect_one() && !abort_word) {
            int stage = 0;
            std::uint32_t phase = 0;
            int buffer = 0;
            std::uint32_t accum_phase = 0;              // bit b = phase of buffer b
            constexpr std::uint32_t idesc = idesc_nvf4(kTile, kN);
            const std::uint32_t sf_tmem = tmem_base + kAccumBuffers * kAccumCols;
            int sf_buffer = 0;
            for (int sequence = 0; !abort_word; ++sequence) {
                // the tile's first stage also publishes its queue entry
                if (!mbar_wait(weight_bar(stage), phase) || !mbar_wait(token_bar(stage), phase)) { give_up(kStatusWaitExpired); break; }
                const int code = tile_queue[sequence % kTileQueue];
                if (!mbar_wait(accum_empty(buffer), ((accum_phase >> buffer) & 1U) ^ 1U)) { give_up(kStatusWaitExpired); break; }
                if (code < 0) {
                    mbar_arrive(accum_full(buffer));        // pass the closing entry on to the epilogue warps
                    break;
                }
                int kind, slot, m_tile;
                decode_tile(code, &kind, &slot, &m_tile);
                tc_fence_after();
                const std::uint32_t accum = tmem_base + buffer * kAccumCols;
                const int n_stages = kind == 0 ? gu_kblocks : dn_stages;
                bool ok = true;
                for (int s = 0; s < n_stages; ++s) {
                    if (s > 0 && (!mbar_wait(weight_bar(stage), phase) || !mbar_wait(token_bar(stage), phase))) {
                        give_up(kStatusWaitExpired);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    if (sequence == 0 && s < 10) stamp(26 + s);
                    issue_stage(kind, base + stage * kStage, kOffB1, kOffSfB0, sf_tmem + sf_buffer * kSfColsPerBuffer, accum,
                                idesc, s == 0);
                    tc_commit(empty_bar(stage));
                    if (sequence == 0 && s < 10) stamp(36 + s);
                    sf_buffer ^= 1;
                    if (++stage == kStages) { stage = 0; phase ^= 1U; }
                }
                if (!ok) break;
                tc_commit(accum_full(buffer));
                accum_phase ^= 1U << buffer;
                buffer = (buffer + 1) % kAccumBuffers;
                if (sequence == 0) stamp(6);                 // first tile's MMAs issued
            }
            stamp(8);
        }
    } else if (!abort_word) {
        if (block == 0) {
            // The routing products go to global memory for the caller (ids, weights, permutation,
            // histogram); these four warps would otherwise idle until the first accumulator is ready.
            const int t = threadIdx.x - 64;
            if (t < assignments) {
                const int pos = rt.less[t] + rt.rank[t];
                p.ids[t] = rt.ids[t];
                p.route_weights[t] = rt.weights[t];
                p.order[pos] = t;
                p.position[t] = pos;
                p.pp_of_flat[t] = rt.pp_tok[rt.slot_a[t]][t / kTop];
            }
            if (t < rows) p.pp_of_flat[assignments + t] = rt.pp_tok[0][t];
            for (int e = t; e <= kExperts; e += 128) {
                if (e < kExperts) {
                    p.counts[e] = __popc(rt.expert_mask[e]);
                    p.offsets[e] = rt.before[e];
                } else {
                    p.offsets[e] = assignments;
                }
            }
        }
        const int quarter = warp & 3;
        int buffer = 0;
        std::uint32_t accum_phase = 0;
        for (int sequence = 0; !abort_word; ++sequence) {
            if (!mbar_wait(accum_full(buffer), (accum_phase >> buffer) & 1U)) { give_up(kStatusWaitExpired); break; }
            accum_phase ^= 1U << buffer;
            const int code = tile_queue[sequence % kTileQueue];
            if (code < 0) break;
            int kind, slot, m_tile;
            decode_tile(code, &kind, &slot, &m_tile);
            tc_fence_after();
            const int expert = rt.active[slot];
            const int entry = expert == kExperts ? p.bank.local_experts : expert - p.bank.first_expert;
            const std::uint32_t lane_base = tmem_base + buffer * kAccumCols + (static_cast<std::uint32_t>(quarter * 32) << 16);
            const int row = m_tile * kTile + quarter * 32 + lane;
            if (kind == 0) {
                const float alpha_g = p.bank.alpha[entry * 3 + 0];
                const float alpha_u = p.bank.alpha[entry * 3 + 1];
                const int sf_col = row >> 4;
                std::uint32_t g[16], u[16];
                tmem_load16(lane_base, g);
                tmem_load16(lane_base + kAccumStride, u);
                tmem_load_wait();
#pragma unroll
                for (int n = 0; n < R; ++n) {
                    const int pp_signed = n < rows ? rt.pp_tok[slot][n] : -1;        // warp uniform
                    if (pp_signed < 0) continue;
                    const float gv = bf16_bits_to_float(float_to_bf16_bits(__uint_as_float(g[n]) * alpha_g));
                    const float uv = bf16_bits_to_float(float_to_bf16_bits(__uint_as_float(u[n]) * alpha_u));
                    const float h = bf16_bits_to_float(float_to_bf16_bits((gv / (1.0F + expf(-gv))) * uv));
                    float amax = fabsf(h);
#pragma unroll
                    for (int off = 8; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffU, amax, off));
                    const __nv_fp8_e4m3 scale(amax * (p.quant_scale / 6.0F));
                    const float decoded = static_cast<float>(scale);
                    const float multiplier = decoded == 0.0F ? 0.0F : p.quant_scale / decoded;
                    const float q = h * multiplier;
                    const float q_next = __shfl_xor_sync(0xffffffffU, q, 1);
                    const std::size_t pp = static_cast<std::size_t>(pp_signed);
                    if ((lane & 1) == 0) {
                        p.hq[pp * (inter / 2) + (row >> 1)] =
                            static_cast<std::uint8_t>(__nv_fp4x2_e2m1(make_float2(q, q_next)).__x);
                    }
                    if ((lane & 15) == 0) {
                        p.hs[((pp >> 7) * (inter / 64) + (sf_col >> 2)) * 512 + (pp & 31) * 16 + ((pp >> 5) & 3) * 4 +
                             (sf_col & 3)] = scale.__x;
                    }
                }
                tc_fence_before();
                __threadfence();
                fence_proxy_async_all();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    mbar_arrive(accum_empty(buffer));
                    mbar_arrive(accum_empty(buffer));
                    mbar_arrive(accum_empty(buffer));
                    mbar_arrive(accum_empty(buffer));
                    atomicAdd(done + slot, 1);
                }
            } else {
                const float alpha = p.bank.alpha[entry * 3 + 2];
                const int pp0 = slab_of_slot(slot, rt.n_active);
                std::uint32_t d[16];
                tmem_load16(lane_base, d);
                tmem_load_wait();
                // row n of this expert belongs to its n-th routed token; that token's slot says where the
                // combine expects it (slot 8 = the shared expert)
                int n = 0;
#pragma unroll
                for (int t = 0; t < R; ++t) {
                    if (t >= rows || rt.pp_tok[slot][t] < 0) continue;             // warp uniform
                    int k = kTop;
                    if (slot != 0) {
                        k = 0;
#pragma unroll
                        for (int kk = 1; kk < kTop; ++kk) k = rt.slot_a[t * kTop + kk] == slot ? kk : k;
                    }
                    std::uint32_t value = 0;
#pragma unroll
                    for (int c = 0; c < R; ++c) value = c == n ? d[c] : value;   // d[n] without dynamic indexing
                    value = float_to_bf16_bits(__uint_as_float(value) * alpha);
                    p.mixed[static_cast<std::size_t>(pp0 + n) * hidden + row] = static_cast<std::uint16_t>(value);
                    const std::uint32_t next = __shfl_down_sync(0xffffffffU, value, 1);
                    if ((lane & 1) == 0) st_tagged(p.ret + static_cast<std::size_t>(t * (kTop + 1) + k) * (hidden / 2) + (row >> 1), value | (next << 16), tag);
                    ++n;
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(accum_empty(buffer));
            }
            buffer = (buffer + 1) % kAccumBuffers;
        }
        if (warp == 2 && lane == 0) stamp(9);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0) stamp(10);

    // ------------------------------------------------------------------ P4
    if (abort_word) return;
    // One thread per four output features: eight routed slots in slot order, then the shared expert;
    // each operand is polled until its words carry this launch's number.
    const int quads = hidden / 4;
    for (int v = block * kMegaThreads + threadIdx.x; v < rows * quads; v += grid * kMegaThreads) {
        const int row = v / quads;
        const int q = v - row * quads;
        float acc[4] = {0.0F, 0.0F, 0.0F, 0.0F};
        bool ok = true;
        const unsigned long long* operand = p.ret + static_cast<std::size_t>(row) * (kTop + 1) * (hidden / 2) + 2 * q;
        uint4 got[kTop + 1];                                  // all nine requested before the first is looked at
#pragma unroll
        for (int slot = 0; slot <= kTop; ++slot) got[slot] = ld_tagged_pair(operand + static_cast<std::size_t>(slot) * (hidden / 2));
#pragma unroll
        for (int slot = 0; slot <= kTop; ++slot) {
            if (got[slot].y != tag || got[slot].w != tag) {
                ok = ok && poll_tagged_pair(operand + static_cast<std::size_t>(slot) * (hidden / 2), tag, &got[slot].x, &got[slot].z);
            }
        }
#pragma unroll
        for (int slot = 0; slot < kTop; ++slot) {
            const float w = rt.weights[row * kTop + slot];
            const std::uint32_t a0 = got[slot].x, a1 = got[slot].z;
            acc[0] = fmaf(__uint_as_float(a0 << 16), w, acc[0]);
            acc[1] = fmaf(__uint_as_float(a0 & 0xffff0000U), w, acc[1]);
            acc[2] = fmaf(__uint_as_float(a1 << 16), w, acc[2]);
            acc[3] = fmaf(__uint_as_float(a1 & 0xffff0000U), w, acc[3]);
        }
        const std::uint32_t s0 = got[kTop].x, s1 = got[kTop].z;
        if (!ok) {
            give_up(kStatusWaitExpired);
            break;
        }
        const float o0 = bf16_bits_to_float(float_to_bf16_bits(acc[0])) + __uint_as_float(s0 << 16);
        const float o1 = bf16_bits_to_float(float_to_bf16_bits(acc[1])) + __uint_as_float(s0 & 0xffff0000U);
        const float o2 = bf16_bits_to_float(float_to_bf16_bits(acc[2])) + __uint_as_float(s1 << 16);
        const float o3 = bf16_bits_to_float(float_to_bf16_bits(acc[3])) + __uint_as_float(s1 & 0xffff0000U);
        const std::uint32_t w0 = static_cast<std::uint32_t>(float_to_bf16_bits(o0)) | (static_cast<std::uint32_t>(float_to_bf16_bits(o1)) << 16);
        const std::uint32_t w1 = static_cast<std::uint32_t>(float_to_bf16_bits(o2)) | (static_cast<std::uint32_t>(float_to_bf16_bits(o3)) << 16);
        if (p.post_norm_w == nullptr) {
            *reinterpret_cast<uint2*>(p.out + static_cast<std::size_t>(row) * hidden + q * 4) = make_uint2(w0, w1);
        } else {
            unsigned long long* words = p.hidden_tagged + static_cast<std::size_t>(row) * (hidden / 2) + 2 * q;
            st_tagged(words, w0, tag);
            st_tagged(words + 1, w1, tag);
        }
    }
    if (p.post_norm_w != nullptr && block < rows) {
        // rmsnorm(post_mlp_norm) of output row `block` (src/model.cpp:216-217,1215-1216): its values were computed all
        // over the grid; this block collects the row, sums the squares in the operator's order and writes the row out
        std::uint16_t* h_row = reinterpret_cast<std::uint16_t*>(smem_raw + (base - smem_u32(smem_raw)));
        bool ok = true;
        for (int i = threadIdx.x; i < hidden / 2; i += kMegaThreads) {
            std::uint32_t pair = 0;
            ok = poll_tagged(p.hidden_tagged + static_cast<std::size_t>(block) * (hidden / 2) + i, tag, &pair) && ok;
            reinterpret_cast<std::uint32_t*>(h_row)[i] = pair;
        }
        if (!ok) give_up(kStatusWaitExpired);
        __syncthreads();
        row_sum_of_squares(h_row, 1);
        const float inverse = norm_inverse[0];
        for (int i = threadIdx.x; i < hidden; i += kMegaThreads) {
            p.out[static_cast<std::size_t>(block) * hidden + i] =
                float_to_bf16_bits(bf16_bits_to_float(h_row[i]) * inverse * bf16_bits_to_float(__ldg(p.post_norm_w + i)));
        }
    }
    if (threadIdx.x == 0) stamp(12);
}

constexpr int kMegaSmem = kStages * kStage + 1024;

}  // namespace

int decode_mega_max_rows() { return kMegaMaxRows; }

cudaError_t launch_decode_mega(p92b_plan* plan, const p92b_bank* bank, const std::uint16_t* x,
                               const std::uint16_t* router_w, const float* bias, std::uint16_t* out, int rows,
                               float routed_scale, cudaStream_t stream, bool pdl, const std::uint16_t* pre_norm_w,
                               const std::uint16_t* post_norm_w, float norm_eps) {
    if (!plan->tc_ready || !bank->tc_ready || rows <= 0 || rows > kMegaMaxRows || plan->hidden != 2560 ||
        plan->intermediate != 1024) {
        return cudaErrorNotSupported;
    }
    const bool wide = rows > 8;
    if (cudaError_t st = wide ? ensure_dynamic_smem<moe_decode_kernel<16>>(kMegaSmem) : ensure_dynamic_smem<moe_decode_kernel<8>>(kMegaSmem);
        st != cudaSuccess) {
        return st;
    }
    MegaParams p {};
    p.bank = bank->view;
    p.x = x;
    p.router_w = router_w;
    p.bias = bias;
    p.out = out;
    p.logits = plan->logits;
    p.ids = plan->ids;
    p.route_weights = plan->route_weights;
    p.order = plan->order;
    p.position = plan->position;
    p.counts = plan->counts;
    p.offsets = plan->offsets;
    p.pp_of_flat = plan->pp_of_flat;
    p.xq_tok = plan->xq_tok;
    p.xs_tok = plan->xs_tok;
    p.hq = plan->hq_pp;
    p.hs = plan->hs_sw;
    p.mixed = plan->mixed_pp;
    p.logits_tagged = plan->mega_logits;
    p.ret = plan->mega_ret;
    p.sync = plan->mega_sync;
    p.gu_done = plan->gu_done;
    p.status = plan->status;
    p.pre_norm_w = pre_norm_w;
    p.post_norm_w = post_norm_w;
    p.hidden_tagged = plan->mega_hidden;
    p.norm_eps = norm_eps;
    p.trace = plan->trace_on ? plan->mega_trace : nullptr;
    p.epoch = plan->mega_epoch++;
    p.routed_scale = routed_scale;
    p.quant_scale = 1.0F;
    p.rows = rows;
    p.hidden = plan->hidden;
    p.inter = plan->intermediate;
    plan->last_launches += 1;
    return wide ? launch_kernel(moe_decode_kernel<16>, dim3(plan->sm_count), dim3(kMegaThreads), kMegaSmem, stream, pdl,
                                plan->map_x_tok, plan->map_h[0], p)
                : launch_kernel(moe_decode_kernel<8>, dim3(plan->sm_count), dim3(kMegaThreads), kMegaSmem, stream, pdl,
                                plan->map_x_tok, plan->map_h[0], p);
}

}  // namespace p92b
