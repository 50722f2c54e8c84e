// Expert-parallel MoE block for small batches (decode, MTP verify) as ONE persistent kernel per GPU,
// the two exchanges done by the kernel itself with stores into the peers' memory over NVLink.
//
// At a handful of tokens per GPU the exchanges carry a few kilobytes; what they cost is latency: a
// library all-to-all is a launch of its own, and around it sit the launches that pack and unpack
// its buffers.  Here the layer is one launch per GPU and the fabric is used the way the sizes ask:
//
//   dispatch = all-gather.  Every GPU pushes its (at most 8) quantised token rows and their top-8
//       expert ids into every peer's window (≈1.5 KB per token and peer), then raises a flag there.
//       With all tokens of the batch present, a GPU runs the single-GPU law restricted to its own
//       experts: per expert the rows are ordered by global token index (home GPU, token), which is
//       the order one GPU would give them (cuda/nvfp4_grouped.cu:117-132).
//   combine = direct placement.  The down product's epilogue stores each BF16 row straight into the
//       home GPU's window at [token][slot]; when all tiles of a GPU are done it raises a flag at
//       every home.  The home GPU then applies the device law in slot order and adds its shared
//       expert (cuda/nvfp4_ops.cu:124-142,92-95).
//
// Inside a GPU the phases are those of the single-GPU decode kernel (decode_mega.cu): router rows
// and token quantisation spread over the grid (logits published as tagged words, no device-wide
// stop), routing lists in shared memory, gate/up and down tiles through one TMA ring and one
// tcgen05 pipeline, tiles handed out from a device-wide counter.  The token side of every MMA is
// the whole gathered batch (16 or 32 columns).  The one device-wide rendezvous left is the one
// behind which the gathered rows are complete in the layout the TMA reads.
//
// Nothing that crosses NVLink is ordered by a fence (a system-scope fence costs about 5 µs here, more
// than the rest of an exchange).  Every word that travels is 8 bytes, {4 bytes of payload, the launch
// number}, stored whole; a reader polls the word itself until the launch number is the one it waits
// for.  So there are no flags and nothing is ever reset; the windows are double-buffered by launch
// parity, and a GPU cannot be more than one launch ahead of any peer (it needs the peer's results of
// launch k to finish launch k), which is what makes two buffers enough.  Every wait - on a peer's
// word, a device-wide counter or an mbarrier - is bounded by wall time and ends in a status word.
#include "decode_pipeline.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <new>

namespace p92b {

using namespace ptx;
using namespace decode;

namespace {

constexpr int kEpThreads = 192;
constexpr int kEpMaxLocalRows = 8;                 // home tokens per GPU
constexpr int kEpMaxTokens = 32;                   // gathered batch (all GPUs)
constexpr int kEpMaxWorld = 16;
constexpr int kMaxSlots = kExperts + 1;            // local experts (all 256 on a single GPU) + the shared expert

// ---- window layout (identical on every GPU) --------------------------------------------------
// arrivals: per parity and global token 368 tagged words = 8 expert ids, 320 words of E2M1 row, 40 of scales
constexpr int kTokIdWords = kTop, kTokRowWords = 320, kTokScaleWords = 40;
constexpr int kTokWords = kTokIdWords + kTokRowWords + kTokScaleWords;
constexpr std::size_t kWinArrive = 0;                                       // u64 [2][32][368]
constexpr std::size_t kWinArriveParity = static_cast<std::size_t>(kEpMaxTokens) * kTokWords * 8;
// the same rows untagged, in the layouts the tensor-core pipeline loads (written by this GPU itself)
constexpr std::size_t kXqRow = 1280;
constexpr std::size_t kWinXq = kWinArrive + 2 * kWinArriveParity;           // [2][32][1280]
constexpr std::size_t kWinXqParity = kEpMaxTokens * kXqRow;
constexpr std::size_t kWinXs = kWinXq + 2 * kWinXqParity;                   // [2][40][512]
constexpr std::size_t kWinXsParity = 40 * 512;
// results: per parity, home token and slot (8 routed + the shared expert) 1280 tagged words of two BF16
constexpr int kRetSlots = kTop + 1;
constexpr int kRetRowWords = 1280;
constexpr std::size_t kWinRet = kWinXs + 2 * kWinXsParity;                  // u64 [2][8][9][1280]
constexpr std::size_t kWinRetParity = static_cast<std::size_t>(kEpMaxLocalRows) * kRetSlots * kRetRowWords * 8;
constexpr std::size_t kWinBytes = kWinRet + 2 * kWinRetParity;
static_assert(kWinXq % 256 == 0 && kWinXs % 16 == 0 && kWinRet % 16 == 0, "window regions must keep their alignment");

struct EpParams {
    BankView bank;
    const std::uint16_t* x;
    const std::uint16_t* router_w;
    const float* bias;
    std::uint16_t* out;
    float* logits;
    std::int32_t* ids;
    float* route_weights;
    std::int32_t* counts;
    std::uint8_t* hq;
    std::uint8_t* hs;
    unsigned long long* logits_tagged;   // [8][256] {value, launch number on this plan}
    unsigned* sync;                // device-wide arrival counter of the plan (monotonic across launches)
    std::int32_t* gu_done;         // [2][264] by launch parity: gate/up tiles finished per active slot, [257] tile counter
    std::int32_t* status;
    unsigned long long* trace;
    std::uint8_t* win[kEpMaxWorld];
    unsigned epoch;                // launches of this kernel on the plan before this one
    unsigned wepoch;               // launches on the window before this one (same on every GPU)
    float routed_scale;
    float quant_scale;
    int rows;                      // this GPU's home tokens
    int rank, world, rows_per_gpu;
    int hidden, inter;
};

struct Routing {
    std::int32_t ids[kEpMaxTokens * kTop];           // gathered, [global token][slot]
    std::uint32_t expert_mask[kMaxSlots];            // local expert -> tokens routed to it; [local] = shared
    std::uint32_t slot_mask[kMaxSlots];              // active slot -> tokens
    std::int32_t active[kMaxSlots];                  // active slot -> bank entry; slot 0 is the shared expert
    std::int32_t n_active;
    float weights[kEpMaxLocalRows * kTop];           // home tokens only
    std::int32_t my_ids[kEpMaxLocalRows * kTop];
    float logits[kEpMaxLocalRows * kExperts];
    float bias[kExperts];
};

template <int kN>
struct StageLayout {
    static constexpr int kOffB1 = kOffB0 + kN * kKB;
    static constexpr int kOffSfB0 = kOffB0 + 2 * kN * kKB;
    static constexpr int kOffSfB1 = kOffSfB0 + kSlab;
    static constexpr int kStage = kOffSfB0 + 2 * kSlab;
    static constexpr int kSmem = kStages * kStage + 1024;
};

template <int kN>
__global__ void __launch_bounds__(kEpThreads, 1) moe_decode_ep_kernel(const __grid_constant__ CUtensorMap map_tok,
                                                                      const __grid_constant__ CUtensorMap map_h,
                                                                      const EpParams p) {
    using L = StageLayout<kN>;
    extern __shared__ std::uint8_t smem_raw[];
    __shared__ Routing rt;
    __shared__ __align__(8) std::uint64_t barrier_words[3 * kStages + 2 * kAccumBuffers];
    __shared__ std::uint32_t tmem_slot_word;
    __shared__ volatile std::uint32_t abort_word;
    __shared__ volatile int tile_queue[kTileQueue];
    __shared__ volatile int first_tile_word;

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
    const int grid = gridDim.x;
    const int block = blockIdx.x;
    const int world = p.world;
    const int rpg = p.rows_per_gpu;
    const int parity = static_cast<int>(p.wepoch & 1U);
    const std::uint32_t tag = p.wepoch + 1U;               // never 0: a fresh window reads as "not yet"
    const std::uint32_t plan_tag = p.epoch + 1U;           // for words that stay on this GPU (the plan's scratch)
    // this launch's counters were zeroed by the launch before (or at plan creation); it zeroes the next one's
    std::int32_t* const done = p.gu_done + (p.epoch & 1U) * 264;
    std::int32_t* const done_next = p.gu_done + ((p.epoch + 1U) & 1U) * 264;
    unsigned* const tile_counter = reinterpret_cast<unsigned*>(done + kExperts + 1);
    std::uint8_t* const my_win = p.win[p.rank];

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
        prefetch_tensormap(&map_tok);
        prefetch_tensormap(&map_h);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_slot_word), kTmemCols);
        tmem_relinquish();
    }
    // router rows and bias do not depend on the kernel upstream
    const int my_experts = block + grid < kExperts ? 2 : (block < kExperts ? 1 : 0);
    std::uint16_t* w_rows = reinterpret_cast<std::uint16_t*>(smem_raw + (base - smem_u32(smem_raw)));
    std::uint16_t* x_rows = w_rows + 2 * hidden;
    const int vec_per_row = hidden / 8;
    for (int i = threadIdx.x; i < my_experts * vec_per_row; i += kEpThreads) {
        const int r = i / vec_per_row;
        const int c = i - r * vec_per_row;
        async_copy16(reinterpret_cast<uint4*>(w_rows + r * hidden) + c,
                     reinterpret_cast<const uint4*>(p.router_w + static_cast<std::size_t>(block + r * grid) * hidden) + c);
    }
    for (int e = threadIdx.x; e < kExperts; e += kEpThreads) async_copy4(&rt.bias[e], p.bias + e);
    pdl_wait();
    pdl_launch_dependents();
    for (int i = threadIdx.x; i < rows * vec_per_row; i += kEpThreads) {
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
    const std::uint32_t tmem_base = tmem_slot_word;
    auto stamp = [&](int slot) {
        if (p.trace != nullptr) p.trace[static_cast<std::size_t>(block) * 64 + slot] = global_timer_ns();
    };
    if (threadIdx.x == 0) stamp(0);
    auto give_up = [&](int code) {
        abort_word = 1;
        atomicCAS(p.status, kStatusOk, code);
    };

    // ------------------------------------------------------------------ P0: home tokens
    {
        // More than one token is in flight across the GPUs, so the router uses the batched order
        // (lane l sums columns l, l+32, ...; shuffle-down tree: cuda/nvfp4_ops.cu:178-207) - unless
        // this is the only GPU and it has one token, which is the single-token law (:161-176).
        if (world == 1 && rows == 1) {
            for (int q = warp; q < my_experts; q += kEpThreads / 32) {
                const std::uint16_t* wr = w_rows + q * hidden;
                float value = 0.0F;
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    float partial = 0.0F;
                    for (int c = lane + 32 * v; c < hidden; c += 256) {
                        partial = fmaf(bf16_bits_to_float(x_rows[c]), bf16_bits_to_float(wr[c]), partial);
                    }
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) partial += __shfl_down_sync(0xffffffffU, partial, off);
                    const float warp_sum = __shfl_sync(0xffffffffU, partial, 0);
                    if (lane == v) value = warp_sum;
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) value += __shfl_down_sync(0xffffffffU, value, off);
                if (lane == 0) {
                    p.logits[block + q * grid] = value;
                    st_tagged(p.logits_tagged + block + q * grid, __float_as_uint(value), plan_tag);
                }
            }
        } else {
            // a warp runs the chains of two tokens against one router row side by side (same order within
            // each chain)
            const int token_pairs = (rows + 1) / 2;
            for (int q = warp; q < my_experts * token_pairs; q += kEpThreads / 32) {
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
                    st_tagged(p.logits_tagged + t0 * kExperts + e, __float_as_uint(va), plan_tag);
                    if (second) {
                        p.logits[static_cast<std::size_t>(t0 + 1) * kExperts + e] = vb;
                        st_tagged(p.logits_tagged + (t0 + 1) * kExperts + e, __float_as_uint(vb), plan_tag);
                    }
                }
            }
        }
        // (the blocks at the END of the grid quantise: those have one router row, the others two)
        const int blocks16 = hidden / 16;
        const int g = (grid - 1 - block) * kEpThreads + threadIdx.x;
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
            // (whole warps take this branch: 160 blocks per row and 192 threads per block are multiples of 32)
            std::uint32_t scales4 = scale_bits;
            scales4 |= __shfl_down_sync(0xffffffffU, static_cast<std::uint32_t>(scale_bits), 1) << 8;
            scales4 |= __shfl_down_sync(0xffffffffU, static_cast<std::uint32_t>(scale_bits), 2) << 16;
            scales4 |= __shfl_down_sync(0xffffffffU, static_cast<std::uint32_t>(scale_bits), 3) << 24;
            // straight into every GPU's window (this one's included): two row words, and from every fourth
            // thread the word of four scales; they travel while the router finishes
            for (int d = 0; d < world; ++d) {
                std::uint64_t* dst = reinterpret_cast<std::uint64_t*>(p.win[d] + kWinArrive + parity * kWinArriveParity) +
                                     static_cast<std::size_t>(p.rank * rpg + t) * kTokWords + kTokIdWords;
                st_tagged(dst + 2 * b, packed.x, tag);
                st_tagged(dst + 2 * b + 1, packed.y, tag);
                if ((b & 3) == 0) st_tagged(dst + kTokRowWords + (b >> 2), scales4, tag);
            }
        } else if (g < rows * blocks16 + (rpg - rows)) {
            // a token slot this GPU does not fill this time: the first word of its row says so (the complement of the
            // launch number can be neither this launch's tag nor an older one), so that the receivers can tell a row that
            // will not come from one that has not come yet without waiting for the ids
            const int t = rows + (g - rows * blocks16);
            for (int d = 0; d < world; ++d) {
                std::uint64_t* dst = reinterpret_cast<std::uint64_t*>(p.win[d] + kWinArrive + parity * kWinArriveParity) +
                                     static_cast<std::size_t>(p.rank * rpg + t) * kTokWords + kTokIdWords;
                st_tagged(dst, 0U, ~tag);
            }
        }
        if (block == 0) {
            for (int i = threadIdx.x; i <= kExperts + 1; i += kEpThreads) done_next[i] = 0;
        }
    }
    if (threadIdx.x == 0) stamp(1);

    // ------------------------------------------------- the batch's rows: tagged words -> the layouts the TMA reads
    // The rows left their GPUs in P0, long before the ids (which need the logits of all blocks and the top-8): the
    // blocks that do not route turn them into the untagged row and scale layouts now, each its share, and count
    // themselves in; the wait for that count sits just before the tiles, by when everybody has long arrived.
    const int tokens = world * rpg;
    const std::uint64_t* arrive = reinterpret_cast<const std::uint64_t*>(my_win + kWinArrive + parity * kWinArriveParity);
    if (!abort_word && (block >= world || grid <= world)) {
        std::uint8_t* xq_dense = my_win + kWinXq + parity * kWinXqParity;
        std::uint8_t* xs_dense = my_win + kWinXs + parity * kWinXsParity;
        const int per_token = kTokRowWords + kTokScaleWords;
        const int copiers = grid > world ? grid - world : grid;
        const int me = grid > world ? block - world : block;
        for (int i = me * kEpThreads + threadIdx.x; i < tokens * per_token; i += copiers * kEpThreads) {
            const int g = i / per_token;
            const int w = i - g * per_token;
            const std::uint64_t* row_words = arrive + static_cast<std::size_t>(g) * kTokWords + kTokIdWords;
            // the slot's first word: this launch's tag (a row) or its complement (no row this time)
            uint2 head = ld_tagged(row_words);
            if (head.y != tag && head.y != ~tag) {
                const std::uint64_t start = global_timer_ns();
                do {
                    if (poll_expired(start)) break;
                    head = ld_tagged(row_words);
                } while (head.y != tag && head.y != ~tag);
            }
            if (head.y == ~tag) continue;
            std::uint32_t word = 0;
            if (head.y != tag || !poll_tagged(row_words + w, tag, &word)) {
                give_up(kStatusWaitExpired);
                break;
            }
            if (w < kTokRowWords) {
                reinterpret_cast<std::uint32_t*>(xq_dense + g * kXqRow)[w] = word;
            } else {
                *reinterpret_cast<std::uint32_t*>(xs_dense + (w - kTokRowWords) * 512 + g * 16) = word;
            }
        }
    }
    // (one arrival per block; what the block wrote is later read by TMA in other blocks)
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        fence_proxy_async_all();
        atomicAdd(p.sync, 1U);
    }
    if (threadIdx.x == 0) stamp(2);

    // ------------------------------------------------- routing of the home tokens: block d tells GPU d
    if (!abort_word && block < world) {
        std::uint64_t* dst = reinterpret_cast<std::uint64_t*>(p.win[block] + kWinArrive + parity * kWinArriveParity) +
                             static_cast<std::size_t>(p.rank * rpg) * kTokWords;
        {
            // the logits come from all blocks: every word still missing is requested again in one batch
            constexpr int kPerThread = (kEpMaxLocalRows * kExperts + kEpThreads - 1) / kEpThreads;
            uint2 word[kPerThread];
            const std::uint64_t poll_start = global_timer_ns();
            while (true) {
                bool missing = false;
#pragma unroll
                for (int j = 0; j < kPerThread; ++j) {
                    const int i = threadIdx.x + j * kEpThreads;
                    if (i < rows * kExperts) word[j] = ld_tagged(p.logits_tagged + i);
                }
#pragma unroll
                for (int j = 0; j < kPerThread; ++j) {
                    const int i = threadIdx.x + j * kEpThreads;
                    if (i < rows * kExperts) {
                        if (word[j].y == plan_tag) {
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
        }
        __syncthreads();
        if (threadIdx.x == 0) stamp(13);
        for (int t = warp; t < rows; t += kEpThreads / 32) {
            warp_top8(rt.logits + t * kExperts, rt.bias, rt.my_ids + t * kTop, rt.weights + t * kTop, p.routed_scale);
        }
        __syncthreads();
        if (threadIdx.x == 0) stamp(14);
        // token slots this GPU does not fill this time say so with id -1
        for (int i = threadIdx.x; i < rpg * kTop; i += kEpThreads) {
            const int t = i / kTop;
            st_tagged(dst + t * kTokWords + (i - t * kTop), static_cast<std::uint32_t>(t < rows ? rt.my_ids[i] : -1), tag);
        }
        if (block == p.rank) {
            for (int i = threadIdx.x; i < rows * kTop; i += kEpThreads) {
                p.ids[i] = rt.my_ids[i];
                p.route_weights[i] = rt.weights[i];
            }
        }
    }
    if (threadIdx.x == 0) stamp(3);

    // ------------------------------------------------- arrivals: ids (every block), rows (one word per thread)
    const int local = p.bank.local_experts;
    for (int i = threadIdx.x; i < kMaxSlots; i += kEpThreads) rt.expert_mask[i] = 0;
    __syncthreads();
    if (!abort_word) {
        for (int a = threadIdx.x; a < tokens * kTop; a += kEpThreads) {
            const int g = a / kTop;
            std::uint32_t word = 0;
            if (!poll_tagged(arrive + static_cast<std::size_t>(g) * kTokWords + (a - g * kTop), tag, &word)) {
                give_up(kStatusWaitExpired);
                break;
            }
            const std::int32_t e = static_cast<std::int32_t>(word);
            const int le = e - p.bank.first_expert;
            if (e >= 0 && le >= 0 && le < local) atomicOr(&rt.expert_mask[le], 1U << g);
            rt.ids[a] = e;
        }
    }
    if (threadIdx.x == 0) {
        rt.expert_mask[local] = ((1U << rows) - 1U) << (p.rank * rpg);
        stamp(4);
    }
    __syncthreads();
    if (!abort_word) {
        // routing lists of this GPU's experts (every block, in shared memory)
        if (warp == 0) {
            int found = 0;
            for (int e0 = 0; e0 < local; e0 += 32) {
                const int e = e0 + lane;
                const std::uint32_t m = e < local ? rt.expert_mask[e] : 0U;
                const unsigned vote = __ballot_sync(0xffffffffU, m != 0U);
                if (m != 0U) {
                    const int slot = 1 + found + __popc(vote & ((1U << lane) - 1U));
                    rt.active[slot] = e;
                    rt.slot_mask[slot] = m;
                }
                found += __popc(vote);
            }
            if (lane == 0) {
                rt.active[0] = local;
                rt.slot_mask[0] = rt.expert_mask[local];
                rt.n_active = found + 1;
            }
        }
        if (block == 0) {
            for (int e = threadIdx.x; e < local; e += kEpThreads) p.counts[p.bank.first_expert + e] = __popc(rt.expert_mask[e]);
        }
    }
    if (threadIdx.x == 0) stamp(5);
    // the untagged batch is complete on this GPU once every block has counted itself in (after P0, above)
    {
        __shared__ int batch_ready;
        if (threadIdx.x == 0) {
            batch_ready = wait_counter(p.sync, (p.epoch + 1U) * static_cast<unsigned>(grid)) ? 1 : 0;
            __threadfence();
            fence_proxy_async_all();
        }
        __syncthreads();
        if (!batch_ready) give_up(kStatusWaitExpired);
    }
    if (threadIdx.x == 0) stamp(6);

    // ------------------------------------------------------------ gate/up and down tiles
    const int gu_tiles = inter / kTile;
    const int dn_tiles = hidden / kTile;
    const int gu_kblocks = (hidden / 2) / kKB;
    const int dn_stages = (inter / 2) / kKB / 2;
    const int gu_items = abort_word ? 0 : rt.n_active * gu_tiles;
    const int total_items = abort_word ? 0 : rt.n_active * (gu_tiles + dn_tiles);
    const int token_row0 = parity * kEpMaxTokens;         // first row of this launch's batch in the token map
    const std::uint8_t* xs_batch = my_win + kWinXs + parity * kWinXsParity;

    if (warp == 0) {
        if (elect_one() && !abort_word) {
            int stage = 0;
            std::uint32_t phase = 0;
            int sequence = 0;
            fence_proxy_async_all();          // the gathered rows were written by ordinary stores
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
                const int entry = rt.active[slot];
                const int n_stages = kind == 0 ? gu_kblocks : dn_stages;
                bool tokens_ready = kind == 0;
                bool ok = true;
                for (int s = 0; s < n_stages; ++s) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1U)) { give_up(kStatusWaitExpired); ok = false; break; }
                    const std::uint32_t st = base + stage * L::kStage;
                    if (s == 0) tile_queue[sequence % kTileQueue] = encode_tile(kind, slot, m_tile);
                    mbar_arrive_expect_tx(weight_bar(stage), kChunkBytes);
                    if (kind == 0) {
                        bulk_load_hint(st, p.bank.g13 + ((static_cast<std::size_t>(entry) * gu_tiles + m_tile) * gu_kblocks + s) *
                                                            kChunkBytes,
                                       kChunkBytes, weight_bar(stage), stream_policy);
                        mbar_arrive_expect_tx(token_bar(stage), kN * kKB + kSlab);
                        tma_load_2d(st + kOffB0, &map_tok, token_bar(stage), s * kKB, token_row0);
                        bulk_load(st + L::kOffSfB0, xs_batch + static_cast<std::size_t>(s * 4) * 512, kSlab, token_bar(stage));
                    } else {
                        bulk_load_hint(st, p.bank.g2 + ((static_cast<std::size_t>(entry) * dn_tiles + m_tile) * dn_stages + s) *
                                                           kChunkBytes,
                                       kChunkBytes, weight_bar(stage), stream_policy);
                        if (!tokens_ready) {
                            if (!wait_counter(reinterpret_cast<const unsigned*>(done + slot), static_cast<unsigned>(gu_tiles))) {
                                give_up(kStatusWaitExpired);
                                ok = false;
                                break;
                            }
                            fence_proxy_async_all();
                            tokens_ready = true;
                        }
                        const int pp0 = slab_of_slot(slot, rt.n_active);
                        mbar_arrive_expect_tx(token_bar(stage), 2 * kN * kKB + 2 * kSlab);
                        tma_load_2d(st + kOffB0, &map_h, token_bar(stage), (2 * s) * kKB, pp0);
                        tma_load_2d(st + L::kOffB1, &map_h, token_bar(stage), (2 * s + 1) * kKB, pp0);
                        const std::uint8_t* bsf = p.hs + (static_cast<std::size_t>(pp0 >> 7) * (inter / 64) + (2 * s) * 4) * 512;
                        bulk_load(st + L::kOffSfB0, bsf, kSlab, token_bar(stage));
                        bulk_load(st + L::kOffSfB1, bsf + 4 * 512, kSlab, token_bar(stage));
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1U; }
                }
                if (!ok) break;
                ++sequence;
                current = following;
            }
            stamp(7);
        }
    } else if (warp == 1) {
        if (elect_one() && !abort_word) {
            int stage = 0;
            std::uint32_t phase = 0;
            int buffer = 0;
            std::uint32_t accum_phase = 0;
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
                    issue_stage(kind, base + stage * L::kStage, L::kOffB1, L::kOffSfB0, sf_tmem + sf_buffer * kSfColsPerBuffer,
                                accum, idesc, s == 0);
                    tc_commit(empty_bar(stage));
                    sf_buffer ^= 1;
                    if (++stage == kStages) { stage = 0; phase ^= 1U; }
                }
                if (!ok) break;
                tc_commit(accum_full(buffer));
                accum_phase ^= 1U << buffer;
                buffer = (buffer + 1) % kAccumBuffers;
            }
            stamp(8);
        }
    } else if (!abort_word) {
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
            const int entry = rt.active[slot];
            const std::uint32_t mask = rt.slot_mask[slot];
            const int pp0 = slab_of_slot(slot, rt.n_active);
            const std::uint32_t lane_base = tmem_base + buffer * kAccumCols + (static_cast<std::uint32_t>(quarter * 32) << 16);
            const int row = m_tile * kTile + quarter * 32 + lane;
            if (kind == 0) {
                const float alpha_g = p.bank.alpha[entry * 3 + 0];
                const float alpha_u = p.bank.alpha[entry * 3 + 1];
                const int sf_col = row >> 4;
#pragma unroll
                for (int c = 0; c < kN / 16; ++c) {
                    if ((mask >> (16 * c) & 0xffffU) == 0U) continue;                 // warp uniform
                    std::uint32_t g[16], u[16];
                    tmem_load16(lane_base + 16 * c, g);
                    tmem_load16(lane_base + kAccumStride + 16 * c, u);
                    tmem_load_wait();
#pragma unroll
                    for (int n = 0; n < 16; ++n) {
                        const int token = 16 * c + n;
                        if (!(mask >> token & 1U)) continue;                          // warp uniform
                        const std::size_t pp = static_cast<std::size_t>(pp0 + __popc(mask & ((1U << token) - 1U)));
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
                        if ((lane & 1) == 0) {
                            p.hq[pp * (inter / 2) + (row >> 1)] =
                                static_cast<std::uint8_t>(__nv_fp4x2_e2m1(make_float2(q, q_next)).__x);
                        }
                        if ((lane & 15) == 0) {
                            p.hs[((pp >> 7) * (inter / 64) + (sf_col >> 2)) * 512 + (pp & 31) * 16 + ((pp >> 5) & 3) * 4 +
                                 (sf_col & 3)] = scale.__x;
                        }
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
                const int expert = p.bank.first_expert + entry;
                std::uint32_t remaining = mask;
#pragma unroll
                for (int c = 0; c < kN / 16; ++c) {
                    if (remaining == 0U) break;                                       // warp uniform
                    std::uint32_t d[16];
                    tmem_load16(lane_base + 16 * c, d);
                    tmem_load_wait();
#pragma unroll
                    for (int n = 0; n < 16; ++n) {
                        if (remaining == 0U) continue;
                        // column 16c+n is the (16c+n)-th row of this expert = its (16c+n)-th token
                        const int token = __ffs(remaining) - 1;
                        remaining &= remaining - 1U;
                        const std::uint32_t value = float_to_bf16_bits(__uint_as_float(d[n]) * alpha);
                        const std::uint32_t next = __shfl_down_sync(0xffffffffU, value, 1);
                        const int home = token / rpg;
                        const int t_local = token - home * rpg;
                        int k = kTop;                                                 // the shared expert's slot
                        if (slot != 0) {
                            k = 0;
#pragma unroll
                            for (int kk = 1; kk < kTop; ++kk) k = rt.ids[token * kTop + kk] == expert ? kk : k;
                        }
                        // two output features per word: even lanes store {own | next << 16, launch number}
                        if ((lane & 1) == 0) {
                            std::uint64_t* ret = reinterpret_cast<std::uint64_t*>(p.win[home] + kWinRet + parity * kWinRetParity) +
                                                 static_cast<std::size_t>(t_local * kRetSlots + k) * kRetRowWords;
                            st_tagged(ret + (row >> 1), value | (next << 16), tag);
                        }
                    }
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

    if (abort_word) return;

    // ------------------------------------------------------------------ combine (home tokens)
    // One thread per four output features: eight routed slots in slot order, then the shared expert;
    // each operand is polled until its words carry this launch's number.
    const std::uint64_t* ret = reinterpret_cast<const std::uint64_t*>(my_win + kWinRet + parity * kWinRetParity);
    const int quads = hidden / 4;
    for (int v = block * kEpThreads + threadIdx.x; v < rows * quads; v += grid * kEpThreads) {
        const int row = v / quads;
        const int q = v - row * quads;
        float acc[4] = {0.0F, 0.0F, 0.0F, 0.0F};
        bool ok = true;
#pragma unroll
        for (int slot = 0; slot < kTop; ++slot) {
            const float w = __ldcg(p.route_weights + row * kTop + slot);
            std::uint32_t a0, a1;
            ok = ok && poll_tagged_pair(ret + static_cast<std::size_t>(row * kRetSlots + slot) * kRetRowWords + 2 * q, tag, &a0, &a1);
            acc[0] = fmaf(__uint_as_float(a0 << 16), w, acc[0]);
            acc[1] = fmaf(__uint_as_float(a0 & 0xffff0000U), w, acc[1]);
            acc[2] = fmaf(__uint_as_float(a1 << 16), w, acc[2]);
            acc[3] = fmaf(__uint_as_float(a1 & 0xffff0000U), w, acc[3]);
        }
        std::uint32_t s0, s1;
        ok = ok && poll_tagged_pair(ret + static_cast<std::size_t>(row * kRetSlots + kTop) * kRetRowWords + 2 * q, tag, &s0, &s1);
        if (!ok) {
            give_up(kStatusWaitExpired);
            break;
        }
        const float o0 = bf16_bits_to_float(float_to_bf16_bits(acc[0])) + __uint_as_float(s0 << 16);
        const float o1 = bf16_bits_to_float(float_to_bf16_bits(acc[1])) + __uint_as_float(s0 & 0xffff0000U);
        const float o2 = bf16_bits_to_float(float_to_bf16_bits(acc[2])) + __uint_as_float(s1 << 16);
        const float o3 = bf16_bits_to_float(float_to_bf16_bits(acc[3])) + __uint_as_float(s1 & 0xffff0000U);
        *reinterpret_cast<uint2*>(p.out + static_cast<std::size_t>(row) * hidden + q * 4) =
            make_uint2(static_cast<std::uint32_t>(float_to_bf16_bits(o0)) | (static_cast<std::uint32_t>(float_to_bf16_bits(o1)) << 16),
                       static_cast<std::uint32_t>(float_to_bf16_bits(o2)) | (static_cast<std::uint32_t>(float_to_bf16_bits(o3)) << 16));
    }
    if (threadIdx.x == 0) stamp(12);
}

}  // namespace

}  // namespace p92b

// ---- the window object ---------------------------------------------------------------------------
namespace p92b {
std::size_t ep_gathered_bytes(int world, int rows_per_gpu);      // ep_gathered.cu
}

extern "C" {

int p92b_ep_window_create(p92b_ep_window** out, int rank, int world, int rows_per_gpu) {
    using namespace p92b;
    if (out == nullptr) return cudaErrorInvalidValue;
    *out = nullptr;
    if (world <= 0 || world > kEpMaxWorld || rank < 0 || rank >= world || kExperts % world != 0 || rows_per_gpu <= 0 ||
        rows_per_gpu > 512 || world * rows_per_gpu > 1024) {
        return cudaErrorInvalidValue;
    }
    p92b_ep_window* w = new (std::nothrow) p92b_ep_window();
    if (w == nullptr) return cudaErrorMemoryAllocation;
    w->rank = rank;
    w->world = world;
    w->rows_per_gpu = rows_per_gpu;
    w->fused_ok = rows_per_gpu <= kEpMaxLocalRows && world * rows_per_gpu <= kEpMaxTokens;
    w->gathered_base = (kWinBytes + 255) / 256 * 256;
    w->bytes = w->gathered_base + ep_gathered_bytes(world, rows_per_gpu);
    cudaError_t st = cudaMalloc(reinterpret_cast<void**>(&w->local), w->bytes);
    if (st == cudaSuccess) st = cudaMemset(w->local, 0, w->bytes);
    if (st == cudaSuccess) st = cudaDeviceSynchronize();
    bool ok = st == cudaSuccess;
    ok = ok && make_operand_map(&w->map_tok[0], w->local + kWinXq, 2 * kEpMaxTokens, kXqRow, 16) == cudaSuccess;
    ok = ok && make_operand_map(&w->map_tok[1], w->local + kWinXq, 2 * kEpMaxTokens, kXqRow, 32) == cudaSuccess;
    if (!ok) {
        if (w->local != nullptr) cudaFree(w->local);
        delete w;
        return st != cudaSuccess ? st : cudaErrorNotSupported;
    }
    w->peers[rank] = w->local;
    w->connected = world == 1;
    *out = w;
    return cudaSuccess;
}

size_t p92b_ep_window_bytes(const p92b_ep_window* window) { return window == nullptr ? 0 : window->bytes; }

int p92b_ep_window_handle(const p92b_ep_window* window, uint8_t* handle64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "inter-process handle size");
    if (window == nullptr || handle64 == nullptr) return cudaErrorInvalidValue;
    cudaIpcMemHandle_t handle;
    const cudaError_t st = cudaIpcGetMemHandle(&handle, window->local);
    if (st != cudaSuccess) return st;
    std::memcpy(handle64, &handle, 64);
    return cudaSuccess;
}

int p92b_ep_window_connect(p92b_ep_window* window, const uint8_t* handles) {
    if (window == nullptr || (window->world > 1 && handles == nullptr)) return cudaErrorInvalidValue;
    if (window->connected) return cudaSuccess;
    for (int r = 0; r < window->world; ++r) {
        if (r == window->rank) continue;
        cudaIpcMemHandle_t handle;
        std::memcpy(&handle, handles + static_cast<size_t>(r) * 64, 64);
        void* ptr = nullptr;
        const cudaError_t st = cudaIpcOpenMemHandle(&ptr, handle, cudaIpcMemLazyEnablePeerAccess);
        if (st != cudaSuccess) return st;
        window->peers[r] = static_cast<std::uint8_t*>(ptr);
        window->opened[r] = true;
    }
    window->connected = true;
    return cudaSuccess;
}

int p92b_ep_window_connect_local(p92b_ep_window* window, p92b_ep_window* const* all_windows) {
    if (window == nullptr || all_windows == nullptr) return cudaErrorInvalidValue;
    for (int r = 0; r < window->world; ++r) {
        if (all_windows[r] == nullptr || all_windows[r]->world != window->world || all_windows[r]->rank != r ||
            all_windows[r]->rows_per_gpu != window->rows_per_gpu) {
            return cudaErrorInvalidValue;
        }
    }
    for (int r = 0; r < window->world; ++r) window->peers[r] = all_windows[r]->local;
    window->connected = true;
    return cudaSuccess;
}

void p92b_ep_window_destroy(p92b_ep_window* window) {
    if (window == nullptr) return;
    for (int r = 0; r < window->world; ++r) {
        if (window->opened[r]) cudaIpcCloseMemHandle(window->peers[r]);
    }
    if (window->local != nullptr) cudaFree(window->local);
    delete window;
}

int p92b_ep_forward_fused(p92b_plan* plan, const p92b_bank* bank, p92b_ep_window* window, const uint16_t* input,
                          const uint16_t* router_weight, const float* correction_bias, uint16_t* output, int rows,
                          float routed_scale, void* stream_) {
    using namespace p92b;
    if (plan == nullptr || bank == nullptr || window == nullptr || input == nullptr || router_weight == nullptr ||
        correction_bias == nullptr || output == nullptr || rows <= 0 || rows > window->rows_per_gpu) {
        return cudaErrorInvalidValue;
    }
    if (window->bulk) return cudaErrorNotSupported;     // a large-batch window has another layout
    if (!window->connected || !window->fused_ok || !plan->tc_ready || !bank->tc_ready || plan->hidden != 2560 || plan->intermediate != 1024 ||
        bank->view.hidden != 2560 || bank->view.intermediate != 1024 || bank->view.local_experts != kExperts / window->world ||
        bank->view.first_expert != window->rank * (kExperts / window->world) ||
        plan->pp_rows < static_cast<std::size_t>(std::min(bank->view.local_experts,
                                                          window->world * window->rows_per_gpu * kTop) + 1) * kTile) {
        return cudaErrorNotSupported;     // one 128-row slab per expert that can be active, plus the shared expert's
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const bool wide = window->world * window->rows_per_gpu > 16 || std::getenv("P92B_EP_WIDE") != nullptr;
    if (cudaError_t st = ensure_dynamic_smem<moe_decode_ep_kernel<16>>(StageLayout<16>::kSmem); st != cudaSuccess) return st;
    if (cudaError_t st = ensure_dynamic_smem<moe_decode_ep_kernel<32>>(StageLayout<32>::kSmem); st != cudaSuccess) return st;
    EpParams p {};
    p.bank = bank->view;
    p.x = input;
    p.router_w = router_weight;
    p.bias = correction_bias;
    p.out = output;
    p.logits = plan->logits;
    p.ids = plan->ids;
    p.route_weights = plan->route_weights;
    p.counts = plan->counts;
    p.hq = plan->hq_pp;
    p.hs = plan->hs_sw;
    p.logits_tagged = plan->ep_logits;
    p.sync = plan->mega_sync + 2;
    p.gu_done = plan->ep_gu_done;
    p.status = plan->status;
    p.trace = plan->trace_on ? plan->mega_trace : nullptr;
    for (int r = 0; r < window->world; ++r) p.win[r] = window->peers[r];
    p.epoch = plan->ep_epoch++;
    p.wepoch = window->epoch++;
    p.routed_scale = routed_scale;
    p.quant_scale = 1.0F;
    p.rows = rows;
    p.rank = window->rank;
    p.world = window->world;
    p.rows_per_gpu = window->rows_per_gpu;
    p.hidden = plan->hidden;
    p.inter = plan->intermediate;
    plan->last_launches = 1;
    plan->last_path = 3;
    const bool pdl = std::getenv("P92B_NO_PDL") == nullptr;
    if (wide) {
        return launch_kernel(moe_decode_ep_kernel<32>, dim3(plan->sm_count), dim3(kEpThreads), StageLayout<32>::kSmem, stream,
                             pdl, window->map_tok[1], plan->map_h[1], p);
    }
    return launch_kernel(moe_decode_ep_kernel<16>, dim3(plan->sm_count), dim3(kEpThreads), StageLayout<16>::kSmem, stream,
                         pdl, window->map_tok[0], plan->map_h[0], p);
}

int p92b_ep_forward_fused_host_async(p92b_plan* plan, const p92b_bank* bank, p92b_ep_window* window,
                                     const uint16_t* pinned_input, const uint16_t* router_weight,
                                     const float* correction_bias, uint16_t* pinned_output, int rows, float routed_scale,
                                     void* stream_) {
    using namespace p92b;
    if (plan == nullptr || pinned_input == nullptr || pinned_output == nullptr || rows <= 0 || rows > plan->max_rows) {
        return cudaErrorInvalidValue;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    std::uint16_t *rows_in = nullptr, *rows_out = nullptr;
    int set = 0;
    cudaError_t st = host_pipeline_begin(plan, pinned_input, rows, stream, &rows_in, &rows_out, &set);
    if (st != cudaSuccess) return st;
    st = static_cast<cudaError_t>(p92b_ep_forward_fused(plan, bank, window, rows_in, router_weight, correction_bias,
                                                        rows_out, rows, routed_scale, stream_));
    if (st != cudaSuccess) return st;
    return host_pipeline_end(plan, pinned_output, rows, stream, set);
}

}  // extern "C"
