// Router for large batches: tensor-core logits, then exact repair of the few that decide the routing.
//
// The reference's logits are FP32 fmaf chains in a fixed order (cuda/nvfp4_ops.cu:178-207): lane l of a warp sums
// columns l, l+32, ... and a shuffle-down tree adds the 32 partial sums.  Expert ids must equal the reference's, so
// every logit that can influence the top-8 has to be THAT number - but almost none can: of 256 logits per token only
// those near the top-8 boundary matter.  Three kernels:
//
//   1. expert_norms_kernel   ||w_e||_2 of the 256 router rows (the error bound below needs them);
//   2. logits_tc_kernel      approximate logits of every (token, expert) as one BF16 x BF16 -> FP32 product on the
//                            5th-generation tensor cores (tcgen05.mma kind::f16, M = 128 tokens, N = 64 experts per
//                            block, operands by TMA, accumulator in TMEM);
//   3. route_repair_kernel   one warp per token: corrected scores from the approximate logits, the approximate 8th
//                            best, the candidate set = every expert whose approximate score is within 2 delta of it,
//                            the candidates' logits recomputed in the reference's exact order, and the reference's
//                            top-8 (cuda/nvfp4_ops.cu:357-433: higher corrected score first, ties to the lower id,
//                            weights from the uncorrected sigmoid, renormalised) taken over the exact values.
//
// Why that is exact.  Let delta bound |approximate - exact| of a corrected score.  An expert outside the candidate set
// has approximate score < a8 - 2 delta (a8 = approximate 8th best), so its exact score is < a8 - delta, while each of
// the eight approximately best experts has exact score >= a8 - delta: eight experts beat it, it is not in the exact
// top-8.  Hence the exact top-8 is a subset of the candidates, and selecting among exactly recomputed candidates
// gives the reference's ids and weights bit for bit.  delta = 0.25 * kLogitBound * ||x_t|| * ||w_e|| + 4e-6: the
// sigmoid's slope is at most 1/4; both the reference chain and the tensor-core sum differ from the true dot product by
// at most (number of sequential roundings) * 2^-23 * sum|x_i w_i| <= that * ||x|| ||w||, with about 85 roundings in the
// reference's order and fewer than 200 in the tensor core's; kLogitBound = 2^-14 is more than twice their sum; 4e-6
// covers the fast-math sigmoid's own error on both sides.  A token whose candidate set would exceed 24 experts, or
// that holds a non-finite logit, has its whole row recomputed exactly instead.
//
// The logits buffer keeps the approximate values except at the recomputed positions, which hold the exact ones.
#include "p92b_common.cuh"
#include "tc_ptx.cuh"

#include <cstdlib>

namespace p92b {

using namespace ptx;

namespace {

constexpr int kTokTile = 128;                 // M: tokens per block (TMEM lanes)
constexpr int kExpTile = 64;                  // N: experts per block
constexpr int kKBytes = 128;                  // one swizzle row: 64 BF16
constexpr int kStageA = kTokTile * kKBytes;   // 16 KB
constexpr int kStageB = kExpTile * kKBytes;   // 8 KB
constexpr int kStageBytes = kStageA + kStageB;
constexpr int kLogitStages = 8;
constexpr int kLogitThreads = 192;            // producer warp, MMA warp, four epilogue warps
constexpr int kLogitSmem = kLogitStages * kStageBytes + 1024;
constexpr float kLogitBound = 1.0F / 16384.0F;
constexpr int kMaxCandidates = 24;

// D[tmem] (+)= A[smem] * B[smem], BF16 operands (both K-major), FP32 accumulate, M=128, K=16 per instruction.
__device__ __forceinline__ void mma_bf16(std::uint32_t d_tmem, std::uint64_t a_desc, std::uint64_t b_desc,
                                         std::uint32_t idesc, bool accumulate) {
    asm volatile(
        "{ .reg .pred p;\n"
        "  setp.ne.b32 p, %4, 0;\n"
        "  tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(static_cast<std::uint32_t>(accumulate))
        : "memory");
}

// Instruction descriptor for kind::f16: FP32 accumulator (bits [4,6) = 1), BF16 A and B (bits [7,10) and [10,13) = 1),
// both K-major, N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr std::uint32_t idesc_bf16(int m, int n) {
    return (1U << 4) | (1U << 7) | (1U << 10) | (static_cast<std::uint32_t>(n >> 3) << 17) |
           (static_cast<std::uint32_t>(m >> 4) << 24);
}

__global__ void __launch_bounds__(256) expert_norms_kernel(const std::uint16_t* __restrict__ w, float* __restrict__ norms,
                                                           int experts, int hidden) {
    // Nothing here reads the upstream kernel's output, so the work comes first and overlaps that kernel's tail; the wait
    // comes last (the kernels behind this one rely on the chain: a kernel that finished without waiting would let them
    // start before the token rows are written).  `norms` alternates between two buffers from call to call, so a repair
    // kernel of the call before cannot still be reading what this one writes.
    pdl_launch_dependents();
    const int e = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (e >= experts) {
        pdl_wait();
        return;
    }
    float s = 0.0F;
    const uint4* row = reinterpret_cast<const uint4*>(w + static_cast<std::size_t>(e) * hidden);
#pragma unroll 4
    for (int v = lane; v < hidden / 8; v += 32) {
        const uint4 q = __ldg(row + v);
        const std::uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float lo = __uint_as_float(words[k] << 16), hi = __uint_as_float(words[k] & 0xffff0000U);
            s = fmaf(lo, lo, s);
            s = fmaf(hi, hi, s);
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffU, s, off);
    if (lane == 0) norms[e] = sqrtf(s) * 1.0001F;             // rounded up a little: it feeds a bound
    pdl_wait();
}

__global__ void __launch_bounds__(kLogitThreads, 1) logits_tc_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                     const __grid_constant__ CUtensorMap map_w,
                                                                     float* __restrict__ logits, int rows, int hidden,
                                                                     std::int32_t* status) {
    // gridDim.z > 1: block z takes a slice of the K blocks and writes its partial sums to slice z of `logits`
    // ([gridDim.z][rows][256]); the repair kernel adds the slices (small batches: 4 blocks would otherwise walk all of
    // K one after the other while 144 SMs idle)
    extern __shared__ std::uint8_t smem_raw[];
    __shared__ __align__(8) std::uint64_t barrier_words[2 * kLogitStages + 1];
    __shared__ std::uint32_t tmem_slot_word;
    __shared__ volatile std::uint32_t abort_word;
    const std::uint32_t base = (smem_u32(smem_raw) + 1023U) & ~1023U;
    const std::uint32_t bars = smem_u32(barrier_words);
    auto full_bar = [&](int s) { return bars + 8U * s; };
    auto empty_bar = [&](int s) { return bars + 8U * (kLogitStages + s); };
    const std::uint32_t accum_bar = bars + 8U * (2 * kLogitStages);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int all_k_blocks = hidden * 2 / kKBytes;
    const int per_split = (all_k_blocks + static_cast<int>(gridDim.z) - 1) / static_cast<int>(gridDim.z);
    const int kb_first = min(all_k_blocks, static_cast<int>(blockIdx.z) * per_split);
    const int k_blocks = min(all_k_blocks, kb_first + per_split) - kb_first;       // this block's share
    const int t0 = blockIdx.x * kTokTile;
    const int e0 = blockIdx.y * kExpTile;
    logits += static_cast<std::size_t>(blockIdx.z) * rows * kExperts;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kLogitStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(accum_bar, 1);
        abort_word = 0;
        fence_mbar_init();
        prefetch_tensormap(&map_x);
        prefetch_tensormap(&map_w);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_slot_word), kExpTile);
        tmem_relinquish();
    }
    pdl_wait();                       // the token rows come from the kernel before this one
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_launch_dependents();
    const std::uint32_t tmem_base = tmem_slot_word;
    auto give_up = [&]() {
        abort_word = 1;
        atomicCAS(status, kStatusOk, kStatusWaitExpired);
    };

    if (warp == 0) {
        if (elect_one()) {
            int stage = 0;
            std::uint32_t phase = 0;
            for (int kb = 0; kb < k_blocks && !abort_word; ++kb) {
                if (!mbar_wait(empty_bar(stage), phase ^ 1U)) { give_up(); break; }
                const std::uint32_t st = base + stage * kStageBytes;
                mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
                tma_load_2d(st, &map_x, full_bar(stage), (kb_first + kb) * kKBytes, t0);        // rows beyond the batch read as zero
                tma_load_2d(st + kStageA, &map_w, full_bar(stage), (kb_first + kb) * kKBytes, e0);
                if (++stage == kLogitStages) { stage = 0; phase ^= 1U; }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            int stage = 0;
            std::uint32_t phase = 0;
            constexpr std::uint32_t idesc = idesc_bf16(kTokTile, kExpTile);
            bool ok = true;
            for (int kb = 0; kb < k_blocks && !abort_word; ++kb) {
                if (!mbar_wait(full_bar(stage), phase)) { give_up(); ok = false; break; }
                tc_fence_after();
                const std::uint32_t st = base + stage * kStageBytes;
                const std::uint64_t a_desc = desc_k_major_sw128(st);
                const std::uint64_t b_desc = desc_k_major_sw128(st + kStageA);
#pragma unroll
                for (int k = 0; k < 4; ++k) mma_bf16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, kb > 0 || k > 0);
                tc_commit(empty_bar(stage));
                if (++stage == kLogitStages) { stage = 0; phase ^= 1U; }
            }
            if (ok && k_blocks > 0) tc_commit(accum_bar);
        }
    } else if (k_blocks > 0) {
        const int quarter = warp & 3;                       // TMEM lanes 32 * quarter ..: the token rows of this warp
        if (mbar_wait(accum_bar, 0)) {
            tc_fence_after();
            const int token = t0 + quarter * 32 + lane;
            const std::uint32_t lane_base = tmem_base + (static_cast<std::uint32_t>(quarter * 32) << 16);
#pragma unroll
            for (int c0 = 0; c0 < kExpTile; c0 += 16) {
                std::uint32_t v[16];
                tmem_load16(lane_base + c0, v);
                tmem_load_wait();
                if (token < rows) {
                    float4* dst = reinterpret_cast<float4*>(logits + static_cast<std::size_t>(token) * kExperts + e0 + c0);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        dst[q] = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                             __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
                    }
                }
            }
        } else {
            give_up();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kExpTile);
    }
}

// 16-byte asynchronous copy global -> shared.
__device__ __forceinline__ void copy16_async(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}

// Exact logit of (token row in shared memory, router row in global memory) in the reference's T > 1 order.
__device__ __forceinline__ float exact_logit(const std::uint16_t* __restrict__ x_row, const std::uint16_t* __restrict__ w_row,
                                             int hidden, int lane) {
    float value = 0.0F;
#pragma unroll 8
    for (int c = lane; c < hidden; c += 32) {
        value = fmaf(bf16_bits_to_float(x_row[c]), bf16_bits_to_float(__ldg(w_row + c)), value);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) value += __shfl_down_sync(0xffffffffU, value, off);
    return __shfl_sync(0xffffffffU, value, 0);
}

constexpr int kRepairWarps = 4;
constexpr int kRepairDepth = 3;                // router rows in flight per warp (register variant)

// CHUNKS = hidden / 32 > 0: the lane's columns of the token row (l, l+32, ...) stay in registers and every candidate's
// router row is brought into shared memory by asynchronous 16-byte copies two candidates ahead (three buffers per warp:
// the rows come from the L2 at about a microsecond each, and 171 MB of them at T=4096 make the L2-to-SM fabric the bound),
// so a chain costs a shared-memory read, a shift and an fmaf per column instead of two 2-byte loads from the L2 that
// the chain has to wait for.  CHUNKS = 0: any hidden size, token row in shared memory, router rows read in place.
// WPT (warps per token) = 1: a warp does everything for its token, four tokens per block - the form for thousands of
// tokens.  WPT = 8: one token per block; the eight warps each build the candidate list (the same list) and then share
// the candidates' exact logits out among themselves, warp 0 finishes - a few hundred tokens would otherwise leave
// most SMs idle while every warp walks eight 2560-step chains one after the other.
// `partials` (splits > 1): the approximate logits arrive as `splits` slices of partial sums ([splits][rows][256]).
template <int CHUNKS, int WPT>
__global__ void __launch_bounds__((WPT > 1 ? WPT : kRepairWarps) * 32) route_repair_kernel(
    const std::uint16_t* __restrict__ x, const std::uint16_t* __restrict__ w, const float* __restrict__ bias,
    const float* __restrict__ w_norms, float* __restrict__ logits, std::int32_t* __restrict__ ids,
    float* __restrict__ weights, int rows, int hidden, float routed_scale, int* __restrict__ stats,
    const float* __restrict__ partials, int splits) {
    extern __shared__ __align__(16) std::uint16_t repair_smem[];
    pdl_launch_dependents();
    pdl_wait();
    constexpr int kWarps = WPT > 1 ? WPT : kRepairWarps;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int token = WPT > 1 ? static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x) * kRepairWarps + warp;
    if (token >= rows) return;                     // WPT > 1: the grid is exactly `rows` blocks
    // per warp: [CHUNKS > 0: two router-row buffers | CHUNKS == 0: the token row], then 256 exact logits, then the candidate list
    constexpr int kRowSlots = CHUNKS > 0 ? kRepairDepth : 1;
    std::uint16_t* x_row = repair_smem + static_cast<std::size_t>(warp) * kRowSlots * hidden;
    std::uint8_t* tail = reinterpret_cast<std::uint8_t*>(repair_smem + static_cast<std::size_t>(kWarps) * kRowSlots * hidden);
    float* exact_row = reinterpret_cast<float*>(tail) + (WPT > 1 ? 0 : warp) * kExperts;      // WPT > 1: one row per block
    std::uint16_t* cand = reinterpret_cast<std::uint16_t*>(tail + kWarps * kExperts * 4) + warp * kExperts;
    float xr[CHUNKS > 0 ? CHUNKS : 1];
    float square = 0.0F;
    if constexpr (CHUNKS > 0) {
        const std::uint16_t* xg = x + static_cast<std::size_t>(token) * hidden + lane;
#pragma unroll
        for (int j = 0; j < CHUNKS; ++j) xr[j] = bf16_bits_to_float(__ldg(xg + 32 * j));
#pragma unroll
        for (int j = 0; j < CHUNKS; ++j) square = fmaf(xr[j], xr[j], square);
    } else {
        for (int v = lane; v < hidden / 8; v += 32) {
            const uint4 q = __ldg(reinterpret_cast<const uint4*>(x + static_cast<std::size_t>(token) * hidden) + v);
            reinterpret_cast<uint4*>(x_row)[v] = q;
            const std::uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float lo = __uint_as_float(words[k] << 16), hi = __uint_as_float(words[k] & 0xffff0000U);
                square = fmaf(lo, lo, square);
                square = fmaf(hi, hi, square);
            }
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) square += __shfl_xor_sync(0xffffffffU, square, off);
    const float x_norm = sqrtf(square) * 1.0001F;
    __syncwarp();

    float* lg = logits + static_cast<std::size_t>(token) * kExperts;
    float approx[8], score[8];
    bool finite = true;
    if (splits > 1) {
        // all loads of the slices are issued before the first sum: one round trip, not one per slice
        float part[kRouterSplits][8];
#pragma unroll
        for (int z = 0; z < kRouterSplits; ++z) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                part[z][i] = z < splits ? __ldg(partials + (static_cast<std::size_t>(z) * rows + token) * kExperts + lane + 32 * i) : 0.0F;
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float sum = part[0][i];
#pragma unroll
            for (int z = 1; z < kRouterSplits; ++z) sum += part[z][i];
            approx[i] = sum;
            if (WPT == 1 || warp == 0) lg[lane + 32 * i] = sum;           // the logits buffer holds the approximate values
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) approx[i] = lg[lane + 32 * i];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        finite = finite && (fabsf(approx[i]) <= 3.0e38F);
        score[i] = 1.0F / (1.0F + expf(-approx[i])) + bias[e];
    }
    finite = __all_sync(0xffffffffU, finite);
    // approximate 8th best corrected score: eight rounds of (remove the current maximum), value only
    float eighth = 0.0F;
    {
        float work[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) work[i] = score[i];
#pragma unroll 1
        for (int round = 0; round < 8; ++round) {
            float best = work[0];
            int at = 0;
#pragma unroll
            for (int i = 1; i < 8; ++i) {
                if (work[i] > best) { best = work[i]; at = i; }
            }
            const std::uint32_t bits = __float_as_uint(best);
            const std::uint32_t key = bits & 0x80000000U ? ~bits : bits | 0x80000000U;
            const std::uint32_t top = __reduce_max_sync(0xffffffffU, key);
            const unsigned holders = __ballot_sync(0xffffffffU, key == top);
            if (lane == __ffs(holders) - 1) {                 // one holder gives its maximum up
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (i == at) work[i] = -3.0e38F;
                }
            }
            const std::uint32_t top_bits = top & 0x80000000U ? top & 0x7fffffffU : ~top;
            eighth = __uint_as_float(top_bits);
        }
    }
    // candidates: approximate score within 2 delta of the approximate 8th
    unsigned member[8];
    int candidates = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        const float delta = 0.25F * kLogitBound * x_norm * w_norms[e] + 4.0e-6F;
        member[i] = __ballot_sync(0xffffffffU, score[i] >= eighth - 2.0F * delta);
        candidates += __popc(member[i]);
    }
    const bool whole_row = !finite || candidates > kMaxCandidates;
    if (whole_row) {
#pragma unroll
        for (int i = 0; i < 8; ++i) member[i] = 0xffffffffU;
    }
    // exact logits of the candidates (or of the whole row), into the logits buffer and into this warp's row
    if constexpr (WPT > 1) {
        for (int e = threadIdx.x; e < kExperts; e += WPT * 32) exact_row[e] = -3.0e38F;
        __syncthreads();                               // before any warp stores a result into the shared row
    } else {
        for (int e = lane; e < kExperts; e += 32) exact_row[e] = -3.0e38F;   // non-candidates can never be selected
    }
    int n_cand = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if ((member[i] >> lane) & 1U) cand[n_cand + __popc(member[i] & ((1U << lane) - 1U))] = static_cast<std::uint16_t>(lane + 32 * i);
        n_cand += __popc(member[i]);
    }
    __syncwarp();
    // this warp's share of the candidates: all of them (WPT = 1) or every WPT-th, starting with its own number
    const int first = WPT > 1 ? warp : 0;
    constexpr int kStep = WPT > 1 ? WPT : 1;
    const int n_mine = n_cand > first ? (n_cand - first + kStep - 1) / kStep : 0;
    if constexpr (CHUNKS > 0) {
        auto fetch = [&](int i) {
            if (i < n_mine) {
                const uint4* src = reinterpret_cast<const uint4*>(w + static_cast<std::size_t>(cand[first + i * kStep]) * hidden);
                uint4* dst = reinterpret_cast<uint4*>(x_row + static_cast<std::size_t>(i % kRepairDepth) * hidden);
                for (int v = lane; v < hidden / 8; v += 32) copy16_async(dst + v, src + v);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");       // an empty group keeps the count in step
        };
#pragma unroll
        for (int i = 0; i < kRepairDepth - 1; ++i) fetch(i);
#pragma unroll 1
        for (int i = 0; i < n_mine; ++i) {
            fetch(i + kRepairDepth - 1);                        // its buffer was last read by candidate i - 1
            asm volatile("cp.async.wait_group %0;" ::"n"(kRepairDepth - 1) : "memory");
            __syncwarp();
            const std::uint16_t* w_row = x_row + static_cast<std::size_t>(i % kRepairDepth) * hidden + lane;
            float value = 0.0F;
#pragma unroll
            for (int j = 0; j < CHUNKS; ++j) value = fmaf(xr[j], bf16_bits_to_float(w_row[32 * j]), value);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) value += __shfl_down_sync(0xffffffffU, value, off);
            if (lane == 0) {
                const int e = cand[first + i * kStep];
                exact_row[e] = value;
                lg[e] = value;
            }
            __syncwarp();                                       // every lane is done with this buffer before it is refilled
        }
    } else {
#pragma unroll 1
        for (int i = 0; i < n_mine; ++i) {
            const int e = cand[first + i * kStep];
            const float value = exact_logit(x_row, w + static_cast<std::size_t>(e) * hidden, hidden, lane);
            if (lane == 0) {
                exact_row[e] = value;
                lg[e] = value;
            }
        }
    }
    if constexpr (WPT > 1) {
        __syncthreads();                                        // every warp's results are in the block's row
        if (warp != 0) return;
    }
    __syncwarp();
    if (lane == 0 && stats != nullptr) {
        atomicAdd(stats + 0, whole_row ? kExperts : candidates);
        if (whole_row) atomicAdd(stats + 1, 1);
    }
    // The reference's top-8 over the exact values.  Every entry gets an order-preserving integer key of its corrected
    // score; experts that were not recomputed (they cannot be in the top-8), NaN scores (a comparison never picks them)
    // and entries already taken carry key 0, below every real score.
    {
        float raw[8];
        std::uint32_t key[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = lane + 32 * i;
            const float v = exact_row[e];
            raw[i] = 1.0F / (1.0F + expf(-v));
            const float corrected = raw[i] + bias[e];
            const std::uint32_t bits = __float_as_uint(corrected);
            const bool usable = v > -1.0e38F && corrected == corrected;
            key[i] = usable ? (bits & 0x80000000U ? ~bits : bits | 0x80000000U) : 0U;
        }
        float chosen_weight = 0.0F;
        int chosen_id = 0;
#pragma unroll 1
        for (int slot = 0; slot < 8; ++slot) {
            // lane-local best: higher key, lower id on ties (ids ascend with i, the comparison is strict)
            std::uint32_t best = key[0];
            int at = 0;
#pragma unroll
            for (int i = 1; i < 8; ++i) {
                if (key[i] > best) { best = key[i]; at = i; }
            }
            const std::uint32_t top = __reduce_max_sync(0xffffffffU, best);
            float my_raw = 0.0F;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (i == at) my_raw = raw[i];
            }
            const int my_id = lane + 32 * at;
            const int winner = static_cast<int>(__reduce_min_sync(0xffffffffU, best == top ? static_cast<std::uint32_t>(my_id) : 0xffffffffU));
            const float winner_raw = __shfl_sync(0xffffffffU, my_raw, winner & 31);
            if ((winner & 31) == lane) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (i == at) key[i] = 0U;
                }
            }
            if (lane == slot) {
                chosen_weight = winner_raw;
                chosen_id = winner;
            }
        }
        float total = 0.0F;
#pragma unroll
        for (int slot = 0; slot < 8; ++slot) total += __shfl_sync(0xffffffffU, chosen_weight, slot);
        const float multiplier = routed_scale / total;
        if (lane < 8) {
            ids[static_cast<std::size_t>(token) * kTop + lane] = chosen_id;
            weights[static_cast<std::size_t>(token) * kTop + lane] = chosen_weight * multiplier;
        }
    }
}

}  // namespace

// Below this the fused decode kernel serves the block (up to 8 rows); the exact-order logits kernels took 50 µs at
// 9 - 31 rows where this router takes 20.
int router_fast_min_rows() { return 9; }

cudaError_t launch_router_fast(p92b_plan* plan, const std::uint16_t* x, const std::uint16_t* router_w, const float* bias,
                               int rows, float routed_scale, cudaStream_t stream, bool pdl) {
    static const bool disabled = std::getenv("P92B_EXACT_LOGITS") != nullptr;
    const int hidden = plan->hidden;
    if (disabled || rows < router_fast_min_rows() || hidden % 64 != 0 || hidden > 8192 ||
        (reinterpret_cast<std::uintptr_t>(x) & 15U) != 0U || (reinterpret_cast<std::uintptr_t>(router_w) & 15U) != 0U) {
        return cudaErrorNotSupported;
    }
    CUtensorMap map_x, map_w;
    cudaError_t st = make_operand_map(&map_x, x, static_cast<std::size_t>(rows), static_cast<std::size_t>(hidden) * 2, kTokTile);
    if (st == cudaSuccess) st = make_operand_map(&map_w, router_w, kExperts, static_cast<std::size_t>(hidden) * 2, kExpTile);
    if (st != cudaSuccess) return cudaErrorNotSupported;
    if ((st = ensure_dynamic_smem<logits_tc_kernel>(kLogitSmem)) != cudaSuccess) return st;
    const bool in_registers = hidden == 2560;
    // small batches: K split over blocks of the logits kernel, and a block of eight warps per token in the repair
    const bool small = rows <= kRouterSplitRows && plan->logit_partials != nullptr && plan->max_rows >= rows &&
                       std::getenv("P92B_ROUTER_NO_SPLIT") == nullptr;
    const int k_blocks = hidden * 2 / kKBytes;
    const int per_split = small ? (k_blocks + kRouterSplits - 1) / kRouterSplits : k_blocks;
    const int splits = (k_blocks + per_split - 1) / per_split;                    // no empty slice
    constexpr int kWide = 8;
    const int repair_warps = small ? kWide : kRepairWarps;
    const std::size_t repair_smem = static_cast<std::size_t>(repair_warps) * (in_registers ? kRepairDepth : 1) * hidden * 2 +
                                    static_cast<std::size_t>(repair_warps) * kExperts * (4 + 2);
    if (small) {
        st = in_registers ? ensure_dynamic_smem<route_repair_kernel<80, kWide>>(static_cast<int>(repair_smem))
                          : ensure_dynamic_smem<route_repair_kernel<0, kWide>>(static_cast<int>(repair_smem));
    } else {
        st = in_registers ? ensure_dynamic_smem<route_repair_kernel<80, 1>>(static_cast<int>(repair_smem))
                          : ensure_dynamic_smem<route_repair_kernel<0, 1>>(static_cast<int>(repair_smem));
    }
    if (st != cudaSuccess) return st;
    float* norms = plan->w_norms + (plan->norms_parity ^= 1) * kExperts;
    st = launch_kernel(expert_norms_kernel, dim3(kExperts / 8), dim3(256), 0, stream, pdl, router_w, norms, kExperts, hidden);
    if (st != cudaSuccess) return st;
    float* approx_out = splits > 1 ? plan->logit_partials : plan->logits;
    st = launch_kernel(logits_tc_kernel, dim3((rows + kTokTile - 1) / kTokTile, kExperts / kExpTile, splits), dim3(kLogitThreads),
                       kLogitSmem, stream, pdl, map_x, map_w, approx_out, rows, hidden, plan->status);
    if (st != cudaSuccess) return st;
    const float* partials = splits > 1 ? plan->logit_partials : nullptr;
    if (small) {
        st = launch_kernel(in_registers ? route_repair_kernel<80, kWide> : route_repair_kernel<0, kWide>, dim3(rows),
                           dim3(kWide * 32), repair_smem, stream, pdl, x, router_w, bias,
                           static_cast<const float*>(norms), plan->logits, plan->ids, plan->route_weights, rows, hidden,
                           routed_scale, plan->router_stats, partials, splits);
    } else {
        st = launch_kernel(in_registers ? route_repair_kernel<80, 1> : route_repair_kernel<0, 1>,
                           dim3((rows + kRepairWarps - 1) / kRepairWarps), dim3(kRepairWarps * 32), repair_smem, stream, pdl, x,
                           router_w, bias, static_cast<const float*>(norms), plan->logits, plan->ids,
                           plan->route_weights, rows, hidden, routed_scale, plan->router_stats, partials, splits);
    }
    plan->last_launches += 3;
    return st;
}

}  // namespace p92b
