// Tensor-core expert kernels: tcgen05 block-scaled MMA (E2M1 x E2M1, one UE4M3
// scale per 16 elements along K) with TMA-staged operands and TMEM accumulators.
//
// Orientation.  The expert weight is the M side of the MMA (128 weight rows per
// tile fill the 128 TMEM lanes), the tokens routed to the expert are the N side
// (N = 16...128 columns).  With one or two tokens per expert (decode) the kernel
// is a pure weight streamer - TMA pulls 128 x 128-byte weight boxes through a
// shared-memory ring and the tensor core consumes them at a small N - and with
// hundreds of tokens per expert (prefill) the same code is a grouped GEMM.
//
// One block = 18 warps, persistent over work items (expert, token tile, 128-row tile):
//   warp 0  producer: one elected lane issues the copies of a K block (256 elements = 128 bytes per row): the
//           weight side is one untiled bulk copy of a contiguous chunk of the bank's tile stream (boxes already in
//           the swizzled shared-memory image, scale slabs behind them), the token side a tiled box load plus its
//           2 KB scale slab; weights and tokens complete on separate mbarriers.  When the weights are read in place
//           from a caller's table of reference-format matrices (SRC 1) the whole warp gathers the box with 16-byte
//           asynchronous copies, writing the same swizzled image;
//   warp 1  MMA issuer: owns TMEM; per K block copies the scale slabs SMEM->TMEM (tcgen05.cp) and issues 4 MMAs of
//           K=64 per weight operand; commits the stage back to the producer and, after the last K block, the
//           accumulator to the epilogue;
//   warps 2-17  epilogue, four per TMEM quarter: each reads 16-column chunks of its 32 lanes of the accumulator
//           (tcgen05.ld), applies the per-tensor scale, rounds to BF16 where the reference does, and either fuses
//           SwiGLU + re-quantisation to NVFP4 (MODE 0), stores the BF16 down rows (MODE 1) or stores BF16 gate and
//           up rows un-fused (MODE 2, the reference's project_expert_gate_up result).
// Every role turns an item number into work from a copy of the routing lists in shared memory (RouteTable), and an
// epilogue warp hands its accumulator buffer back as soon as it has read its columns into registers.
// Two more kernels in this file serve large batches with the same three roles: expert_gu_pair_kernel (one weight stage
// against two 64-row token tiles) and expert_down_slab_kernel (a 128-token slab resident, weights streaming past).
// Scale factors stay in the 128x4-tiled layout the reference keeps them in
// (cuda/nvfp4_ops.cu:869-890): one 512-byte tile is exactly one tcgen05.cp atom.
//
// Every mbarrier wait is bounded; on expiry the block records kStatusWaitExpired,
// stops issuing work, frees its TMEM and returns.
#include "p92b_common.cuh"
#include "tc_ptx.cuh"

#include <algorithm>
#include <cstdlib>

namespace p92b {

using namespace ptx;

namespace {

constexpr int kTileM = 128;
constexpr int kBlockKBytes = 128;                 // one swizzle row: 256 E2M1 values
constexpr int kSfSlab = 2048;                     // 128 rows x 16 scales of one K block
constexpr int kEpilogueWarps = 16;                // four per TMEM quarter: they split the 16-column chunks
constexpr int kThreadsTc = 64 + 32 * kEpilogueWarps;

template <int MODE, int N>
struct Tc {
    static constexpr int kA = MODE == 1 ? 1 : 2;          // gate and up share a token tile (MODE 0 fused, MODE 2 un-fused)
    static constexpr int kABytes = kTileM * kBlockKBytes;
    static constexpr int kBBytes = N * kBlockKBytes;
    static constexpr int kWeightBytes = kA * (kABytes + kSfSlab);          // per stage, independent of the tokens
    // stage image: weight boxes | their scale slabs | token box | token scale slab; for the gate/up
    // kernel the first kWeightBytes are exactly one chunk of the bank's tile stream
    static constexpr int kOffSfA = kA * kABytes;
    static constexpr int kOffB = kA * (kABytes + kSfSlab);
    static constexpr int kOffSfB = kOffB + kBBytes;
    static constexpr int kTokenBytes = kBBytes + kSfSlab;
    static constexpr int kStageBytes = kWeightBytes + kTokenBytes;
    static constexpr int kStagesRaw = (196 * 1024) / kStageBytes;
    static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
    static constexpr int kAccumStride = N < 32 ? 32 : N;          // each accumulator starts on a multiple of 32 columns
    static constexpr int kAccumCols = kA * kAccumStride;
    static constexpr int kSfCols = (kA + 1) * 16;                 // per buffer: 4 columns per K=64 step
    static constexpr int kAccumBuffers = 2 * kAccumCols + 2 * kSfCols <= 512 ? 2 : 1;
    static constexpr int kNeedCols = kAccumBuffers * kAccumCols + 2 * kSfCols;
    static constexpr int kTmemCols = kNeedCols <= 32 ? 32 : kNeedCols <= 64 ? 64 : kNeedCols <= 128 ? 128
                                     : kNeedCols <= 256 ? 256 : 512;
    static constexpr int kBarriers = 3 * kStages + 2 * kAccumBuffers;
    static constexpr int kBarrierBytes = kBarriers * 8 + 16;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 1024;   // + alignment slack
    static_assert(kNeedCols <= 512, "accumulators and scale factors must fit TMEM");
};

struct TcParams {
    BankView bank;
    RouteView route;
    const std::int32_t* pp_off;        // [258]
    const std::int32_t* tile_prefix;   // [active_count + 1]
    const std::uint8_t* b_sf;          // token-side scales, 128x4 tiled over padded positions
    std::uint8_t* hq;                  // MODE 0 out: packed SwiGLU rows [PP][I/2]
    std::uint8_t* hs;                  // MODE 0 out: their scales, 128x4 tiled over padded positions
    std::uint16_t* out;                // MODE 1 out: BF16 down rows [PP][H]
    std::int32_t* status;
    float quant_scale;                 // 1.0, passed at run time so the quantiser's divisions stay run-time operations
    int k_bytes;                       // K/2: bytes per operand row
    int m_total;                       // output rows per expert matrix
    int m_tiles;
    int routing_is_upstream;           // 1: the routing lists are written by the kernel just before this one in the stream
    // optional redirections (stage entry points, p92b_nvfp4_grouped_rows)
    const std::int32_t* out_row;       // null: output rows sit at their padded position; else [dense position] -> output row
    std::uint16_t* gate_out;           // MODE 2: BF16 [output row][m_total]
    std::uint16_t* up_out;
    const p92b_expert_projection* table;   // SRC 1: device table of reference-format matrices, entry expert * 3 + kind
    int table_kind;                    // SRC 1, MODE 1: which of an expert's three matrices
    int skip_shared;                   // 1: the shared expert's items are not computed (the caller has none)
    std::uint16_t* const* row_dest;    // slab kernel of the down product: null, or [padded position] -> destination row
};

struct Item {
    int expert;
    int entry;
    int count;
    int m_tile;
    int pp0;
    int valid;     // tokens of this tile that exist
    int dense0;    // dense (unpadded) position of the tile's first row
};

// The routing lists a block needs to turn an item number into work, copied to shared memory once per block:
// every role decodes every item, and from global memory that is a dozen dependent loads (a binary search over
// the tile prefix, then the expert's entries) - about 1.4 µs per item, which in the MMA lane is time the tensor
// pipe runs dry.  Indexed by active slot.
struct RouteTable {
    std::int32_t prefix[kExperts + 2];      // exclusive prefix of token tiles over the active list, total at [active_count]
    std::int32_t expert[kExperts + 1];
    std::int32_t count[kExperts + 1];
    std::int32_t pp_off[kExperts + 1];
    std::int32_t offset[kExperts + 1];
    std::int32_t active_count;
};

// All threads of the block, after the lists are known to be written; the caller synchronises the block afterwards.
__device__ __forceinline__ void load_route_table(const TcParams& p, RouteTable* t) {
    const int n = min(*p.route.active_count, kExperts + 1);
    for (int a = threadIdx.x; a <= n; a += blockDim.x) {
        t->prefix[a] = p.tile_prefix[a];
        if (a < n) {
            const int e = p.route.active[a];
            t->expert[a] = e;
            t->count[a] = p.route.counts[e];
            t->pp_off[a] = p.pp_off[e];
            t->offset[a] = p.route.offsets[e];
        }
    }
    if (threadIdx.x == 0) t->active_count = n;
}

template <int N>
__device__ __forceinline__ bool decode_item(const TcParams& p, const RouteTable& t, int item, Item* it) {
    const int tt = item / p.m_tiles;
    it->m_tile = item - tt * p.m_tiles;
    int lo = 0, hi = t.active_count;         // find a: prefix[a] <= tt < prefix[a+1]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (t.prefix[mid] <= tt) lo = mid; else hi = mid;
    }
    const int n_tile = tt - t.prefix[lo];
    it->expert = t.expert[lo];
    it->entry = it->expert == kExperts ? p.bank.local_experts : it->expert - p.bank.first_expert;
    it->count = t.count[lo];
    it->pp0 = t.pp_off[lo] + n_tile * N;
    it->valid = min(N, it->count - n_tile * N);
    it->dense0 = t.offset[lo] + n_tile * N;
    if (p.skip_shared && it->expert == kExperts) return false;
    if (p.table != nullptr) {          // weights in place: the table is indexed by the global expert id
        it->entry = it->expert;
        return it->expert >= 0 && it->expert < kExperts;
    }
    return it->entry >= 0 && it->entry <= p.bank.local_experts;
}

// 16-byte asynchronous copy global -> shared (through the load/store unit, not the bulk-copy engine).
__device__ __forceinline__ void async_copy16_tc(std::uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}

// Two floats rounded to BF16 (nearest even) in one conversion: the first in the low half.
__device__ __forceinline__ std::uint32_t bf16x2_bits(float low, float high) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<const std::uint32_t*>(&pair);
}

// The gate/up epilogue for one chunk of 16 token columns (shared by expert_tc_kernel<0, N> and
// expert_gu_pair_kernel).  A lane holds one weight row (row0 + lane of the intermediate dimension): gate g[j] and
// up u[j] for token column c0 + j.  bf16(alpha * product) for both, SwiGLU rounded to BF16
// (cuda/nvfp4_ops.cu:97-105), then the activation quantiser (cuda/nvfp4_ops.cu:818-841) along the intermediate
// dimension, whose 16-element blocks are the two 16-lane halves of the warp:
//   * block maximum of every column: one warp reduction per column over the half (|h| is a non-negative float, so
//     its bit pattern orders like an unsigned integer);
//   * the E4M3 scale and the multiplier of column c are computed ONCE, by lane c of the half, which also stores the
//     scale byte; the other lanes fetch the multiplier with one shuffle per column;
//   * a lane packs its 16 quantised values (one row, 16 tokens) into 64 bits, and a four-round butterfly over the
//     half transposes the 16 x 16 nibble matrix, after which lane c holds the 16 rows of token c0 + c: one 8-byte
//     store per lane instead of a byte store per lane pair and column.
// The arithmetic per element is the reference's; only who computes what has changed.
// hq_rows = packed rows of the tile's first token (p.hq + pp0 * inter / 2); hs_tile = the 128-row scale tile row of
// that token (p.hs + (pp0 >> 7) * (inter / 64) * 512); n_base = pp0 & 127; columns from `valid` on are not stored.
__device__ __forceinline__ void swiglu_requant_chunk(const std::uint32_t (&g)[16], const std::uint32_t (&u)[16], float alpha_g,
                                                     float alpha_u, float quant_scale, int lane, int c0, int valid, int n_base,
                                                     int inter, int row0, std::uint8_t* hq_rows, std::uint8_t* hs_tile) {
    const int half = lane >> 4;                       // which 16-row block of the warp's 32 rows
    const int c = lane & 15;                          // the column this lane owns after the reductions
    const unsigned half_mask = half ? 0xffff0000U : 0x0000ffffU;
    float h[16];
    std::uint32_t amax_bits[16];
    // the three BF16 roundings per element go through the two-wide conversion (one instruction for gate and up of a
    // column, one for the results of two columns): same round-to-nearest-even, fewer trips through the conversion pipe
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        float silu_times_up[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int j = 2 * k + i;
            const std::uint32_t gu = bf16x2_bits(__uint_as_float(g[j]) * alpha_g, __uint_as_float(u[j]) * alpha_u);
            const float gv = __uint_as_float(gu << 16);
            const float uv = __uint_as_float(gu & 0xffff0000U);
            silu_times_up[i] = (gv / (1.0F + expf(-gv))) * uv;
        }
        const std::uint32_t hh = bf16x2_bits(silu_times_up[0], silu_times_up[1]);
        h[2 * k] = __uint_as_float(hh << 16);
        h[2 * k + 1] = __uint_as_float(hh & 0xffff0000U);
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) amax_bits[j] = __reduce_max_sync(half_mask, __float_as_uint(h[j]) & 0x7fffffffU);
    // amax of the column this lane owns: a select tree over the 16 results (register arrays take no run-time index)
    std::uint32_t mine8[8], mine4[4], mine2[2];
#pragma unroll
    for (int i = 0; i < 8; ++i) mine8[i] = (c & 8) ? amax_bits[8 + i] : amax_bits[i];
#pragma unroll
    for (int i = 0; i < 4; ++i) mine4[i] = (c & 4) ? mine8[4 + i] : mine8[i];
#pragma unroll
    for (int i = 0; i < 2; ++i) mine2[i] = (c & 2) ? mine4[2 + i] : mine4[i];
    const float amax = __uint_as_float((c & 1) ? mine2[1] : mine2[0]);
    const __nv_fp8_e4m3 scale(amax * (quant_scale / 6.0F));
    const float decoded = static_cast<float>(scale);
    const float my_multiplier = decoded == 0.0F ? 0.0F : quant_scale / decoded;
    const int n_mine = c0 + c;
    if (n_mine < valid) {
        const int sf_col = (row0 >> 4) + half;
        const int tn = n_base + n_mine;
        hs_tile[static_cast<std::size_t>(sf_col >> 2) * 512 + (sf_col & 3) + (tn & 31) * 16 + (tn >> 5) * 4] = scale.__x;
    }
    // this lane's row: 16 E2M1 values, column j at nibble j
    std::uint32_t w0 = 0U, w1 = 0U;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float m0 = __shfl_sync(0xffffffffU, my_multiplier, (lane & 16) | (2 * k));
        const float m1 = __shfl_sync(0xffffffffU, my_multiplier, (lane & 16) | (2 * k + 1));
        const std::uint32_t byte = __nv_fp4x2_e2m1(make_float2(h[2 * k] * m0, h[2 * k + 1] * m1)).__x;
        if (k < 4) w0 |= byte << (8 * k); else w1 |= byte << (8 * (k - 4));
    }
    // transpose the half's 16 x 16 nibble matrix: afterwards nibble r of lane c is (row r, column c)
    {
        const bool up8 = (lane & 8) != 0;                  // distance 8: whole words change hands
        const std::uint32_t got = __shfl_xor_sync(0xffffffffU, up8 ? w0 : w1, 8);
        if (up8) w0 = got; else w1 = got;
    }
#pragma unroll
    for (int d = 4; d >= 1; d >>= 1) {
        const std::uint32_t low = d == 4 ? 0x0000ffffU : d == 2 ? 0x00ff00ffU : 0x0f0f0f0fU;
        const int shift = 4 * d;
        const bool upper = (lane & d) != 0;
        const std::uint32_t s0 = upper ? (w0 & low) << shift : (w0 >> shift) & low;
        const std::uint32_t s1 = upper ? (w1 & low) << shift : (w1 >> shift) & low;
        const std::uint32_t r0 = __shfl_xor_sync(0xffffffffU, s0, d);
        const std::uint32_t r1 = __shfl_xor_sync(0xffffffffU, s1, d);
        w0 = (upper ? w0 & ~low : w0 & low) | r0;
        w1 = (upper ? w1 & ~low : w1 & low) | r1;
    }
    if (n_mine < valid) {
        *reinterpret_cast<uint2*>(hq_rows + static_cast<std::size_t>(n_mine) * (inter / 2) + ((row0 + 16 * half) >> 1)) =
            make_uint2(w0, w1);
    }
}

template <int MODE, int N, int SRC>
__global__ void __launch_bounds__(kThreadsTc, 1) expert_tc_kernel(const __grid_constant__ CUtensorMap map_b,
                                                                   const TcParams p) {
    using C = Tc<MODE, N>;
    extern __shared__ std::uint8_t smem_raw[];
    __shared__ RouteTable route_table;
    const std::uint32_t base = (smem_u32(smem_raw) + 1023U) & ~1023U;
    const std::uint32_t bars = base + C::kStages * C::kStageBytes;
    // per stage: weights landed, tokens landed, stage free; per accumulator buffer: full, empty
    auto weight_bar = [&](int s) { return bars + 8U * s; };
    auto token_bar = [&](int s) { return bars + 8U * (C::kStages + s); };
    auto empty_bar = [&](int s) { return bars + 8U * (2 * C::kStages + s); };
    auto accum_full = [&](int b) { return bars + 8U * (3 * C::kStages + b); };
    auto accum_empty = [&](int b) { return bars + 8U * (3 * C::kStages + C::kAccumBuffers + b); };
    const std::uint32_t tmem_slot = bars + 8U * C::kBarriers;
    volatile std::uint32_t* tmem_slot_ptr =
        reinterpret_cast<volatile std::uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
    volatile std::uint32_t* abort_ptr = tmem_slot_ptr + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int k_blocks = p.k_bytes / kBlockKBytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            // in-place weights: the scale slabs arrive by bulk copy (one arrival with the byte count), the boxes by
            // the 32 producer lanes' own copies (one arrival each, after their copies have landed)
            mbar_init(weight_bar(s), SRC == 1 ? 33 : 1);
            mbar_init(token_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < C::kAccumBuffers; ++b) {
            mbar_init(accum_full(b), 1);
            mbar_init(accum_empty(b), kEpilogueWarps);
        }
        *abort_ptr = 0;
        fence_mbar_init();
        prefetch_tensormap(&map_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::kTmemCols);
        tmem_relinquish();
    }
    // the routing lists come from the kernel just upstream (gate/up) or from one further up (down):
    // only the former has to wait for its predecessor before it can look at its work list
    if (p.routing_is_upstream || SRC == 1) pdl_wait();
    load_route_table(p, &route_table);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_launch_dependents();
    const std::uint32_t tmem_base = *tmem_slot_ptr;
    const int total_items = route_table.prefix[route_table.active_count] * p.m_tiles;
    auto give_up = [&]() {
        *abort_ptr = 1;
        atomicCAS(p.status, kStatusOk, kStatusWaitExpired);
    };

    if (warp == 0 && SRC == 1) {
        // ------------------------------------------------ producer, weights read in place
        // The matrices are row-major [rows][K/2] wherever the caller keeps them, so a stage's box is gathered: 128
        // rows x eight 16-byte pieces per box, piece j of row r to r * 128 + ((j ^ (r & 7)) * 16) - the image a
        // 128-byte-swizzle tile load would have written.  A lane's copies of a stage form one group; a stage is
        // handed to the MMA lane (fence to the asynchronous proxy, arrival) when its group has landed, kLag stages
        // behind the one being issued, so kLag stages of copies are always in flight.
        constexpr int kLag = C::kStages - 1;
        int stage = 0, oldest = 0, in_flight = 0;
        std::uint32_t phase = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < total_items && !*abort_ptr && ok; item += gridDim.x) {
            Item it;
            if (!decode_item<N>(p, route_table, item, &it)) continue;
            const p92b_expert_projection first = p.table[it.entry * 3 + (MODE == 1 ? p.table_kind : 0)];
            const p92b_expert_projection second = MODE == 1 ? first : p.table[it.entry * 3 + 1];
            if (((reinterpret_cast<std::uintptr_t>(first.weight) | reinterpret_cast<std::uintptr_t>(second.weight) |
                  reinterpret_cast<std::uintptr_t>(first.scales_swizzled) | reinterpret_cast<std::uintptr_t>(second.scales_swizzled)) & 15U) != 0U) {
                *abort_ptr = 1;                                       // the copies need 16-byte aligned matrices
                atomicCAS(p.status, kStatusOk, kStatusBadPointer);
                break;
            }
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(empty_bar(stage), phase ^ 1U)) { give_up(); ok = false; break; }
                const std::uint32_t st = base + stage * C::kStageBytes;
#pragma unroll
                for (int a = 0; a < C::kA; ++a) {
                    const std::uint8_t* src = (a == 0 ? first.weight : second.weight) +
                                              static_cast<std::size_t>(it.m_tile) * kTileM * p.k_bytes + kb * kBlockKBytes;
#pragma unroll 8
                    for (int q = 0; q < kTileM * 8 / 32; ++q) {
                        const int piece = lane + 32 * q;
                        const int r = piece >> 3, j = piece & 7;
                        async_copy16_tc(st + a * C::kABytes + r * 128 + ((j ^ (r & 7)) * 16),
                                        src + static_cast<std::size_t>(r) * p.k_bytes + j * 16);
                    }
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
                if (lane == 0) {
                    // scale slabs: row block m_tile, scale column blocks 4 kb .. 4 kb + 3 of the 128x4 tiling: 2 KB contiguous
                    mbar_arrive_expect_tx(weight_bar(stage), C::kA * kSfSlab);
#pragma unroll
                    for (int a = 0; a < C::kA; ++a) {
                        const std::uint8_t* sf = (a == 0 ? first.scales_swizzled : second.scales_swizzled) +
                                                 (static_cast<std::size_t>(it.m_tile) * (k_blocks * 4) + kb * 4) * 512;
                        bulk_load(st + C::kOffSfA + a * kSfSlab, sf, kSfSlab, weight_bar(stage));
                    }
                    mbar_arrive_expect_tx(token_bar(stage), C::kTokenBytes);
                    tma_load_2d(st + C::kOffB, &map_b, token_bar(stage), kb * kBlockKBytes, it.pp0);
                    const std::uint8_t* bsf = p.b_sf + (static_cast<std::size_t>(it.pp0 >> 7) * (p.k_bytes / 32) + kb * 4) * 512;
                    bulk_load(st + C::kOffSfB, bsf, kSfSlab, token_bar(stage));
                }
                if (++in_flight > kLag) {
                    asm volatile("cp.async.wait_group %0;" ::"n"(kLag) : "memory");
                    fence_proxy_async();
                    mbar_arrive(weight_bar(oldest));
                    if (++oldest == C::kStages) oldest = 0;
                    --in_flight;
                }
                if (++stage == C::kStages) { stage = 0; phase ^= 1U; }
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        fence_proxy_async();
        while (in_flight > 0) {
            mbar_arrive(weight_bar(oldest));
            if (++oldest == C::kStages) oldest = 0;
            --in_flight;
        }
    } else if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (elect_one()) {
            int stage = 0;
            std::uint32_t phase = 0;
            bool upstream_done = p.routing_is_upstream != 0;
            for (int item = blockIdx.x; item < total_items && !*abort_ptr; item += gridDim.x) {
                Item it;
                if (!decode_item<N>(p, route_table, item, &it)) continue;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1U)) { give_up(); break; }
                    const std::uint32_t st = base + stage * C::kStageBytes;
                    // weights never depend on the upstream kernel: they start streaming at once
                    mbar_arrive_expect_tx(weight_bar(stage), C::kWeightBytes);
                    if constexpr (MODE != 1) {
                        // one chunk = gate box, up box and both scale slabs of this (row tile, K block)
                        const std::uint8_t* chunk = p.bank.g13 +
                            ((static_cast<std::size_t>(it.entry) * p.m_tiles + it.m_tile) * k_blocks + kb) * kChunkBytes;
                        bulk_load(st, chunk, kChunkBytes, weight_bar(stage));
                    } else {
                        // chunks of the down stream hold two K blocks: take this block's box and slab
                        const std::uint8_t* chunk = p.bank.g2 +
                            ((static_cast<std::size_t>(it.entry) * p.m_tiles + it.m_tile) * (k_blocks / 2) + (kb >> 1)) *
                                kChunkBytes;
                        bulk_load(st, chunk + (kb & 1) * kChunkBox, kChunkBox, weight_bar(stage));
                        bulk_load(st + C::kOffSfA, chunk + kChunkScaleOffset + (kb & 1) * kChunkScaleBytes, kSfSlab,
                                  weight_bar(stage));
                    }
                    if (upstream_done) {
                        mbar_arrive_expect_tx(token_bar(stage), C::kTokenBytes);
                        tma_load_2d(st + C::kOffB, &map_b, token_bar(stage), kb * kBlockKBytes, it.pp0);
                        const std::uint8_t* bsf = p.b_sf +
                            (static_cast<std::size_t>(it.pp0 >> 7) * (p.k_bytes / 32) + kb * 4) * 512;
                        bulk_load(st + C::kOffSfB, bsf, kSfSlab, token_bar(stage));
                    }
                    const bool ring_full = stage == C::kStages - 1;
                    const bool last_load = kb == k_blocks - 1 && item + static_cast<int>(gridDim.x) >= total_items;
                    if (!upstream_done && (ring_full || last_load)) {
                        // every stage now has its weights in flight; the token rows are written by the
                        // upstream kernel, so wait for it, then issue the token loads that were held back
                        pdl_wait();
                        upstream_done = true;
                        int it_item = blockIdx.x, it_kb = 0;
                        for (int s = 0; s <= stage; ++s) {
                            Item held;
                            while (!decode_item<N>(p, route_table, it_item, &held)) it_item += gridDim.x;
                            const std::uint32_t hst = base + s * C::kStageBytes;
                            mbar_arrive_expect_tx(token_bar(s), C::kTokenBytes);
                            tma_load_2d(hst + C::kOffB, &map_b, token_bar(s), it_kb * kBlockKBytes, held.pp0);
                            const std::uint8_t* hsf = p.b_sf +
                                (static_cast<std::size_t>(held.pp0 >> 7) * (p.k_bytes / 32) + it_kb * 4) * 512;
                            bulk_load(hst + C::kOffSfB, hsf, kSfSlab, token_bar(s));
                            if (++it_kb == k_blocks) { it_kb = 0; it_item += gridDim.x; }
                        }
                    }
                    if (++stage == C::kStages) { stage = 0; phase ^= 1U; }
                }
            }
            if (!upstream_done) pdl_wait();      // no work at all: still order this grid after its predecessor
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issuer
        if (elect_one()) {
            int stage = 0;
            std::uint32_t phase = 0;
            int buffer = 0;
            std::uint32_t accum_phase[2] = {0U, 0U};
            constexpr std::uint32_t idesc = idesc_nvf4(kTileM, N);
            const std::uint32_t sf_tmem = tmem_base + C::kAccumBuffers * C::kAccumCols;
            int sf_buffer = 0;
            for (int item = blockIdx.x; item < total_items && !*abort_ptr; item += gridDim.x) {
                Item it;
                if (!decode_item<N>(p, route_table, item, &it)) continue;
                if (!mbar_wait(accum_empty(buffer), accum_phase[buffer] ^ 1U)) { give_up(); break; }
                tc_fence_after();
                const std::uint32_t accum = tmem_base + buffer * C::kAccumCols;
                // a 64-row token tile may start in the middle of a 128-row scale tile: its scales then sit
                // two TMEM columns further (rows 64..127 are quarters 2 and 3 of the tile)
                const std::uint32_t b_quarter = static_cast<std::uint32_t>((it.pp0 & 127) >> 5);
                bool ok = true;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(weight_bar(stage), phase) || !mbar_wait(token_bar(stage), phase)) {
                        give_up();
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const std::uint32_t st = base + stage * C::kStageBytes;
                    const std::uint32_t sfc = sf_tmem + sf_buffer * C::kSfCols;
#pragma unroll
                    for (int o = 0; o < C::kA + 1; ++o) {
                        const std::uint32_t slab = o < C::kA ? st + C::kOffSfA + o * kSfSlab : st + C::kOffSfB;
#pragma unroll
                        for (int k = 0; k < 4; ++k) tc_copy_sf(sfc + o * 16 + k * 4, desc_scale_atom(slab + k * 512));
                    }
                    const std::uint64_t b_desc = desc_k_major_sw128(st + C::kOffB);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
#pragma unroll
                        for (int a = 0; a < C::kA; ++a) {
                            const std::uint64_t a_desc = desc_k_major_sw128(st + a * C::kABytes);
                            mma_nvf4(accum + a * C::kAccumStride, a_desc + 2 * k, b_desc + 2 * k, idesc,
                                     sfc + a * 16 + k * 4, sfc + C::kA * 16 + k * 4 + b_quarter, kb > 0 || k > 0);
                        }
                    }
                    tc_commit(empty_bar(stage));
                    sf_buffer ^= 1;
                    if (++stage == C::kStages) { stage = 0; phase ^= 1U; }
                }
                if (!ok) break;
                tc_commit(accum_full(buffer));
                accum_phase[buffer] ^= 1U;
                if (C::kAccumBuffers == 2) buffer ^= 1;
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        // Sixteen warps: warp w reads TMEM lanes 32*(w & 3) .. +31 (one output row per lane) and the four
        // warps of a quarter take every fourth 16-column chunk.  A chunk is processed without any
        // data-dependent branch so the sixteen per-column dependency chains interleave; only the
        // stores are predicated on the column being a real token.
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        int buffer = 0;
        std::uint32_t accum_phase[2] = {0U, 0U};
        for (int item = blockIdx.x; item < total_items && !*abort_ptr; item += gridDim.x) {
            Item it;
            if (!decode_item<N>(p, route_table, item, &it)) continue;
            if (!mbar_wait(accum_full(buffer), accum_phase[buffer])) { give_up(); break; }
            accum_phase[buffer] ^= 1U;
            tc_fence_after();
            const std::uint32_t lane_base =
                tmem_base + buffer * C::kAccumCols + (static_cast<std::uint32_t>(quarter * 32) << 16);
            const int row = it.m_tile * kTileM + quarter * 32 + lane;          // output row of this lane
            if constexpr (MODE == 0) {
                const float alpha_g = p.bank.alpha[it.entry * 3 + 0];
                const float alpha_u = p.bank.alpha[it.entry * 3 + 1];
                const int inter = p.m_total;
                // the token tile's packed rows and its 128-row scale tile; pp0 is a multiple of N
                std::uint8_t* hs_tile = p.hs + static_cast<std::size_t>(it.pp0 >> 7) * (inter / 64) * 512;
                std::uint8_t* hq_rows = p.hq + static_cast<std::size_t>(it.pp0) * (inter / 2);
                const int n_base = it.pp0 & 127;
                const int row0 = it.m_tile * kTileM + quarter * 32;
#pragma unroll 1
                for (int c0 = half * 16; c0 < N; c0 += 16 * (kEpilogueWarps / 4)) {
                    if (c0 >= it.valid) break;                                    // warp uniform
                    std::uint32_t g[16], u[16];
                    tmem_load16(lane_base + c0, g);
                    tmem_load16(lane_base + C::kAccumStride + c0, u);
                    tmem_load_wait();
                    swiglu_requant_chunk(g, u, alpha_g, alpha_u, p.quant_scale, lane, c0, it.valid, n_base, inter, row0, hq_rows, hs_tile);
                }
            } else if constexpr (MODE == 2) {
                // gate and up rows as the reference's project_expert_gate_up returns them: bf16(alpha * product),
                // row (token, slot) of the caller's [rows * 8][intermediate] buffers
                const float alpha_g = SRC == 1 ? *p.table[it.entry * 3 + 0].alpha : p.bank.alpha[it.entry * 3 + 0];
                const float alpha_u = SRC == 1 ? *p.table[it.entry * 3 + 1].alpha : p.bank.alpha[it.entry * 3 + 1];
                const int inter = p.m_total;
#pragma unroll 1
                for (int c0 = half * 16; c0 < N; c0 += 16 * (kEpilogueWarps / 4)) {
                    if (c0 >= it.valid) break;
                    std::uint32_t g[16], u[16];
                    tmem_load16(lane_base + c0, g);
                    tmem_load16(lane_base + C::kAccumStride + c0, u);
                    tmem_load_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int n = c0 + j;
                        if (n < it.valid) {
                            const std::size_t r = static_cast<std::size_t>(p.out_row != nullptr ? p.out_row[it.dense0 + n] : it.pp0 + n);
                            p.gate_out[r * inter + row] = float_to_bf16_bits(__uint_as_float(g[j]) * alpha_g);
                            p.up_out[r * inter + row] = float_to_bf16_bits(__uint_as_float(u[j]) * alpha_u);
                        }
                    }
                }
            } else {
                const float alpha = SRC == 1 ? *p.table[it.entry * 3 + p.table_kind].alpha : p.bank.alpha[it.entry * 3 + 2];
                const int hidden = p.m_total;
#pragma unroll 1
                for (int c0 = half * 16; c0 < N; c0 += 16 * (kEpilogueWarps / 4)) {
                    if (c0 >= it.valid) break;
                    std::uint32_t d[16];
                    tmem_load16(lane_base + c0, d);
                    tmem_load_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int n = c0 + j;
                        if (n < it.valid) {
                            const std::size_t r = static_cast<std::size_t>(p.out_row != nullptr ? p.out_row[it.dense0 + n] : it.pp0 + n);
                            p.out[r * hidden + row] = float_to_bf16_bits(__uint_as_float(d[j]) * alpha);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(accum_empty(buffer));
            if (C::kAccumBuffers == 2) buffer ^= 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// ---- gate/up for large batches: two 64-row token tiles per weight stage ---------------------------
// At thousands of tokens the gate/up product is bound by L2-to-SM traffic: every 64-row token tile of an
// expert pulls the expert's 128-row weight tile (36 KB per K block) across again.  Here an item is a PAIR
// of neighbouring token tiles (one 128-row slab of the padded position space): a weight stage is loaded
// once and multiplied with both, which halves the weight traffic of experts with more than 64 rows.
// Each half keeps its own accumulator pair (gate | up, 64 columns each); three such buffers rotate, so
// the epilogue of one item still overlaps the loads and MMAs of the next.
struct GuPair {
    static constexpr int kN = 64;
    static constexpr int kChunk = 2 * (kTileM * kBlockKBytes + kSfSlab);            // 36,864: one chunk of the bank's stream
    static constexpr int kOffSfA = 2 * kTileM * kBlockKBytes;
    static constexpr int kOffB0 = kChunk;
    static constexpr int kOffB1 = kOffB0 + kN * kBlockKBytes;
    static constexpr int kOffSfB = kOffB1 + kN * kBlockKBytes;
    static constexpr int kStageBytes = kOffSfB + kSfSlab;                           // 55,296
    static constexpr int kStages = 4;
    static constexpr int kAccumCols = 2 * kN;                                       // gate at +0, up at +64
    static constexpr int kAccumBuffers = 3;
    static constexpr int kSfCols = 3 * 16;                                          // SFA gate, SFA up, SFB
    static constexpr int kTmemCols = 512;                                           // 3 * 128 + 2 * 48 = 480
    static constexpr int kBarriers = 3 * kStages + 2 * kAccumBuffers;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBarriers * 8 + 16 + 1024;
    // the epilogue (SwiGLU + re-quantisation, about 40 instructions per element) is what the issue slots are spent
    // on: four warps per TMEM quarter, each taking one 16-column chunk of a half
    static constexpr int kEpilogueWarps = 16;
    static constexpr int kThreads = 64 + 32 * kEpilogueWarps;
};

__global__ void __launch_bounds__(GuPair::kThreads, 1) expert_gu_pair_kernel(const __grid_constant__ CUtensorMap map_b,
                                                                        const TcParams p) {
    using C = GuPair;
    extern __shared__ std::uint8_t smem_raw[];
    __shared__ RouteTable route_table;
    const std::uint32_t base = (smem_u32(smem_raw) + 1023U) & ~1023U;
    const std::uint32_t bars = base + C::kStages * C::kStageBytes;
    auto weight_bar = [&](int s) { return bars + 8U * s; };
    auto token_bar = [&](int s) { return bars + 8U * (C::kStages + s); };
    auto empty_bar = [&](int s) { return bars + 8U * (2 * C::kStages + s); };
    auto accum_full = [&](int b) { return bars + 8U * (3 * C::kStages + b); };
    auto accum_empty = [&](int b) { return bars + 8U * (3 * C::kStages + C::kAccumBuffers + b); };
    const std::uint32_t tmem_slot = bars + 8U * C::kBarriers;
    volatile std::uint32_t* tmem_slot_ptr =
        reinterpret_cast<volatile std::uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
    volatile std::uint32_t* abort_ptr = tmem_slot_ptr + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int k_blocks = p.k_bytes / kBlockKBytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(weight_bar(s), 1);
            mbar_init(token_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < C::kAccumBuffers; ++b) {
            mbar_init(accum_full(b), 1);
            mbar_init(accum_empty(b), C::kEpilogueWarps);
        }
        *abort_ptr = 0;
        fence_mbar_init();
        prefetch_tensormap(&map_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::kTmemCols);
        tmem_relinquish();
    }
    pdl_wait();                       // routing lists and token rows come from the kernels upstream
    load_route_table(p, &route_table);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_launch_dependents();
    const std::uint32_t tmem_base = *tmem_slot_ptr;
    const int total_items = route_table.prefix[route_table.active_count] * p.m_tiles;       // the prefix counts 128-row slabs here
    auto give_up = [&]() {
        *abort_ptr = 1;
        atomicCAS(p.status, kStatusOk, kStatusWaitExpired);
    };

    if (warp == 0) {
        if (elect_one()) {
            int stage = 0;
            std::uint32_t phase = 0;
            for (int item = blockIdx.x; item < total_items && !*abort_ptr; item += gridDim.x) {
                Item it;
                if (!decode_item<2 * C::kN>(p, route_table, item, &it)) continue;
                const bool two = it.valid > C::kN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1U)) { give_up(); break; }
                    const std::uint32_t st = base + stage * C::kStageBytes;
                    mbar_arrive_expect_tx(weight_bar(stage), C::kChunk);
                    bulk_load(st, p.bank.g13 + ((static_cast<std::size_t>(it.entry) * p.m_tiles + it.m_tile) * k_blocks + kb) *
                                                   kChunkBytes,
                              kChunkBytes, weight_bar(stage));
                    mbar_arrive_expect_tx(token_bar(stage), (two ? 2 : 1) * C::kN * kBlockKBytes + kSfSlab);
                    tma_load_2d(st + C::kOffB0, &map_b, token_bar(stage), kb * kBlockKBytes, it.pp0);
                    if (two) tma_load_2d(st + C::kOffB1, &map_b, token_bar(stage), kb * kBlockKBytes, it.pp0 + C::kN);
                    bulk_load(st + C::kOffSfB,
                              p.b_sf + (static_cast<std::size_t>(it.pp0 >> 7) * (p.k_bytes / 32) + kb * 4) * 512, kSfSlab,
                              token_bar(stage));
                    if (++stage == C::kStages) { stage = 0; phase ^= 1U; }
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            int stage = 0;
            std::uint32_t phase = 0;
            int next_buffer = 0;
            std::uint32_t accum_phase = 0;                      // bit b = phase of buffer b
            constexpr std::uint32_t idesc = idesc_nvf4(kTileM, C::kN);
            const std::uint32_t sf_tmem = tmem_base + C::kAccumBuffers * C::kAccumCols;
            int sf_buffer = 0;
            for (int item = blockIdx.x; item < total_items && !*abort_ptr; item += gridDim.x) {
                Item it;
                if (!decode_item<2 * C::kN>(p, route_table, item, &it)) continue;
                const int halves = it.valid > C::kN ? 2 : 1;
                int buffer[2];
                bool ok = true;
                for (int h = 0; h < halves && ok; ++h) {
                    buffer[h] = next_buffer;
                    next_buffer = (next_buffer + 1) % C::kAccumBuffers;
                    if (!mbar_wait(accum_empty(buffer[h]), ((accum_phase >> buffer[h]) & 1U) ^ 1U)) { give_up(); ok = false; }
                }
                if (!ok) break;
                tc_fence_after();
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(weight_bar(stage), phase) || !mbar_wait(token_bar(stage), phase)) {
                        give_up();
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const std::uint32_t st = base + stage * C::kStageBytes;
                    const std::uint32_t sfc = sf_tmem + sf_buffer * C::kSfCols;
#pragma unroll
                    for (int o = 0; o < 3; ++o) {
                        const std::uint32_t slab = o < 2 ? st + C::kOffSfA + o * kSfSlab : st + C::kOffSfB;
#pragma unroll
                        for (int k = 0; k < 4; ++k) tc_copy_sf(sfc + o * 16 + k * 4, desc_scale_atom(slab + k * 512));
                    }
                    for (int h = 0; h < halves; ++h) {
                        const std::uint32_t accum = tmem_base + buffer[h] * C::kAccumCols;
                        const std::uint64_t b_desc = desc_k_major_sw128(st + (h == 0 ? C::kOffB0 : C::kOffB1));
                        // rows 64..127 of the slab are quarters 2 and 3 of its 128-row scale tile: two TMEM columns further
                        const std::uint32_t b_quarter = h == 0 ? 0U : 2U;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
#pragma unroll
                            for (int a = 0; a < 2; ++a) {
                                const std::uint64_t a_desc = desc_k_major_sw128(st + a * kTileM * kBlockKBytes);
                                mma_nvf4(accum + a * C::kN, a_desc + 2 * k, b_desc + 2 * k, idesc, sfc + a * 16 + k * 4,
                                         sfc + 32 + k * 4 + b_quarter, kb > 0 || k > 0);
                            }
                        }
                    }
                    tc_commit(empty_bar(stage));
                    sf_buffer ^= 1;
                    if (++stage == C::kStages) { stage = 0; phase ^= 1U; }
                }
                if (!ok) break;
                for (int h = 0; h < halves; ++h) {
                    tc_commit(accum_full(buffer[h]));
                    accum_phase ^= 1U << buffer[h];
                }
            }
        }
    } else {
        // epilogue: the code of expert_tc_kernel<0, 64>, once per half of the item
        const int quarter = warp & 3;
        const int sub = (warp - 2) >> 2;                  // 0..3: which 16-column chunk of every 64
        int next_buffer = 0;
        std::uint32_t accum_phase = 0;
        for (int item = blockIdx.x; item < total_items && !*abort_ptr; item += gridDim.x) {
            Item it;
            if (!decode_item<2 * C::kN>(p, route_table, item, &it)) continue;
            const int halves = it.valid > C::kN ? 2 : 1;
            const float alpha_g = p.bank.alpha[it.entry * 3 + 0];
            const float alpha_u = p.bank.alpha[it.entry * 3 + 1];
            const int inter = p.m_total;
            const int row0 = it.m_tile * kTileM + quarter * 32;
            bool ok = true;
            for (int hh = 0; hh < halves; ++hh) {
                const int buffer = next_buffer;
                next_buffer = (next_buffer + 1) % C::kAccumBuffers;
                if (!mbar_wait(accum_full(buffer), (accum_phase >> buffer) & 1U)) { give_up(); ok = false; break; }
                accum_phase ^= 1U << buffer;
                tc_fence_after();
                const int pp0 = it.pp0 + hh * C::kN;
                const int valid = hh == 0 ? min(C::kN, it.valid) : it.valid - C::kN;
                const std::uint32_t lane_base =
                    tmem_base + buffer * C::kAccumCols + (static_cast<std::uint32_t>(quarter * 32) << 16);
                std::uint8_t* hs_tile = p.hs + static_cast<std::size_t>(pp0 >> 7) * (inter / 64) * 512;
                std::uint8_t* hq_rows = p.hq + static_cast<std::size_t>(pp0) * (inter / 2);
                const int n_base = pp0 & 127;
                // Sixteen warps, sixteen (quarter, 16-column chunk) pieces per half: a warp has exactly one.  It takes its
                // piece into registers and gives the buffer back at once - the arithmetic that follows is several times
                // longer than the read, and the MMA lane needs two free buffers to start the next item.
                static_assert(C::kN == 16 * (C::kEpilogueWarps / 4), "one chunk per warp and half");
                const int c0 = sub * 16;
                const bool mine = c0 < valid;                                        // warp uniform
                std::uint32_t g[16], u[16];
                if (mine) {
                    tmem_load16(lane_base + c0, g);
                    tmem_load16(lane_base + C::kN + c0, u);
                    tmem_load_wait();
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(accum_empty(buffer));
                if (mine) swiglu_requant_chunk(g, u, alpha_g, alpha_u, p.quant_scale, lane, c0, valid, n_base, inter, row0, hq_rows, hs_tile);
            }
            if (!ok) break;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// ---- down product for large batches: the token slab stays in shared memory ---------------------------------
// In the tile-by-tile down kernel half of what a block loads is the token slab, fetched again for each of the 20
// row tiles of the weight, and a ring stage that waits for it is a stage less of weights in flight.  Here an item is (128-token slab of an expert, half of the row
// tiles): the slab's four K blocks (64 KB) and their scale slabs (8 KB) are loaded ONCE and stay resident, their
// scale factors stay in TMEM, and only weight chunks stream through the ring - half the bytes per result.
// Needs the whole K extent of a slab in shared memory: intermediate sizes up to 1024.
struct DownSlab {
    static constexpr int kN = 128;
    static constexpr int kKBlocksMax = 4;
    static constexpr int kBBytes = kKBlocksMax * (kN * kBlockKBytes + kSfSlab);     // 73,728
    static constexpr int kOffBSf = kKBlocksMax * kN * kBlockKBytes;                 // scale slabs behind the boxes
    static constexpr int kStages = 3;                                               // one chunk (two K blocks of the weight) each
    static constexpr int kStageBytes = kChunkBytes;
    static constexpr int kStoreBytes = 16 * 32 * 2;                                 // per epilogue warp (a group of four shares 4 KB): 16 tokens x 32 rows of BF16
    static constexpr int kAccumBuffers = 2;
    static constexpr int kSfbCols = kKBlocksMax * 16;                               // resident for an item
    static constexpr int kSfaCols = 2 * 16;                                         // per chunk, two buffers
    static constexpr int kTmemCols = 512;                                           // 2 * 128 + 64 + 2 * 32 = 384
    static constexpr int kBarriers = 2 + 2 * kStages + 2 * kAccumBuffers;
    static constexpr int kSmemBytes = kBBytes + kStages * kStageBytes + kEpilogueWarps * kStoreBytes + kBarriers * 8 + 16 + 1024;
    static constexpr int kGroups = 2;                                               // row-tile halves per slab
};

// Named barriers over the 128 threads of one epilogue group (barrier 0 is __syncthreads).
__device__ __forceinline__ void group_sync(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }
__device__ __forceinline__ bool group_all(bool mine, int id) {
    std::uint32_t all;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, %2, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(all)
        : "r"(static_cast<std::uint32_t>(mine)), "r"(id)
        : "memory");
    return all != 0U;
}

__global__ void __launch_bounds__(kThreadsTc, 1) expert_down_slab_kernel(const __grid_constant__ CUtensorMap map_b,
                                                                         const TcParams p) {
    using C = DownSlab;
    extern __shared__ std::uint8_t smem_raw[];
    __shared__ RouteTable route_table;
    const std::uint32_t base = (smem_u32(smem_raw) + 1023U) & ~1023U;
    const std::uint32_t ring = base + C::kBBytes;
    const std::uint32_t store_area = ring + C::kStages * C::kStageBytes;
    const std::uint32_t bars = store_area + kEpilogueWarps * C::kStoreBytes;
    const std::uint32_t b_full = bars, b_empty = bars + 8U;
    auto weight_bar = [&](int s) { return bars + 8U * (2 + s); };
    auto empty_bar = [&](int s) { return bars + 8U * (2 + C::kStages + s); };
    auto accum_full = [&](int b) { return bars + 8U * (2 + 2 * C::kStages + b); };
    auto accum_empty = [&](int b) { return bars + 8U * (2 + 2 * C::kStages + C::kAccumBuffers + b); };
    const std::uint32_t tmem_slot = bars + 8U * C::kBarriers;
    volatile std::uint32_t* tmem_slot_ptr =
        reinterpret_cast<volatile std::uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
    volatile std::uint32_t* abort_ptr = tmem_slot_ptr + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int k_blocks = p.k_bytes / kBlockKBytes;              // <= 4, even
    const int chunks = k_blocks / 2;
    const int tiles_per_group = p.m_tiles / C::kGroups;

    if (threadIdx.x == 0) {
        mbar_init(b_full, 1);
        mbar_init(b_empty, 1);
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(weight_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < C::kAccumBuffers; ++b) {
            mbar_init(accum_full(b), 1);
            mbar_init(accum_empty(b), kEpilogueWarps);
        }
        *abort_ptr = 0;
        fence_mbar_init();
        prefetch_tensormap(&map_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::kTmemCols);
        tmem_relinquish();
    }
    pdl_wait();                       // routing lists and the SwiGLU rows come from the kernels upstream
    load_route_table(p, &route_table);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_launch_dependents();
    const std::uint32_t tmem_base = *tmem_slot_ptr;
    const int total_items = route_table.prefix[route_table.active_count] * C::kGroups;      // the prefix counts 128-row slabs here
    auto give_up = [&]() {
        *abort_ptr = 1;
        atomicCAS(p.status, kStatusOk, kStatusWaitExpired);
    };
    // item -> (slab, first row tile); decode_item wants an index over (slab, row tile)
    auto decode = [&](int item, Item* it) {
        const int slab = item / C::kGroups;
        const int group = item - slab * C::kGroups;
        const bool ok = decode_item<C::kN>(p, route_table, slab * p.m_tiles + group * tiles_per_group, it);
        return ok;
    };

    if (warp == 0) {
        if (elect_one()) {
            int stage = 0;
            std::uint32_t phase = 0, b_phase = 0;
            for (int item = blockIdx.x; item < total_items && !*abort_ptr; item += gridDim.x) {
                Item it;
                if (!decode(item, &it)) continue;
                if (!mbar_wait(b_empty, b_phase ^ 1U)) { give_up(); break; }
                b_phase ^= 1U;
                mbar_arrive_expect_tx(b_full, k_blocks * (C::kN * kBlockKBytes + kSfSlab));
                for (int kb = 0; kb < k_blocks; ++kb) {
                    tma_load_2d(base + kb * C::kN * kBlockKBytes, &map_b, b_full, kb * kBlockKBytes, it.pp0);
                    bulk_load(base + C::kOffBSf + kb * kSfSlab,
                              p.b_sf + (static_cast<std::size_t>(it.pp0 >> 7) * (p.k_bytes / 32) + kb * 4) * 512, kSfSlab, b_full);
                }
                bool ok = true;
                for (int t = 0; t < tiles_per_group && ok; ++t) {
                    const int m_tile = it.m_tile + t;
                    for (int c = 0; c < chunks; ++c) {
                        if (!mbar_wait(empty_bar(stage), phase ^ 1U)) { give_up(); ok = false; break; }
                        mbar_arrive_expect_tx(weight_bar(stage), kChunkBytes);
                        bulk_load(ring + stage * C::kStageBytes,
                                  p.bank.g2 + ((static_cast<std::size_t>(it.entry) * p.m_tiles + m_tile) * chunks + c) * kChunkBytes,
                                  kChunkBytes, weight_bar(stage));
                        if (++stage == C::kStages) { stage = 0; phase ^= 1U; }
                    }
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            int stage = 0;
            std::uint32_t phase = 0, b_phase = 0;
            int buffer = 0;
            std::uint32_t accum_phase[2] = {0U, 0U};
            constexpr std::uint32_t idesc = idesc_nvf4(kTileM, C::kN);
            const std::uint32_t sfb_tmem = tmem_base + C::kAccumBuffers * C::kN;
            const std::uint32_t sfa_tmem = sfb_tmem + C::kSfbCols;
            int sfa_buffer = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < total_items && !*abort_ptr && ok; item += gridDim.x) {
                Item it;
                if (!decode(item, &it)) continue;
                if (!mbar_wait(b_full, b_phase)) { give_up(); break; }
                b_phase ^= 1U;
                tc_fence_after();
                // the slab's scale factors: 16 TMEM columns per K block, kept for the whole item
                for (int kb = 0; kb < k_blocks; ++kb) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        tc_copy_sf(sfb_tmem + kb * 16 + k * 4, desc_scale_atom(base + C::kOffBSf + kb * kSfSlab + k * 512));
                    }
                }
                for (int t = 0; t < tiles_per_group && ok; ++t) {
                    if (!mbar_wait(accum_empty(buffer), accum_phase[buffer] ^ 1U)) { give_up(); ok = false; break; }
                    tc_fence_after();
                    const std::uint32_t accum = tmem_base + buffer * C::kN;
                    for (int c = 0; c < chunks; ++c) {
                        if (!mbar_wait(weight_bar(stage), phase)) { give_up(); ok = false; break; }
                        tc_fence_after();
                        const std::uint32_t st = ring + stage * C::kStageBytes;
                        const std::uint32_t sfa = sfa_tmem + sfa_buffer * C::kSfaCols;
#pragma unroll
                        for (int o = 0; o < 2; ++o) {
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                tc_copy_sf(sfa + o * 16 + k * 4, desc_scale_atom(st + kChunkScaleOffset + o * kChunkScaleBytes + k * 512));
                            }
                        }
#pragma unroll
                        for (int o = 0; o < 2; ++o) {
                            const int kb = 2 * c + o;
                            const std::uint64_t a_desc = desc_k_major_sw128(st + o * kChunkBox);
                            const std::uint64_t b_desc = desc_k_major_sw128(base + kb * C::kN * kBlockKBytes);
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                mma_nvf4(accum, a_desc + 2 * k, b_desc + 2 * k, idesc, sfa + o * 16 + k * 4,
                                         sfb_tmem + kb * 16 + k * 4, kb > 0 || k > 0);
                            }
                        }
                        tc_commit(empty_bar(stage));
                        sfa_buffer ^= 1;
                        if (++stage == C::kStages) { stage = 0; phase ^= 1U; }
                    }
                    if (!ok) break;
                    tc_commit(accum_full(buffer));
                    accum_phase[buffer] ^= 1U;
                    buffer ^= 1;
                }
                if (!ok) break;
                tc_commit(b_empty);           // every product that reads the slab has been issued and will have completed
            }
        }
    } else {
        const int quarter = warp & 3;
        const int sub = (warp - 2) >> 2;
        int buffer = 0;
        std::uint32_t accum_phase[2] = {0U, 0U};
        bool ok = true;
        for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
            if (!group_all(*abort_ptr == 0U, 1 + sub)) break;       // the four warps of a group leave together
            Item it;
            if (!decode(item, &it)) continue;
            const float alpha = p.bank.alpha[it.entry * 3 + 2];
            const int hidden = p.m_total;
            for (int t = 0; t < tiles_per_group; ++t) {
                // the four warps of a group (one per 32-lane quarter of the accumulator) move in step: they share a
                // staging area and its barriers, so a wait that ran out in one of them ends the tile for all four
                if (!group_all(mbar_wait(accum_full(buffer), accum_phase[buffer]), 1 + sub)) { give_up(); ok = false; break; }
                accum_phase[buffer] ^= 1U;
                tc_fence_after();
                const std::uint32_t lane_base = tmem_base + buffer * C::kN + (static_cast<std::uint32_t>(quarter * 32) << 16);
                // A lane holds one weight row for 16 tokens; the output is token-major, so 2-byte stores would touch a
                // 64-byte piece per instruction.  The group turns its 128 x 16 block round through 4 KB of shared
                // memory and every lane stores 16 bytes: a token's 128 rows leave as one 256-byte run, which is what
                // keeps a store that crosses NVLink (TcIo::row_dest) efficient.
                std::uint16_t* stage_rows = reinterpret_cast<std::uint16_t*>(smem_raw + (store_area - smem_u32(smem_raw))) +
                                            sub * (4 * C::kStoreBytes / 2);
                const int first_row = (it.m_tile + t) * kTileM;
                // a warp's two chunks of 16 columns (sub * 16 and 64 + sub * 16) go into registers first and the buffer
                // back to the MMA lane at once; staging and stores follow
                constexpr int kChunks = C::kN / (16 * (kEpilogueWarps / 4));
                static_assert(kChunks == 2, "two chunks per warp and tile");
                std::uint32_t d[kChunks][16];
#pragma unroll
                for (int q = 0; q < kChunks; ++q) {
                    const int c0 = sub * 16 + q * 16 * (kEpilogueWarps / 4);
                    if (c0 < it.valid) tmem_load16(lane_base + c0, d[q]);              // group uniform
                }
                tmem_load_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(accum_empty(buffer));
                buffer ^= 1;
#pragma unroll
                for (int q = 0; q < kChunks; ++q) {
                    const int c0 = sub * 16 + q * 16 * (kEpilogueWarps / 4);
                    if (c0 >= it.valid) break;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        stage_rows[j * kTileM + quarter * 32 + lane] = float_to_bf16_bits(__uint_as_float(d[q][j]) * alpha);
                    }
                    group_sync(1 + sub);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int v = lane + 32 * h;                 // this warp: 4 tokens x 16 pieces of 16 bytes
                        const int j = quarter * 4 + (v >> 4);
                        const int n = c0 + j;
                        if (n < it.valid) {
                            std::uint16_t* to = p.row_dest != nullptr ? p.row_dest[it.pp0 + n]
                                                                      : p.out + static_cast<std::size_t>(it.pp0 + n) * hidden;
                            *reinterpret_cast<uint4*>(to + first_row + (v & 15) * 8) =
                                *reinterpret_cast<const uint4*>(stage_rows + j * kTileM + (v & 15) * 8);
                        }
                    }
                    group_sync(1 + sub);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// Quantises the token rows into the padded position space of the tensor-core
// kernels: row pp gets the NVFP4 bytes of its token, and the scales go straight
// into the 128x4-tiled layout (cuda/nvfp4_ops.cu:818-841 and :869-890 in one pass).
// One warp per TOKEN: the row is read and quantised once (lane l owns 16-element blocks l, l+32, ...)
// and written to the nine places it is needed, its eight routed slots and its shared-expert row.
__global__ void __launch_bounds__(256) quantize_padded_kernel(const std::uint16_t* __restrict__ x,
                                                              const std::int32_t* __restrict__ pp_of_flat,
                                                              std::uint8_t* __restrict__ xq,
                                                              std::uint8_t* __restrict__ xs, int rows, int hidden,
                                                              float global_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (token >= rows) return;
    const int blocks = hidden / 16;
    const int col_blocks = (blocks + 3) / 4;
    constexpr int kMaxPerLane = 8;                   // hidden <= 4096
    uint2 packed[kMaxPerLane];
    std::uint32_t scale_word[kMaxPerLane];           // lanes 0, 4, 8, ...: the scales of four neighbouring blocks
    // the nine destinations of the row, fetched before the row itself so that the stores wait for nothing
    const int place_index = lane < kTop ? token * kTop + lane : rows * kTop + token;
    const int my_pp = lane <= kTop ? __ldg(pp_of_flat + place_index) : 0;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
        const int b = lane + 32 * j;
        std::uint8_t scale_bits = 0;
        if (b < blocks) {                            // blocks is a multiple of 4: a quad of lanes is in or out together
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
            packed[j] = quantize_block16(v, global_scale, &scale_bits);
        }
        std::uint32_t word = scale_bits;
        word |= __shfl_down_sync(0xffffffffU, word, 1) << 8;
        word |= __shfl_down_sync(0xffffffffU, word, 2) << 16;
        scale_word[j] = word;
    }
#pragma unroll 1
    for (int place = 0; place <= kTop; ++place) {
        const std::size_t pp = static_cast<std::size_t>(__shfl_sync(0xffffffffU, my_pp, place));
        std::uint8_t* row_q = xq + pp * (hidden / 2);
        std::uint8_t* row_s = xs + (pp >> 7) * col_blocks * 512 + (pp & 31) * 16 + ((pp >> 5) & 3) * 4;
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) {
            const int b = lane + 32 * j;
            if (b >= blocks) break;
            *reinterpret_cast<uint2*>(row_q + b * 8) = packed[j];
            if ((lane & 3) == 0) *reinterpret_cast<std::uint32_t*>(row_s + (b >> 2) * 512) = scale_word[j];
        }
    }
}

// The same for rows that each have ONE destination (the dense MLP's token rows, the (row, slot) intermediate rows
// of the down stage entry point): row i of `x` [n][width] goes to padded position index[i] (i itself if index is null).
__global__ void __launch_bounds__(256) quantize_rows_to_pp_kernel(const std::uint16_t* __restrict__ x,
                                                                  const std::int32_t* __restrict__ index,
                                                                  std::uint8_t* __restrict__ xq,
                                                                  std::uint8_t* __restrict__ xs, int n, int width,
                                                                  float global_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n) return;
    const int blocks = width / 16;
    const int col_blocks = (blocks + 3) / 4;
    const std::size_t pp = static_cast<std::size_t>(index != nullptr ? index[row] : row);
    std::uint8_t* row_q = xq + pp * (width / 2);
    std::uint8_t* row_s = xs + (pp >> 7) * col_blocks * 512 + (pp & 31) * 16 + ((pp >> 5) & 3) * 4;
    for (int b = lane; b < blocks; b += 32) {
        const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<std::size_t>(row) * width + b * 16);
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
        const uint2 packed = quantize_block16(v, global_scale, &scale_bits);
        *reinterpret_cast<uint2*>(row_q + b * 8) = packed;
        row_s[(b >> 2) * 512 + (b & 3)] = scale_bits;
    }
}

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled fn = nullptr;
    if (fn == nullptr) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &query) == cudaSuccess &&
            query == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiled>(sym);
        }
    }
    return fn;
}

template <int MODE, int N, int SRC = 0>
cudaError_t launch_tc(const p92b_plan* plan, const CUtensorMap& map_b, const TcParams& p, cudaStream_t stream,
                      bool pdl) {
    using C = Tc<MODE, N>;
    auto kernel = expert_tc_kernel<MODE, N, SRC>;
    if (cudaError_t st = ensure_dynamic_smem<expert_tc_kernel<MODE, N, SRC>>(C::kSmemBytes); st != cudaSuccess) return st;
    return launch_kernel(kernel, dim3(plan->sm_count), dim3(kThreadsTc), C::kSmemBytes, stream, pdl, map_b, p);
}

}  // namespace

// Row-major byte matrix [rows][row_bytes] as a 2-D tensor map with a 128-byte x box_rows box and
// the 128-byte swizzle (what the K-major operand descriptors expect).
cudaError_t make_operand_map(CUtensorMap* map, const void* base, std::size_t rows, std::size_t row_bytes,
                             int box_rows) {
    EncodeTiled encode = encode_tiled();
    if (encode == nullptr) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBlockKBytes), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// Token tile of the expert kernels.  Above 32 rows it stays at 64 columns: two gate/up accumulator pairs
// then fit TMEM side by side, so the epilogue of one tile overlaps the MMAs of the next.
int tc_tile_rows(int rows) { return rows <= 16 ? 16 : rows <= 32 ? 32 : 64; }
// Every entry's rows start on a multiple of 128 padded positions, so a token tile always begins at
// row 0 of a 128-row scale-factor tile (TMEM lane 0, first scale column).
int tc_pad_align(int rows) { (void)rows; return 128; }

cudaError_t launch_quantize_padded(const p92b_plan* plan, const std::uint16_t* x, int rows, cudaStream_t stream,
                                   bool pdl) {
    if (plan->hidden > 4096) return cudaErrorNotSupported;
    const int warps = rows;                        // one per token
    return launch_kernel(quantize_padded_kernel, dim3((warps + 7) / 8), dim3(256), 0, stream, pdl, x,
                         static_cast<const std::int32_t*>(plan->pp_of_flat), plan->xq_pp, plan->xs_sw, rows,
                         plan->hidden, 1.0F);
}

cudaError_t launch_quantize_rows_to_pp(const std::uint16_t* x, const std::int32_t* index, std::uint8_t* xq,
                                       std::uint8_t* xs, int n, int width, cudaStream_t stream, bool pdl) {
    if (x == nullptr || xq == nullptr || xs == nullptr || n <= 0 || width <= 0 || width % 64 != 0) return cudaErrorInvalidValue;
    return launch_kernel(quantize_rows_to_pp_kernel, dim3((n + 7) / 8), dim3(256), 0, stream, pdl, x, index, xq, xs, n, width,
                         1.0F);
}

namespace {
bool slab_shape(const p92b_plan* plan) {
    const int k_blocks = plan->intermediate / 2 / kBlockKBytes;
    return plan->wide_rows == 128 && k_blocks <= DownSlab::kKBlocksMax && k_blocks % 2 == 0 &&
           (plan->hidden / kTileM) % DownSlab::kGroups == 0 && std::getenv("P92B_NO_DOWN_SLAB") == nullptr;
}
}  // namespace

bool down_slab_applies(const p92b_plan* plan, int rows) { return tc_tile_rows(rows) == 64 && slab_shape(plan); }

cudaError_t launch_experts_tc(const p92b_plan* plan, const p92b_bank* bank, int rows, bool down,
                              cudaStream_t stream, bool pdl, const TcIo* io) {
    const bool in_place = io != nullptr && io->table != nullptr;
    if (!plan->tc_ready || (!in_place && (bank == nullptr || !bank->tc_ready))) return cudaErrorNotSupported;
    TcParams p {};
    if (bank != nullptr) p.bank = bank->view;
    p.route.counts = plan->counts;
    p.route.offsets = plan->offsets;
    p.route.row_token = plan->row_token;
    p.route.active = plan->active;
    p.route.active_count = plan->active_count;
    p.pp_off = plan->pp_off;
    p.tile_prefix = plan->tile_prefix;
    p.status = plan->status;
    p.quant_scale = 1.0F;
    if (io != nullptr) {
        p.out_row = io->out_row;
        p.gate_out = io->gate_out;
        p.up_out = io->up_out;
        p.table = io->table;
        p.table_kind = io->table_kind;
        p.skip_shared = io->skip_shared ? 1 : 0;
        p.row_dest = io->row_dest;
    }
    const bool unfused = io != nullptr && io->gate_out != nullptr;
    const bool single = io != nullptr && io->single_matrix;      // one matrix of the token-row side (gate or up alone)
    const int n = tc_tile_rows(rows);
    const int which = n == 16 ? 0 : n == 32 ? 1 : 2;
    p.routing_is_upstream = down && !(io != nullptr && io->wait_upstream) ? 0 : 1;
    if (!down) {
        p.b_sf = plan->xs_sw;
        p.hq = plan->hq_pp;
        p.hs = plan->hs_sw;
        p.k_bytes = plan->hidden / 2;
        p.m_total = plan->intermediate;
        p.m_tiles = plan->intermediate / kTileM;
        if (single) {
            if (!in_place || io->down_out == nullptr) return cudaErrorInvalidValue;
            p.out = io->down_out;
            switch (which) {
                case 0: return launch_tc<1, 16, 1>(plan, plan->map_x[0], p, stream, pdl);
                case 1: return launch_tc<1, 32, 1>(plan, plan->map_x[1], p, stream, pdl);
                default: return launch_tc<1, 64, 1>(plan, plan->map_x[2], p, stream, pdl);
            }
        }
        if (unfused) {
            if (io->up_out == nullptr) return cudaErrorInvalidValue;
            switch (which) {
                case 0: return in_place ? launch_tc<2, 16, 1>(plan, plan->map_x[0], p, stream, pdl)
                                        : launch_tc<2, 16, 0>(plan, plan->map_x[0], p, stream, pdl);
                case 1: return in_place ? launch_tc<2, 32, 1>(plan, plan->map_x[1], p, stream, pdl)
                                        : launch_tc<2, 32, 0>(plan, plan->map_x[1], p, stream, pdl);
                default: return in_place ? launch_tc<2, 64, 1>(plan, plan->map_x[2], p, stream, pdl)
                                         : launch_tc<2, 64, 0>(plan, plan->map_x[2], p, stream, pdl);
            }
        }
        if (in_place) return cudaErrorNotSupported;              // the fused gate/up epilogue reads the bank's stream
        switch (which) {
            case 0: return launch_tc<0, 16>(plan, plan->map_x[0], p, stream, pdl);
            case 1: return launch_tc<0, 32>(plan, plan->map_x[1], p, stream, pdl);
            default:
                if (plan->wide_rows == 128 && std::getenv("P92B_NO_GU_PAIR") == nullptr) {
                    // large batches: pairs of 64-row token tiles share one weight stage (one 128-column tile was
                    // tried too: a single accumulator buffer and three stages then, 377 µs against 283 µs at T=4096)
                    p.tile_prefix = plan->tile_prefix_wide;
                    if (cudaError_t st = ensure_dynamic_smem<expert_gu_pair_kernel>(GuPair::kSmemBytes); st != cudaSuccess) return st;
                    return launch_kernel(expert_gu_pair_kernel, dim3(plan->sm_count), dim3(GuPair::kThreads), GuPair::kSmemBytes,
                                         stream, pdl, plan->map_x[2], p);
                }
                return launch_tc<0, 64>(plan, plan->map_x[2], p, stream, pdl);
        }
    }
    p.b_sf = plan->hs_sw;
    p.out = io != nullptr && io->down_out != nullptr ? io->down_out : plan->mixed_pp;
    p.k_bytes = plan->intermediate / 2;
    p.m_total = plan->hidden;
    p.m_tiles = plan->hidden / kTileM;
    if (in_place) {
        switch (which) {
            case 0: return launch_tc<1, 16, 1>(plan, plan->map_h[0], p, stream, pdl);
            case 1: return launch_tc<1, 32, 1>(plan, plan->map_h[1], p, stream, pdl);
            default: return launch_tc<1, 64, 1>(plan, plan->map_h[2], p, stream, pdl);
        }
    }
    if (p.row_dest != nullptr && which != 2) return cudaErrorNotSupported;
    switch (which) {
        case 0: return launch_tc<1, 16>(plan, plan->map_h[0], p, stream, pdl);
        case 1: return launch_tc<1, 32>(plan, plan->map_h[1], p, stream, pdl);
        default:
            if (plan->wide_rows == 128) {
                // every expert segment starts on a multiple of 128 padded rows, so 128-row tiles stay inside it
                p.tile_prefix = plan->tile_prefix_wide;
                const bool plain = io == nullptr || (io->down_out == nullptr && io->out_row == nullptr && !io->skip_shared);
                if (plain && slab_shape(plan)) {
                    // the token slab resident in shared memory, only weights streaming
                    if (cudaError_t st = ensure_dynamic_smem<expert_down_slab_kernel>(DownSlab::kSmemBytes); st != cudaSuccess) return st;
                    return launch_kernel(expert_down_slab_kernel, dim3(plan->sm_count), dim3(kThreadsTc), DownSlab::kSmemBytes,
                                         stream, pdl, plan->map_h[3], p);
                }
                if (p.row_dest != nullptr) return cudaErrorNotSupported;
                return launch_tc<1, 128>(plan, plan->map_h[3], p, stream, pdl);
            }
            if (p.row_dest != nullptr) return cudaErrorNotSupported;
            return launch_tc<1, 64>(plan, plan->map_h[2], p, stream, pdl);
    }
}

// Rows that the caller has already quantised in the reference's layout (packed [R][K/2], scales 128x4-tiled over
// the R rows): assignment i takes source row src_row (i itself, or its token i / 8 when the eight slots of a token
// share one row) and is copied to padded position pp_of_flat[i], its scale bytes to the tiled position of that row.
namespace {
__global__ void __launch_bounds__(256) gather_quantized_rows_kernel(const std::uint8_t* __restrict__ packed,
                                                                    const std::uint8_t* __restrict__ scales_swizzled,
                                                                    const std::int32_t* __restrict__ pp_of_flat,
                                                                    std::uint8_t* __restrict__ xq, std::uint8_t* __restrict__ xs,
                                                                    int assignments, int k_bytes, int distinct_rows) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= assignments) return;
    const std::size_t src = static_cast<std::size_t>(distinct_rows ? i : i / kTop);
    const std::size_t pp = static_cast<std::size_t>(pp_of_flat[i]);
    const uint4* from = reinterpret_cast<const uint4*>(packed + src * k_bytes);
    uint4* to = reinterpret_cast<uint4*>(xq + pp * k_bytes);
    for (int v = lane; v < k_bytes / 16; v += 32) to[v] = __ldg(from + v);
    const int scale_columns = k_bytes / 8;                       // K / 16
    const int col_blocks = (scale_columns + 3) / 4;
    const std::uint8_t* sf_from = scales_swizzled + (src >> 7) * col_blocks * 512 + (src & 31) * 16 + ((src >> 5) & 3) * 4;
    std::uint8_t* sf_to = xs + (pp >> 7) * col_blocks * 512 + (pp & 31) * 16 + ((pp >> 5) & 3) * 4;
    for (int c = lane; c < scale_columns; c += 32) sf_to[(c >> 2) * 512 + (c & 3)] = sf_from[(c >> 2) * 512 + (c & 3)];
}
}  // namespace

cudaError_t launch_gather_quantized_rows(const std::uint8_t* packed, const std::uint8_t* scales_swizzled,
                                         const std::int32_t* pp_of_flat, std::uint8_t* xq, std::uint8_t* xs, int assignments,
                                         int k_bytes, bool distinct_rows, cudaStream_t stream, bool pdl) {
    if (packed == nullptr || scales_swizzled == nullptr || assignments <= 0 || k_bytes % 16 != 0 ||
        (reinterpret_cast<std::uintptr_t>(packed) & 15U) != 0U) {
        return cudaErrorInvalidValue;
    }
    return launch_kernel(gather_quantized_rows_kernel, dim3((assignments + 7) / 8), dim3(256), 0, stream, pdl, packed,
                         scales_swizzled, pp_of_flat, xq, xs, assignments, k_bytes, distinct_rows ? 1 : 0);
}

}  // namespace p92b
