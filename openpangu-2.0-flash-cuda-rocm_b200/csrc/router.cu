// Router: BF16 logits in the reference's two FP32 summation orders, and the
// sigmoid + correction-bias top-8 with renormalised weights.
//
// Bit-exactness contract.  Expert ids must equal the reference's, so the logits
// reproduce its FP32 fmaf chains and reduction trees value for value:
//   T == 1 (cuda/nvfp4_ops.cu:161-176): thread t of 256 sums columns t, t+256, ...;
//           warp shuffle-down tree; tree over the 8 warp sums (block_sum, :38-51).
//   T  > 1 (cuda/nvfp4_ops.cu:178-207): lane l of a warp sums columns l, l+32, ...;
//           warp shuffle-down tree.
// The score is written as the reference writes it, 1/(1+expf(-x)), and this
// file is compiled with --use_fast_math like the reference (CMakeLists.txt:98)
// so expf and the divisions lower to the same hardware approximations.
// Selection is pure comparison with ties to the lower id, which is order
// independent, so the top-8 itself is free to use a warp-per-token layout.
#include "p92b_common.cuh"

#include <cstdlib>
#include "tc_ptx.cuh"

#include <cfloat>

namespace p92b {

using ptx::pdl_launch_dependents;
using ptx::pdl_wait;

namespace {

// ---- T == 1 order ---------------------------------------------------------
// One block of 256 threads per expert row; thread t owns columns t + 256 j.
// The 5 KB row is one fully coalesced pass (ten 512-byte warp requests).
__global__ void __launch_bounds__(256) logits_gemv_kernel(const std::uint16_t* __restrict__ x,
                                                          const std::uint16_t* __restrict__ w,
                                                          float* __restrict__ out, int rows,
                                                          int columns) {
    const int row = blockIdx.x;
    if (row >= rows) return;
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float warp_sums[8];
    const std::uint16_t* wr = w + static_cast<std::size_t>(row) * columns;
    float value = 0.0F;
    for (int c = threadIdx.x; c < columns; c += 256) {
        value = fmaf(bf16_bits_to_float(x[c]), bf16_bits_to_float(wr[c]), value);
    }
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_down_sync(0xffffffffU, value, offset);
    if (lane == 0) warp_sums[warp] = value;
    __syncthreads();
    if (warp == 0) {
        value = lane < 8 ? warp_sums[lane] : 0.0F;
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_down_sync(0xffffffffU, value, offset);
        if (lane == 0) out[row] = value;
    }
}

// ---- T > 1 order ----------------------------------------------------------
// A warp owns a TE x TT tile of (expert, token) outputs; lane l accumulates the
// columns l, l+32, ... of every output in the tile (the reference's per-lane
// chain), so one pass over K yields TE*TT fmaf per TE+TT shared-memory reads,
// and the final shuffle-down tree is the reference's.  K is staged through
// shared memory in ascending chunks, which keeps each chain's order.
template <int TE, int TT, int WE, int WT>
__global__ void __launch_bounds__(WE* WT * 32) logits_rows_kernel(
    const std::uint16_t* __restrict__ x, const std::uint16_t* __restrict__ w,
    float* __restrict__ out, int batch_rows, int rows, int columns, int kc) {
    constexpr int BE = TE * WE;             // experts per block
    constexpr int BT = TT * WT;             // tokens per block
    constexpr int THREADS = WE * WT * 32;
    extern __shared__ __align__(16) std::uint16_t staged[];
    std::uint16_t* ws = staged;                                 // [BE][kc]
    std::uint16_t* xs = staged + static_cast<std::size_t>(BE) * kc;   // [BT][kc]
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int we = warp % WE;
    const int wt = warp / WE;
    const int e0 = blockIdx.x * BE;
    const int t0 = blockIdx.y * BT;
    const int kc8 = kc / 8;
    float acc[TE][TT];
#pragma unroll
    for (int i = 0; i < TE; ++i)
#pragma unroll
        for (int j = 0; j < TT; ++j) acc[i][j] = 0.0F;

    pdl_launch_dependents();
    for (int k0 = 0; k0 < columns; k0 += kc) {
        if (k0 != 0) __syncthreads();
        // 16-byte coalesced staging; rows beyond the edge are zero filled.  The router weight does
        // not depend on the upstream kernel, the token rows do.
        for (int idx = threadIdx.x; idx < BE * kc8; idx += THREADS) {
            const int r = idx / kc8;
            const int c8 = idx - r * kc8;
            uint4 v = make_uint4(0U, 0U, 0U, 0U);
            if (e0 + r < rows) {
                v = *reinterpret_cast<const uint4*>(w + static_cast<std::size_t>(e0 + r) * columns + k0 + c8 * 8);
            }
            *reinterpret_cast<uint4*>(ws + static_cast<std::size_t>(r) * kc + c8 * 8) = v;
        }
        if (k0 == 0) pdl_wait();
        for (int idx = threadIdx.x; idx < BT * kc8; idx += THREADS) {
            const int r = idx / kc8;
            const int c8 = idx - r * kc8;
            uint4 v = make_uint4(0U, 0U, 0U, 0U);
            if (t0 + r < batch_rows) {
                v = *reinterpret_cast<const uint4*>(x + static_cast<std::size_t>(t0 + r) * columns + k0 + c8 * 8);
            }
            *reinterpret_cast<uint4*>(xs + static_cast<std::size_t>(r) * kc + c8 * 8) = v;
        }
        __syncthreads();
#pragma unroll 4
        for (int j = 0; j < kc / 32; ++j) {
            float wv[TE];
            float xv[TT];
#pragma unroll
            for (int i = 0; i < TE; ++i) wv[i] = bf16_bits_to_float(ws[static_cast<std::size_t>(we * TE + i) * kc + j * 32 + lane]);
#pragma unroll
            for (int i = 0; i < TT; ++i) xv[i] = bf16_bits_to_float(xs[static_cast<std::size_t>(wt * TT + i) * kc + j * 32 + lane]);
#pragma unroll
            for (int i = 0; i < TE; ++i)
#pragma unroll
                for (int t = 0; t < TT; ++t) acc[i][t] = fmaf(xv[t], wv[i], acc[i][t]);
        }
    }
#pragma unroll
    for (int i = 0; i < TE; ++i) {
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            float value = acc[i][t];
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_down_sync(0xffffffffU, value, offset);
            const int e = e0 + we * TE + i;
            const int tok = t0 + wt * TT + t;
            if (lane == 0 && e < rows && tok < batch_rows) out[static_cast<std::size_t>(tok) * rows + e] = value;
        }
    }
}

// ---- T > 1 order, large batches ----------------------------------------------
// Same per-lane chains as above, organised for throughput: a block of four warps computes 16 experts x
// 16 tokens, a warp 8 x 8 of them.  K advances in chunks of 256 columns that sit TRANSPOSED in shared
// memory - element (row, column l + 32 j) at [row][l][j] - so that a lane fetches its eight j-values of
// a row with one 16-byte read.  A chunk arrives by asynchronous 16-byte copies issued a whole chunk ahead
// (no registers; loading into registers instead left the global latency exposed: 274 µs against 230 µs
// at T=4096; one 512-byte bulk copy of the TMA unit per row was slower too: 242 µs against 199 µs), and is
// transposed inside shared memory with 16-byte reads, byte permutes and 8-byte
// stores laid out so that every bank is hit exactly twice per instruction, the minimum for 256 bytes.
// Two buffers of each image, one block synchronisation per chunk.  The fmaf order of every
// chain is still j ascending; the multiply uses the two-wide FP32 fused multiply-add of sm_100, each half
// of which is an ordinary round-to-nearest fmaf.
__device__ __forceinline__ void async_copy16(std::uint32_t dst_smem, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;          // 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(bytes) : "memory");
}

template <int MIN_BLOCKS>
__global__ void __launch_bounds__(128, MIN_BLOCKS) logits_rows_large_kernel(const std::uint16_t* __restrict__ x,
                                                                           const std::uint16_t* __restrict__ w,
                                                                           float* __restrict__ out, int batch_rows, int rows,
                                                                           int columns) {
    constexpr int TE = 8, TT = 8, WE = 2, WT = 2, KC = 256;
    constexpr int BE = TE * WE, BT = TT * WT, ROWS = BE + BT;      // 16 expert rows + 16 token rows
    constexpr int ROW_WORDS = 32 * 4 + 4;                           // 512 bytes + 16 bytes of padding
    static_assert(ROWS == 32, "one transposition unit per thread: 32 rows x 2 j-quads x 2 lane halves = 128 threads");
    extern __shared__ __align__(16) std::uint8_t large_smem[];
    std::uint32_t (*raw)[ROWS][ROW_WORDS] = reinterpret_cast<std::uint32_t (*)[ROWS][ROW_WORDS]>(large_smem);
    std::uint32_t (*tile)[ROWS][ROW_WORDS] =
        reinterpret_cast<std::uint32_t (*)[ROWS][ROW_WORDS]>(large_smem + 2 * ROWS * ROW_WORDS * 4);
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int we = warp % WE, wt = warp / WE;
    const int e0 = blockIdx.x * BE, t0 = blockIdx.y * BT;
    float2 acc[TE][TT / 2];
#pragma unroll
    for (int i = 0; i < TE; ++i)
#pragma unroll
        for (int j = 0; j < TT / 2; ++j) acc[i][j] = make_float2(0.0F, 0.0F);

    // global -> raw image, asynchronously: 32 rows x 32 pieces of 16 bytes, eight per thread, consecutive
    // threads on consecutive pieces of a row
    auto fetch = [&](int k0, int buffer) {
#pragma unroll
        for (int q = 0; q < ROWS * 32 / 128; ++q) {
            const int idx = threadIdx.x + q * 128;
            const int r = idx >> 5, piece = idx & 31;
            const bool is_w = r < BE;
            const int src_row = is_w ? e0 + r : t0 + (r - BE);
            const bool ok = is_w ? src_row < rows : src_row < batch_rows;
            const std::uint16_t* src = (is_w ? w : x) + static_cast<std::size_t>(ok ? src_row : 0) * columns + k0 + piece * 8;
            async_copy16(static_cast<std::uint32_t>(__cvta_generic_to_shared(&raw[buffer][r][piece * 4])), src, ok);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // raw image -> transposed image.  A thread takes, for one row, four j-values (j = 4q .. 4q+3) of sixteen
    // neighbouring lanes: eight 16-byte reads, byte permutes, sixteen 8-byte stores whose lanes are spread
    // over sixteen rows and both j-quads, so every bank is hit exactly twice per instruction.
    const int s_row = (warp >> 1) * 16 + (lane >> 4) * 8 + (lane & 7);
    const int s_q = (lane >> 3) & 1;
    const int s_side = warp & 1;
    auto transpose = [&](int buffer) {
        const uint4* src = reinterpret_cast<const uint4*>(&raw[buffer][s_row][(128 * s_q + 16 * s_side) / 2]);
        std::uint32_t* row = &tile[buffer][s_row][0];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 p0 = src[h], p1 = src[4 + h], p2 = src[8 + h], p3 = src[12 + h];     // j = 4q .. 4q+3: 64 bytes apart
            const std::uint32_t words[4][4] = {{p0.x, p0.y, p0.z, p0.w}, {p1.x, p1.y, p1.z, p1.w},
                                               {p2.x, p2.y, p2.z, p2.w}, {p3.x, p3.y, p3.z, p3.w}};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const unsigned select = (i & 1) ? 0x7632U : 0x5410U;       // the high or the low BF16 of both words
                const int l = 16 * s_side + 8 * h + i;
                uint2 v;
                v.x = __byte_perm(words[0][i >> 1], words[1][i >> 1], select);     // j = 4q, 4q+1
                v.y = __byte_perm(words[2][i >> 1], words[3][i >> 1], select);     // j = 4q+2, 4q+3
                *reinterpret_cast<uint2*>(row + l * 4 + 2 * s_q) = v;
            }
        }
    };
    fetch(0, 0);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (KC < columns) fetch(KC, 1);
    transpose(0);
    int buffer = 0;
    for (int k0 = 0; k0 < columns; k0 += KC) {
        // chunk k0 is transposed in tile[buffer] (by every thread: not yet visible), chunk k0 + KC is arriving in raw[buffer ^ 1]
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (k0 + KC < columns) {
            if (k0 + 2 * KC < columns) fetch(k0 + 2 * KC, buffer);   // raw[buffer] was transposed before the barrier
            transpose(buffer ^ 1);                                    // tile[buffer ^ 1] was last read before the barrier
        }
        uint4 wv[TE], xv[TT];
#pragma unroll
        for (int i = 0; i < TE; ++i) wv[i] = *reinterpret_cast<const uint4*>(&tile[buffer][we * TE + i][lane * 4]);
#pragma unroll
        for (int i = 0; i < TT; ++i) xv[i] = *reinterpret_cast<const uint4*>(&tile[buffer][BE + wt * TT + i][lane * 4]);
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
            float wf[TE], xf[TT];
#pragma unroll
            for (int i = 0; i < TE; ++i) {
                const std::uint32_t word = jj < 2 ? wv[i].x : jj < 4 ? wv[i].y : jj < 6 ? wv[i].z : wv[i].w;
                wf[i] = __uint_as_float((jj & 1) ? (word & 0xffff0000U) : (word << 16));
            }
#pragma unroll
            for (int i = 0; i < TT; ++i) {
                const std::uint32_t word = jj < 2 ? xv[i].x : jj < 4 ? xv[i].y : jj < 6 ? xv[i].z : xv[i].w;
                xf[i] = __uint_as_float((jj & 1) ? (word & 0xffff0000U) : (word << 16));
            }
#pragma unroll
            for (int i = 0; i < TE; ++i) {
                const float2 w2 = make_float2(wf[i], wf[i]);
#pragma unroll
                for (int t = 0; t < TT / 2; ++t) acc[i][t] = __ffma2_rn(make_float2(xf[2 * t], xf[2 * t + 1]), w2, acc[i][t]);
            }
        }
        buffer ^= 1;
    }
#pragma unroll
    for (int i = 0; i < TE; ++i) {
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            float value = (t & 1) ? acc[i][t / 2].y : acc[i][t / 2].x;
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_down_sync(0xffffffffU, value, offset);
            const int e = e0 + we * TE + i;
            const int tok = t0 + wt * TT + t;
            if (lane == 0 && e < rows && tok < batch_rows) out[static_cast<std::size_t>(tok) * rows + e] = value;
        }
    }
}

// ---- top-8 ----------------------------------------------------------------
// One warp per token; lane l holds experts l, l+32, ..., l+224 in registers.
// Eight rounds of (local best, warp butterfly arg-max) with the reference's
// total order: higher corrected score first, equal scores -> lower id
// (cuda/nvfp4_ops.cu:391-392,411-412).  Weights are the uncorrected sigmoid of
// the winners, summed in slot order and scaled by routed_scale/total (:420,425-432).
__global__ void __launch_bounds__(128) router_top8_kernel(const float* __restrict__ logits,
                                                          const float* __restrict__ bias,
                                                          std::int32_t* __restrict__ ids,
                                                          float* __restrict__ weights, int rows,
                                                          float routed_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    warp_top8(logits + static_cast<std::size_t>(row) * kExperts, bias, ids + static_cast<std::size_t>(row) * 8,
              weights + static_cast<std::size_t>(row) * 8, routed_scale);
}

}  // namespace

cudaError_t launch_router_logits(const std::uint16_t* x, const std::uint16_t* w, float* out,
                                 int batch_rows, int rows, int columns, bool gemv_order,
                                 cudaStream_t stream, bool pdl) {
    if (x == nullptr || w == nullptr || out == nullptr || batch_rows <= 0 || rows <= 0 ||
        columns <= 0 || columns % 128 != 0) {
        return cudaErrorInvalidValue;
    }
    if (gemv_order) {
        if (batch_rows != 1) return cudaErrorInvalidValue;
        return launch_kernel(logits_gemv_kernel, dim3(rows), dim3(256), 0, stream, pdl, x, w, out, rows, columns);
    } else if (batch_rows <= 8) {
        // decode: the whole K extent of 2 expert rows and of every token sits in
        // shared memory, so all global loads of a block are in flight at once
        constexpr int TE = 1, TT = 8, WE = 4, WT = 1;
        const std::size_t smem = static_cast<std::size_t>(TE * WE + TT * WT) * columns * 2;
        if (smem > 200 * 1024) return cudaErrorInvalidValue;
        auto kernel = logits_rows_kernel<TE, TT, WE, WT>;
        if (cudaError_t st = ensure_dynamic_smem<logits_rows_kernel<TE, TT, WE, WT>>(200 * 1024); st != cudaSuccess) return st;
        dim3 grid((rows + TE * WE - 1) / (TE * WE), 1);
        return launch_kernel(kernel, grid, dim3(WE * WT * 32), smem, stream, pdl, x, w, out, batch_rows, rows, columns,
                             columns);
    } else if (batch_rows >= 256 && columns % 256 == 0) {
        // 16 experts x 16 tokens per block of four warps.  (Measured at T=4096 with the chunk copied asynchronously
        // into shared memory and transposed there: 230 µs with this block shape, 237 - 296 µs with three others.)
        dim3 grid((rows + 15) / 16, (batch_rows + 15) / 16);
        constexpr std::size_t smem = 4 * 32 * (32 * 4 + 4) * 4;     // raw and transposed images of 32 padded rows, two of each
        if (cudaError_t st = ensure_dynamic_smem<logits_rows_large_kernel<3>>(static_cast<int>(smem)); st != cudaSuccess) return st;
        return launch_kernel(logits_rows_large_kernel<3>, grid, dim3(128), smem, stream, pdl, x, w, out, batch_rows, rows,
                             columns);
    } else {
        constexpr int TE = 8, TT = 8, WE = 2, WT = 4;
        constexpr int KC = 128;
        const std::size_t smem = static_cast<std::size_t>(TE * WE + TT * WT) * KC * 2;
        dim3 grid((rows + TE * WE - 1) / (TE * WE), (batch_rows + TT * WT - 1) / (TT * WT));
        return launch_kernel(logits_rows_kernel<TE, TT, WE, WT>, grid, dim3(WE * WT * 32), smem, stream, pdl, x, w, out,
                             batch_rows, rows, columns, KC);
    }
}

cudaError_t launch_router_top8(const float* logits, const float* bias, std::int32_t* ids,
                               float* weights, int rows, float routed_scale, cudaStream_t stream, bool pdl) {
    if (logits == nullptr || bias == nullptr || ids == nullptr || weights == nullptr || rows <= 0) {
        return cudaErrorInvalidValue;
    }
    return launch_kernel(router_top8_kernel, dim3((rows + 3) / 4), dim3(128), 0, stream, pdl, logits, bias, ids, weights,
                         rows, routed_scale);
}

}  // namespace p92b
