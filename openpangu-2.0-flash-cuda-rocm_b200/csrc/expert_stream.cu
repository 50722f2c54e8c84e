// Weight-streaming expert kernels for small row counts (decode, MTP verify).
//
// At T <= a few dozen rows every routed expert sees one or two rows, so the
// expert products are GEMV-class and bound by streaming the NVFP4 weights from
// HBM once: 2 x 1.47 MB (gate, up) + 1.47 MB (down) per distinct expert.  These
// kernels therefore keep the math on the SIMT pipes and spend their design on
// the memory side: 16-byte fully coalesced weight loads, every load of a work
// item in flight before the first use, persistent blocks that walk (expert,
// row-tile) items so consecutive blocks stream consecutive DRAM pages.
//
// Arithmetic.  Both operands are NVFP4.  E2M1 pairs are widened to f16x2 with
// cvt.rn.f16x2.e2m1x2 (exact); the 16 products of one scale block are summed in
// two f16x2 chains of 8 (exact: every partial is a multiple of 1/4 below 2^9),
// then scaled by the two E4M3 block scales and accumulated in FP32.  The
// per-tensor FP32 scale (alpha) is applied to the FP32 sum and the result is
// rounded to BF16 where the reference rounds (D of the grouped GEMM,
// cuda/nvfp4_grouped.cu:195-204).  SwiGLU (cuda/nvfp4_ops.cu:97-105) and the
// re-quantisation of its BF16 result (src/executor.cpp:85-91,
// cuda/nvfp4_ops.cu:818-841) are fused into the gate/up kernel, so gate and up
// never travel through HBM.
#include "p92b_common.cuh"

namespace p92b {
namespace {

constexpr int kThreads = 256;
constexpr int kWarpsPerBlock = kThreads / 32;
constexpr int kGateUpRows = 2 * kWarpsPerBlock;   // 16 intermediate rows per item = one scale block
constexpr int kDownRowsPerWarp = 8;
constexpr int kDownRows = kDownRowsPerWarp * kWarpsPerBlock;   // 64 output rows per item

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ std::uint32_t ldg_u16(const void* p) {
    return static_cast<std::uint32_t>(__ldg(reinterpret_cast<const unsigned short*>(p)));
}

// 16 packed bytes -> 16 f16x2 registers (elements 2i, 2i+1 in register i).
__device__ __forceinline__ void decode16(const uint4& raw, std::uint32_t (&h)[16]) {
    const std::uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
        for (int b = 0; b < 4; ++b) h[wi * 4 + b] = e2m1x2_to_f16x2((words[wi] >> (8 * b)) & 0xffU);
    }
}

__device__ __forceinline__ std::uint32_t hfma2_bits(std::uint32_t a, std::uint32_t b, std::uint32_t c) {
    std::uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ std::uint32_t hmul2_bits(std::uint32_t a, std::uint32_t b) {
    std::uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

__device__ __forceinline__ float half2_sum(std::uint32_t bits) {
    const __half2 h = *reinterpret_cast<const __half2*>(&bits);
    const float2 f = __half22float2(h);
    return f.x + f.y;
}

// Dot product of 32 weight values (two scale blocks) with 32 activation values,
// both as f16x2 registers; returns the two exact block sums.
__device__ __forceinline__ void dot32(const std::uint32_t (&w)[16], const std::uint32_t (&x)[16], float* s0,
                                      float* s1) {
    std::uint32_t a0 = hmul2_bits(w[0], x[0]);
    std::uint32_t a1 = hmul2_bits(w[8], x[8]);
#pragma unroll
    for (int i = 1; i < 8; ++i) {
        a0 = hfma2_bits(w[i], x[i], a0);
        a1 = hfma2_bits(w[8 + i], x[8 + i], a1);
    }
    *s0 = half2_sum(a0);
    *s1 = half2_sum(a1);
}

__device__ __forceinline__ float e4m3_lo(std::uint32_t two) { return decode_e4m3(static_cast<std::uint8_t>(two & 0xffU)); }
__device__ __forceinline__ float e4m3_hi(std::uint32_t two) { return decode_e4m3(static_cast<std::uint8_t>((two >> 8) & 0xffU)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffU, v, offset);
    return v;
}

// Sums eight per-lane values over the warp with 9 shuffles instead of 40: three
// halving exchanges leave one value per lane, two butterflies finish it.  On
// return every lane holds the total of value index ((lane>>4)&1)*4 + ((lane>>3)&1)*2 + ((lane>>2)&1).
__device__ __forceinline__ float warp_sum8(float (&v)[8]) {
    const int lane = threadIdx.x & 31;
    {
        const bool upper = lane & 16;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float send = upper ? v[i] : v[i + 4];
            const float keep = upper ? v[i + 4] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffU, send, 16);
        }
    }
    {
        const bool upper = lane & 8;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float send = upper ? v[i] : v[i + 2];
            const float keep = upper ? v[i + 2] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffU, send, 8);
        }
    }
    {
        const bool upper = lane & 4;
        const float send = upper ? v[0] : v[1];
        const float keep = upper ? v[1] : v[0];
        v[0] = keep + __shfl_xor_sync(0xffffffffU, send, 4);
    }
    v[0] += __shfl_xor_sync(0xffffffffU, v[0], 2);
    v[0] += __shfl_xor_sync(0xffffffffU, v[0], 1);
    return v[0];
}

// Bank entry of a global expert id (256 = the shared expert); -1 if not held.
__device__ __forceinline__ int bank_entry(const BankView& bank, int expert) {
    if (expert == kExperts) return bank.local_experts;
    const int local = expert - bank.first_expert;
    return (local >= 0 && local < bank.local_experts) ? local : -1;
}

// ---------------------------------------------------------------------------
// gate/up + SwiGLU + re-quantise.  H = hidden size (K of the product).
// Item = (active expert, 16 consecutive intermediate rows).  Warp w owns rows
// 2w and 2w+1 of the tile for both matrices; the two rows are one contiguous
// 2*H/2-byte stream that the lanes cover in 16-byte chunks (c = lane + 32 j).
// ---------------------------------------------------------------------------
template <int H>
struct GateUpShared {
    static constexpr int kChunks = H / 32;                 // 16-byte chunks per row
    // activations of up to 4 rows, decoded to f16; piece p of chunk c at ((p*kChunks + c) * 16) bytes
    // so that lanes reading consecutive chunks touch consecutive 16-byte slots
    uint4 x[4][4 * kChunks];
    float xs[4][H / 16];
    float sums[2][4][kGateUpRows];                         // [gate|up][row of pass][tile row]
    float hval[4][kGateUpRows];
};

template <int H, int NT>
__device__ __forceinline__ void gate_up_pass(const uint4 (&wg)[(2 * (H / 32) + 31) / 32],
                                             const uint4 (&wu)[(2 * (H / 32) + 31) / 32],
                                             const std::uint32_t (&sg)[(2 * (H / 32) + 31) / 32],
                                             const std::uint32_t (&su)[(2 * (H / 32) + 31) / 32],
                                             GateUpShared<H>& sm, int warp, int lane) {
    constexpr int kChunks = H / 32;
    constexpr int NJ = (2 * kChunks + 31) / 32;
    float acc[2][NT][2];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < NT; ++n) acc[m][n][0] = acc[m][n][1] = 0.0F;

#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int c = j * 32 + lane;
        if (c < 2 * kChunks) {
            const bool second = c >= kChunks;
            const int kc = second ? c - kChunks : c;
            std::uint32_t wh[16];
            std::uint32_t uh[16];
            decode16(wg[j], wh);
            decode16(wu[j], uh);
            const float g0 = e4m3_lo(sg[j]), g1 = e4m3_hi(sg[j]);
            const float u0 = e4m3_lo(su[j]), u1 = e4m3_hi(su[j]);
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                std::uint32_t xh[16];
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    const uint4 v = sm.x[n][p * kChunks + kc];
                    xh[4 * p] = v.x;
                    xh[4 * p + 1] = v.y;
                    xh[4 * p + 2] = v.z;
                    xh[4 * p + 3] = v.w;
                }
                const float x0 = sm.xs[n][2 * kc];
                const float x1 = sm.xs[n][2 * kc + 1];
                float s0, s1;
                dot32(wh, xh, &s0, &s1);
                const float pg = fmaf(s0, g0 * x0, s1 * (g1 * x1));
                dot32(uh, xh, &s0, &s1);
                const float pu = fmaf(s0, u0 * x0, s1 * (u1 * x1));
                acc[0][n][0] += second ? 0.0F : pg;
                acc[0][n][1] += second ? pg : 0.0F;
                acc[1][n][0] += second ? 0.0F : pu;
                acc[1][n][1] += second ? pu : 0.0F;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const float total = warp_sum(acc[m][n][r]);
                if (lane == 0) sm.sums[m][n][2 * warp + r] = total;
            }
}

template <int H, bool FUSED>
__global__ void __launch_bounds__(kThreads, 2) gate_up_stream_kernel(
    BankView bank, RouteView route, const std::uint8_t* __restrict__ xq, const std::uint8_t* __restrict__ xs,
    std::uint8_t* __restrict__ hq, std::uint8_t* __restrict__ hs, std::uint16_t* __restrict__ gate_out,
    std::uint16_t* __restrict__ up_out, const std::int32_t* __restrict__ order, std::int32_t* status) {
    constexpr int kChunks = H / 32;
    constexpr int NJ = (2 * kChunks + 31) / 32;
    __shared__ GateUpShared<H> sm;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int inter = bank.intermediate;
    const int tiles = inter / kGateUpRows;
    const int active_count = *route.active_count;
    // unfused mode serves the routed experts only (the stage API of the reference has no shared expert)
    const int first_active = FUSED ? 0 : 1;
    const int items = (active_count - first_active) * tiles;

    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int a = first_active + item / tiles;
        const int tile = item - (item / tiles) * tiles;
        const int expert = route.active[a];
        const int entry = bank_entry(bank, expert);
        if (entry < 0) {
            if (threadIdx.x == 0) atomicCAS(status, kStatusOk, kStatusBadExpertId);
            continue;
        }
        const int count = route.counts[expert];
        const int first_pos = route.offsets[expert];
        const int r0 = tile * kGateUpRows;
        const std::size_t matrix_bytes = static_cast<std::size_t>(inter) * (H / 2);
        const std::size_t scale_bytes = static_cast<std::size_t>(inter) * (H / 16);
        const std::uint8_t* gate_w = bank.w13 + (static_cast<std::size_t>(entry) * 2) * matrix_bytes +
                                     static_cast<std::size_t>(r0 + 2 * warp) * (H / 2);
        const std::uint8_t* up_w = gate_w + matrix_bytes;
        const std::uint8_t* gate_s = bank.sf13 + (static_cast<std::size_t>(entry) * 2) * scale_bytes +
                                     static_cast<std::size_t>(r0 + 2 * warp) * (H / 16);
        const std::uint8_t* up_s = gate_s + scale_bytes;

        // every weight byte of the item goes in flight before anything is used
        uint4 wg[NJ], wu[NJ];
        std::uint32_t sg[NJ], su[NJ];
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int c = j * 32 + lane;
            if (c < 2 * kChunks) {
                wg[j] = ldg_stream(gate_w + static_cast<std::size_t>(c) * 16);
                wu[j] = ldg_stream(up_w + static_cast<std::size_t>(c) * 16);
                sg[j] = ldg_u16(gate_s + c * 2);
                su[j] = ldg_u16(up_s + c * 2);
            } else {
                wg[j] = wu[j] = make_uint4(0U, 0U, 0U, 0U);
                sg[j] = su[j] = 0U;
            }
        }
        const float alpha_g = bank.alpha[entry * 3 + 0];
        const float alpha_u = bank.alpha[entry * 3 + 1];

        for (int pass = 0; pass < count; pass += 4) {
            const int nt = min(4, count - pass);
            __syncthreads();   // previous pass / item has finished with shared memory
            // stage the activation rows of this pass: E2M1 -> f16, E4M3 -> f32
            for (int idx = threadIdx.x; idx < nt * (H / 8); idx += kThreads) {
                const int n = idx / (H / 8);
                const int word = idx - n * (H / 8);              // 4 bytes = 8 elements
                const int token = route.row_token[first_pos + pass + n];
                const std::uint32_t raw =
                    __ldg(reinterpret_cast<const std::uint32_t*>(xq + static_cast<std::size_t>(token) * (H / 2)) + word);
                uint4 v;
                v.x = e2m1x2_to_f16x2(raw & 0xffU);
                v.y = e2m1x2_to_f16x2((raw >> 8) & 0xffU);
                v.z = e2m1x2_to_f16x2((raw >> 16) & 0xffU);
                v.w = e2m1x2_to_f16x2(raw >> 24);
                const int chunk = word >> 2;
                const int piece = word & 3;
                sm.x[n][piece * kChunks + chunk] = v;
            }
            for (int idx = threadIdx.x; idx < nt * (H / 16); idx += kThreads) {
                const int n = idx / (H / 16);
                const int g = idx - n * (H / 16);
                const int token = route.row_token[first_pos + pass + n];
                sm.xs[n][g] = decode_e4m3(xs[static_cast<std::size_t>(token) * (H / 16) + g]);
            }
            __syncthreads();
            switch (nt) {
                case 1: gate_up_pass<H, 1>(wg, wu, sg, su, sm, warp, lane); break;
                case 2: gate_up_pass<H, 2>(wg, wu, sg, su, sm, warp, lane); break;
                case 3: gate_up_pass<H, 3>(wg, wu, sg, su, sm, warp, lane); break;
                default: gate_up_pass<H, 4>(wg, wu, sg, su, sm, warp, lane); break;
            }
            __syncthreads();
            // epilogue: alpha, BF16 rounding of gate and up, SwiGLU, BF16 rounding
            if (threadIdx.x < nt * kGateUpRows) {
                const int n = threadIdx.x / kGateUpRows;
                const int r = threadIdx.x - n * kGateUpRows;
                const std::uint16_t g_bits = float_to_bf16_bits(sm.sums[0][n][r] * alpha_g);
                const std::uint16_t u_bits = float_to_bf16_bits(sm.sums[1][n][r] * alpha_u);
                if constexpr (FUSED) {
                    const float g = bf16_bits_to_float(g_bits);
                    const float h = (g / (1.0F + expf(-g))) * bf16_bits_to_float(u_bits);
                    sm.hval[n][r] = bf16_bits_to_float(float_to_bf16_bits(h));
                } else {
                    const int flat = order[first_pos + pass + n];
                    gate_out[static_cast<std::size_t>(flat) * inter + r0 + r] = g_bits;
                    up_out[static_cast<std::size_t>(flat) * inter + r0 + r] = u_bits;
                }
            }
            if constexpr (FUSED) {
                __syncthreads();
                if (threadIdx.x < nt) {
                    const int n = threadIdx.x;
                    float v[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = sm.hval[n][i];
                    std::uint8_t scale_bits;
                    const uint2 packed = quantize_block16(v, 1.0F, &scale_bits);
                    const std::size_t pos = static_cast<std::size_t>(first_pos + pass + n);
                    *reinterpret_cast<uint2*>(hq + pos * (inter / 2) + r0 / 2) = packed;
                    hs[pos * (inter / 16) + r0 / 16] = scale_bits;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// down projection.  I = intermediate size (K of the product) = 32 chunks * 32:
// one 16-byte chunk per lane per weight row, so a warp reads a whole 512-byte
// row per request.  Item = (active expert, 64 output rows); warp w owns 8 rows.
// Activation chunks (one per lane per row of the pass) stay in registers.
// ---------------------------------------------------------------------------
template <int I, int NT>
__device__ __forceinline__ void down_pass(const uint4 (&wr)[kDownRowsPerWarp], const std::uint32_t (&sr)[kDownRowsPerWarp],
                                          const std::uint8_t* __restrict__ hq, const std::uint8_t* __restrict__ hs,
                                          const std::int32_t* __restrict__ in_rows, int first, float alpha,
                                          std::uint16_t* __restrict__ out, const std::int32_t* __restrict__ out_rows,
                                          int hidden, int row_base, int lane) {
    std::uint32_t xh[NT][16];
    float x0[NT], x1[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        const std::size_t src = in_rows != nullptr ? static_cast<std::size_t>(in_rows[first + n])
                                                   : static_cast<std::size_t>(first + n);
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(hq + src * (I / 2)) + lane);
        decode16(raw, xh[n]);
        const std::uint32_t two = ldg_u16(hs + src * (I / 16) + lane * 2);
        x0[n] = e4m3_lo(two);
        x1[n] = e4m3_hi(two);
    }
    float part[NT][kDownRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kDownRowsPerWarp; ++r) {
        std::uint32_t wh[16];
        decode16(wr[r], wh);
        const float w0 = e4m3_lo(sr[r]), w1 = e4m3_hi(sr[r]);
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            float s0, s1;
            dot32(wh, xh[n], &s0, &s1);
            part[n][r] = fmaf(s0, w0 * x0[n], s1 * (w1 * x1[n]));
        }
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        const float total = warp_sum8(part[n]);
        if ((lane & 3) == 0) {
            const int r = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
            const std::size_t dst = out_rows != nullptr ? static_cast<std::size_t>(out_rows[first + n])
                                                        : static_cast<std::size_t>(first + n);
            out[dst * hidden + row_base + r] = float_to_bf16_bits(total * alpha);
        }
    }
}

// in_rows / out_rows (nullable): position -> row of hq/hs and of `out`; identity when null.
template <int I>
__global__ void __launch_bounds__(kThreads, 2) down_stream_kernel(
    BankView bank, RouteView route, const std::uint8_t* __restrict__ hq, const std::uint8_t* __restrict__ hs,
    std::uint16_t* __restrict__ out, const std::int32_t* __restrict__ in_rows,
    const std::int32_t* __restrict__ out_rows, int first_active, std::int32_t* status) {
    static_assert(I == 1024, "one 16-byte chunk per lane per row");
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int hidden = bank.hidden;
    const int tiles = hidden / kDownRows;
    const int active_count = *route.active_count;
    const int items = (active_count - first_active) * tiles;

    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int a = first_active + item / tiles;
        const int tile = item - (item / tiles) * tiles;
        const int expert = route.active[a];
        const int entry = bank_entry(bank, expert);
        if (entry < 0) {
            if (threadIdx.x == 0) atomicCAS(status, kStatusOk, kStatusBadExpertId);
            continue;
        }
        const int count = route.counts[expert];
        const int first_pos = route.offsets[expert];
        const int row_base = tile * kDownRows + warp * kDownRowsPerWarp;
        const std::uint8_t* w = bank.w2 + (static_cast<std::size_t>(entry) * hidden + row_base) * (I / 2);
        const std::uint8_t* s = bank.sf2 + (static_cast<std::size_t>(entry) * hidden + row_base) * (I / 16);
        uint4 wr[kDownRowsPerWarp];
        std::uint32_t sr[kDownRowsPerWarp];
#pragma unroll
        for (int r = 0; r < kDownRowsPerWarp; ++r) {
            wr[r] = ldg_stream(w + static_cast<std::size_t>(r) * (I / 2) + lane * 16);
            sr[r] = ldg_u16(s + r * (I / 16) + lane * 2);
        }
        const float alpha = bank.alpha[entry * 3 + 2];
        for (int pass = 0; pass < count; pass += 2) {
            if (count - pass >= 2) {
                down_pass<I, 2>(wr, sr, hq, hs, in_rows, first_pos + pass, alpha, out, out_rows, hidden, row_base, lane);
            } else {
                down_pass<I, 1>(wr, sr, hq, hs, in_rows, first_pos + pass, alpha, out, out_rows, hidden, row_base, lane);
            }
        }
    }
}

int persistent_blocks(const p92b_plan* plan, int per_sm) { return plan->sm_count * per_sm; }

}  // namespace

cudaError_t launch_gate_up(const p92b_plan* plan, const BankView& bank, const RouteView& route,
                           const std::uint8_t* xq, const std::uint8_t* xs, std::uint8_t* hq,
                           std::uint8_t* hs, std::uint16_t* gate_out, std::uint16_t* up_out,
                           const std::int32_t* order, int rows, cudaStream_t stream) {
    (void)rows;
    if (bank.w13 == nullptr || bank.hidden != 2560 || bank.intermediate % kGateUpRows != 0) return cudaErrorNotSupported;
    const int blocks = persistent_blocks(plan, 2);
    if (gate_out == nullptr) {
        gate_up_stream_kernel<2560, true><<<blocks, kThreads, 0, stream>>>(bank, route, xq, xs, hq, hs, nullptr,
                                                                           nullptr, order, plan->status);
    } else {
        gate_up_stream_kernel<2560, false><<<blocks, kThreads, 0, stream>>>(bank, route, xq, xs, nullptr, nullptr,
                                                                            gate_out, up_out, order, plan->status);
    }
    return cudaGetLastError();
}

cudaError_t launch_down(const p92b_plan* plan, const BankView& bank, const RouteView& route,
                        const std::uint8_t* hq, const std::uint8_t* hs, std::uint16_t* mixed,
                        const std::int32_t* in_rows, const std::int32_t* out_rows, int first_active,
                        cudaStream_t stream) {
    if (bank.w2 == nullptr || bank.intermediate != 1024 || bank.hidden % kDownRows != 0) return cudaErrorNotSupported;
    const int blocks = persistent_blocks(plan, 2);
    down_stream_kernel<1024><<<blocks, kThreads, 0, stream>>>(bank, route, hq, hs, mixed, in_rows, out_rows,
                                                             first_active, plan->status);
    return cudaGetLastError();
}

}  // namespace p92b
