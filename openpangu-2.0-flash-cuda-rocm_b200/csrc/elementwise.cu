// Element-wise stages of the MoE block: NVFP4 quantisation (activations and the
// offline weight law), scale swizzle, SwiGLU, weighted combine, shared-expert add.
// Each kernel keeps the reference's rounding points; citations are on the kernels.
// All of these are HBM-bound byte work: 16-byte accesses, one pass.
#include "p92b_common.cuh"
#include "tc_ptx.cuh"

#include <algorithm>

namespace p92b {
namespace {

// BF16 -> NVFP4, one thread per 16-element block (two 16-byte loads, one 8-byte
// store).  Arithmetic of cuda/nvfp4_ops.cu:818-841 == cuda/nvfp4_pack.cu:151-176.
// global_scale comes either by value or from 1 / *weight_scale_2 (weights).
__global__ void __launch_bounds__(256) quantize_kernel(const std::uint16_t* __restrict__ input,
                                                       std::uint8_t* __restrict__ output,
                                                       std::uint8_t* __restrict__ scales, long groups,
                                                       float global_scale,
                                                       const float* __restrict__ weight_scale_2) {
    const long group = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (group >= groups) return;
    if (weight_scale_2 != nullptr) global_scale = __fdiv_rn(1.0F, *weight_scale_2);   // host IEEE division in the reference (cuda/nvfp4_pack.cu:256)
    const uint4* src = reinterpret_cast<const uint4*>(input + group * 16);
    const uint4 a = src[0];
    const uint4 b = src[1];
    const std::uint32_t words[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float v[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[2 * i] = __uint_as_float(words[i] << 16);
        v[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000U);
    }
    std::uint8_t scale_bits;
    const uint2 packed = quantize_block16(v, global_scale, &scale_bits);
    *reinterpret_cast<uint2*>(output + group * 8) = packed;
    scales[group] = scale_bits;
}

// cuda/nvfp4_pack.cu:141-149: |x| maximum of a BF16 tensor as float bits (atomicMax on
// the bit pattern is order preserving for non-negative floats).
__global__ void __launch_bounds__(256) amax_kernel(const std::uint16_t* __restrict__ input, std::size_t elements,
                                                   unsigned* maximum) {
    unsigned local = 0;
    const std::size_t vectors = elements / 8;
    const uint4* src = reinterpret_cast<const uint4*>(input);
    for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < vectors;
         i += static_cast<std::size_t>(gridDim.x) * blockDim.x) {
        const uint4 v = src[i];
        const std::uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            local = max(local, (words[k] << 16) & 0x7fffffffU);
            local = max(local, words[k] & 0x7fff0000U);
        }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) local = max(local, __shfl_xor_sync(0xffffffffU, local, offset));
    if ((threadIdx.x & 31) == 0 && local != 0) atomicMax(maximum, local);
}

// cuda/nvfp4_pack.cu:255: weight_scale_2 = amax / (6 * 448).
__global__ void weight_scale_kernel(const unsigned* maximum, float* weight_scale_2, int matrices) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m < matrices) weight_scale_2[m] = __fdiv_rn(__uint_as_float(maximum[m]), 6.0F * 448.0F);
}

// The two kernels above for a batch of equally sized matrices stored back to back: blockIdx.y = matrix.
__global__ void __launch_bounds__(256) amax_batch_kernel(const std::uint16_t* __restrict__ input, std::size_t elements,
                                                         unsigned* maximum) {
    unsigned local = 0;
    const std::size_t vectors = elements / 8;
    const uint4* src = reinterpret_cast<const uint4*>(input + static_cast<std::size_t>(blockIdx.y) * elements);
    for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < vectors;
         i += static_cast<std::size_t>(gridDim.x) * blockDim.x) {
        const uint4 v = src[i];
        const std::uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            local = max(local, (words[k] << 16) & 0x7fffffffU);
            local = max(local, words[k] & 0x7fff0000U);
        }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) local = max(local, __shfl_xor_sync(0xffffffffU, local, offset));
    if ((threadIdx.x & 31) == 0 && local != 0) atomicMax(maximum + blockIdx.y, local);
}

__global__ void __launch_bounds__(256) quantize_batch_kernel(const std::uint16_t* __restrict__ input,
                                                             std::uint8_t* __restrict__ output,
                                                             std::uint8_t* __restrict__ scales, long groups_per_matrix,
                                                             const float* __restrict__ weight_scale_2) {
    const long local_group = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (local_group >= groups_per_matrix) return;
    const long group = static_cast<long>(blockIdx.y) * groups_per_matrix + local_group;
    const float global_scale = __fdiv_rn(1.0F, weight_scale_2[blockIdx.y]);
    const uint4* src = reinterpret_cast<const uint4*>(input + group * 16);
    const uint4 a = src[0];
    const uint4 b = src[1];
    const std::uint32_t words[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float v[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[2 * i] = __uint_as_float(words[i] << 16);
        v[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000U);
    }
    std::uint8_t scale_bits;
    const uint2 packed = quantize_block16(v, global_scale, &scale_bits);
    *reinterpret_cast<uint2*>(output + group * 8) = packed;
    scales[group] = scale_bits;
}

// cuda/nvfp4_ops.cu:869-890: linear [row][K/16] -> 128-row x 4-column tiles.
__global__ void __launch_bounds__(256) swizzle_kernel(const std::uint8_t* __restrict__ linear,
                                                      std::uint8_t* __restrict__ swizzled, int rows,
                                                      int scale_columns, int column_blocks) {
    const long index = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= static_cast<long>(rows) * scale_columns) return;
    const int row = static_cast<int>(index / scale_columns);
    const int column = static_cast<int>(index - static_cast<long>(row) * scale_columns);
    const int row_block = row >> 7;
    const int row_in_block = row & 127;
    const std::size_t destination =
        (static_cast<std::size_t>(row_block) * column_blocks + (column >> 2)) * 512 + (row_in_block & 31) * 16 +
        (row_in_block >> 5) * 4 + (column & 3);
    swizzled[destination] = linear[index];
}

// The three element-wise operators of the block's stage interface.  Each thread takes eight BF16 values through one
// 16-byte load per operand and one 16-byte store; `vectors` is the number of such groups (0 when a pointer or a row
// pitch is not 16-byte aligned) and the threads after them take the remaining values one each.
struct Bf16x8 {
    float v[8];
    __device__ __forceinline__ explicit Bf16x8(const uint4 raw) {
        const std::uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000U);
        }
    }
};
__device__ __forceinline__ uint4 pack_bf16x8(const float (&v)[8]) {
    std::uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        w[i] = static_cast<std::uint32_t>(float_to_bf16_bits(v[2 * i])) |
               (static_cast<std::uint32_t>(float_to_bf16_bits(v[2 * i + 1])) << 16);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
__host__ inline bool aligned16(const void* a, const void* b = nullptr, const void* c = nullptr) {
    return ((reinterpret_cast<std::uintptr_t>(a) | reinterpret_cast<std::uintptr_t>(b) | reinterpret_cast<std::uintptr_t>(c)) & 15U) == 0U;
}

// SwiGLU, bf16( g / (1 + expf(-g)) * u ) with the fast-math expf and division of cuda/nvfp4_ops.cu:97-105.
__device__ __forceinline__ float silu_times(float g, float u) { return (g / (1.0F + expf(-g))) * u; }
__global__ void __launch_bounds__(256) swiglu_kernel(const std::uint16_t* __restrict__ gate,
                                                     const std::uint16_t* __restrict__ up,
                                                     std::uint16_t* __restrict__ output, long elements, long vectors) {
    const long t = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t < vectors) {
        const Bf16x8 g(__ldg(reinterpret_cast<const uint4*>(gate) + t));
        const Bf16x8 u(__ldg(reinterpret_cast<const uint4*>(up) + t));
        float r[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) r[i] = silu_times(g.v[i], u.v[i]);
        reinterpret_cast<uint4*>(output)[t] = pack_bf16x8(r);
        return;
    }
    const long i = vectors * 8 + (t - vectors);
    if (i < elements) output[i] = float_to_bf16_bits(silu_times(bf16_bits_to_float(gate[i]), bf16_bits_to_float(up[i])));
}

// Weighted sum of a token's expert rows: one FP32 fmaf chain per output value over the slots in slot order, one
// rounding at the end (cuda/nvfp4_ops.cu:124-142).  grid.y = batch row; `vectors` counts 8-value groups per row.
__global__ void __launch_bounds__(256) combine_rows_kernel(const std::uint16_t* __restrict__ expert_rows,
                                                           const float* __restrict__ route_weights,
                                                           std::uint16_t* __restrict__ output, int experts,
                                                           int elements, int vectors) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    const std::size_t route_base = static_cast<std::size_t>(blockIdx.y) * experts;
    std::uint16_t* out_row = output + static_cast<std::size_t>(blockIdx.y) * elements;
    if (t < vectors) {
        float acc[8] = {0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F};
        for (int slot = 0; slot < experts; ++slot) {
            const float w = __ldg(route_weights + route_base + slot);
            const Bf16x8 row(__ldg(reinterpret_cast<const uint4*>(expert_rows + (route_base + slot) * elements) + t));
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(row.v[i], w, acc[i]);
        }
        reinterpret_cast<uint4*>(out_row)[t] = pack_bf16x8(acc);
        return;
    }
    const int element = vectors * 8 + (t - vectors);
    if (element >= elements) return;
    float value = 0.0F;
    for (int slot = 0; slot < experts; ++slot) {
        value = fmaf(bf16_bits_to_float(expert_rows[(route_base + slot) * elements + element]),
                     __ldg(route_weights + route_base + slot), value);
    }
    out_row[element] = float_to_bf16_bits(value);
}

// destination = bf16(destination + source), the residual add of cuda/nvfp4_ops.cu:92-95.
__global__ void __launch_bounds__(256) add_kernel(std::uint16_t* __restrict__ destination,
                                                  const std::uint16_t* __restrict__ source, long elements, long vectors) {
    const long t = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t < vectors) {
        const Bf16x8 d(reinterpret_cast<const uint4*>(destination)[t]);
        const Bf16x8 s(__ldg(reinterpret_cast<const uint4*>(source) + t));
        float r[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) r[i] = d.v[i] + s.v[i];
        reinterpret_cast<uint4*>(destination)[t] = pack_bf16x8(r);
        return;
    }
    const long i = vectors * 8 + (t - vectors);
    if (i < elements) destination[i] = float_to_bf16_bits(bf16_bits_to_float(destination[i]) + bf16_bits_to_float(source[i]));
}

// RMSNorm of BF16 rows, bit-exact with the reference operator (cuda/nvfp4_ops.cu:67-90, called either side of
// the block, src/model.cpp:211-218,1210-1217): the sum of squares is the reference's 256 chains per row - chain t
// takes elements t, t+256, ... with fmaf - reduced by a shuffle-down tree per 32 chains and a second tree over the
// eight results (block_sum, :38-51); inverse = rsqrtf(sum / elements + eps) and out = bf16(x * inverse * w), all in
// a file compiled with --use_fast_math like the reference, with `elements` a run-time value as there.  The row is
// staged in shared memory with 16-byte loads; the chains then read it conflict-free.
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const std::uint16_t* __restrict__ input,
                                                           const std::uint16_t* __restrict__ weight,
                                                           std::uint16_t* __restrict__ output, int elements,
                                                           int input_stride, int output_stride, float epsilon) {
    extern __shared__ __align__(16) std::uint16_t norm_row[];
    __shared__ float warp_sums[8];
    __shared__ float inverse_shared;
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    const std::uint16_t* in = input + static_cast<std::size_t>(blockIdx.x) * input_stride;
    std::uint16_t* out = output + static_cast<std::size_t>(blockIdx.x) * output_stride;
    const bool vector_ok = (elements & 7) == 0 && (input_stride & 7) == 0 && (reinterpret_cast<std::uintptr_t>(input) & 15) == 0;
    if (vector_ok) {
        for (int i = threadIdx.x; i < elements / 8; i += 256) {
            reinterpret_cast<uint4*>(norm_row)[i] = __ldg(reinterpret_cast<const uint4*>(in) + i);
        }
    } else {
        for (int i = threadIdx.x; i < elements; i += 256) norm_row[i] = in[i];
    }
    __syncthreads();
    float square_sum = 0.0F;
    for (int i = threadIdx.x; i < elements; i += 256) {
        const float value = bf16_bits_to_float(norm_row[i]);
        square_sum = fmaf(value, value, square_sum);
    }
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) square_sum += __shfl_down_sync(0xffffffffU, square_sum, offset);
    if (lane == 0) warp_sums[warp] = square_sum;
    __syncthreads();
    if (warp == 0) {
        float total = lane < 8 ? warp_sums[lane] : 0.0F;
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) total += __shfl_down_sync(0xffffffffU, total, offset);
        if (lane == 0) inverse_shared = rsqrtf(total / static_cast<float>(elements) + epsilon);
    }
    __syncthreads();
    const float inverse = inverse_shared;
    for (int i = threadIdx.x; i < elements; i += 256) {
        out[i] = float_to_bf16_bits(bf16_bits_to_float(norm_row[i]) * inverse * bf16_bits_to_float(__ldg(weight + i)));
    }
}

// Fused tail of the block: the weighted combine above (gathering each slot's
// down row from position space), rounded to BF16 exactly where the reference
// stores `hidden_`, then the shared expert's BF16 down row added and rounded
// again (src/model.cpp:1505-1508 then :1571-1572).  Eight columns per thread.
__global__ void __launch_bounds__(256) combine_shared_kernel(const std::uint16_t* __restrict__ mixed,
                                                             const std::int32_t* __restrict__ mixed_index,
                                                             const float* __restrict__ route_weights,
                                                             std::uint16_t* __restrict__ output, int rows,
                                                             int hidden) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    const int row = blockIdx.y;
    const int c8 = blockIdx.x * blockDim.x + threadIdx.x;
    if (c8 * 8 >= hidden) return;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0F;
    uint4 slot_rows[kTop];
    float w[kTop];
#pragma unroll
    for (int slot = 0; slot < kTop; ++slot) {
        const int pos = mixed_index[row * kTop + slot];
        w[slot] = route_weights[row * kTop + slot];
        slot_rows[slot] = *reinterpret_cast<const uint4*>(mixed + static_cast<std::size_t>(pos) * hidden + c8 * 8);
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
    const uint4 sh = *reinterpret_cast<const uint4*>(
        mixed + static_cast<std::size_t>(mixed_index[rows * kTop + row]) * hidden + c8 * 8);
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

// Row-major packed weights + tiled scales of one matrix -> the chunk stream (see BankView).
// One thread per 16 bytes: first the weight pieces, then the scale bytes.
__device__ __forceinline__ void retile_piece(const std::uint8_t* __restrict__ weight,
                                             const std::uint8_t* __restrict__ scales,
                                             std::uint8_t* __restrict__ chunks, long index, int rows, int k_bytes,
                                             int blocks_per_chunk, int slot) {
    const int pieces_per_row = k_bytes / 16;
    const int k_blocks = k_bytes / 128;
    const int chunks_per_tile = k_blocks / blocks_per_chunk;
    const long weight_pieces = static_cast<long>(rows) * pieces_per_row;
    if (index < weight_pieces) {
        const int row = static_cast<int>(index / pieces_per_row);
        const int piece = static_cast<int>(index - static_cast<long>(row) * pieces_per_row);
        const int tile = row >> 7, r = row & 127;
        const int kb = piece >> 3, j = piece & 7;
        const int which = blocks_per_chunk == 1 ? slot : (kb & 1);
        const std::size_t chunk = static_cast<std::size_t>(tile) * chunks_per_tile + kb / blocks_per_chunk;
        const uint4 v = *reinterpret_cast<const uint4*>(weight + static_cast<std::size_t>(row) * k_bytes + piece * 16);
        *reinterpret_cast<uint4*>(chunks + chunk * kChunkBytes + which * kChunkBox + r * 128 + ((j ^ (r & 7)) * 16)) = v;
        return;
    }
    const long scale_piece = index - weight_pieces;                     // 16 scale bytes each
    const long scale_pieces = static_cast<long>(rows / 128) * k_blocks * (kChunkScaleBytes / 16);
    if (scale_piece >= scale_pieces) return;
    const int per_block = kChunkScaleBytes / 16;                        // 128 pieces per (tile, K block)
    const long block_index = scale_piece / per_block;                   // tile * k_blocks + kb
    const int within = static_cast<int>(scale_piece - block_index * per_block);
    const int tile = static_cast<int>(block_index / k_blocks);
    const int kb = static_cast<int>(block_index - static_cast<long>(tile) * k_blocks);
    const int which = blocks_per_chunk == 1 ? slot : (kb & 1);
    const std::size_t chunk = static_cast<std::size_t>(tile) * chunks_per_tile + kb / blocks_per_chunk;
    // source: tile row-block `tile`, scale column blocks 4*kb .. 4*kb+3, 512 bytes each, contiguous
    const uint4 v = *reinterpret_cast<const uint4*>(
        scales + (static_cast<std::size_t>(tile) * (k_blocks * 4) + kb * 4) * 512 + within * 16);
    *reinterpret_cast<uint4*>(chunks + chunk * kChunkBytes + kChunkScaleOffset + which * kChunkScaleBytes + within * 16) = v;
}

// All entries of one kind in one launch: blockIdx.y = entry, the matrix pointers come from the
// caller's table of reference-format projections (entry * 3 + kind), uploaded once.
__global__ void __launch_bounds__(256) retile_table_kernel(const p92b_expert_projection* __restrict__ table, int kind,
                                                           std::uint8_t* __restrict__ chunks, std::size_t entry_bytes,
                                                           int rows, int k_bytes, int blocks_per_chunk, int slot,
                                                           float* __restrict__ alpha) {
    const int entry = blockIdx.y;
    const p92b_expert_projection src = table[entry * 3 + kind];
    const long index = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index == 0) alpha[entry * 3 + kind] = *src.alpha;
    retile_piece(src.weight, src.scales_swizzled, chunks + static_cast<std::size_t>(entry) * entry_bytes, index, rows,
                 k_bytes, blocks_per_chunk, slot);
}

inline unsigned blocks_for(long n, int per_block) { return static_cast<unsigned>((n + per_block - 1) / per_block); }

}  // namespace

cudaError_t launch_quantize(const std::uint16_t* input, std::uint8_t* output, std::uint8_t* scales,
                            long groups, float global_scale, cudaStream_t stream) {
    if (input == nullptr || output == nullptr || scales == nullptr || groups <= 0) return cudaErrorInvalidValue;
    quantize_kernel<<<blocks_for(groups, 256), 256, 0, stream>>>(input, output, scales, groups, global_scale, nullptr);
    return cudaGetLastError();
}

cudaError_t launch_combine_shared(const std::uint16_t* mixed, const std::int32_t* mixed_index,
                                  const float* route_weights, std::uint16_t* output, int rows,
                                  int hidden, cudaStream_t stream, bool pdl) {
    dim3 grid(blocks_for(hidden / 8, 256), rows);
    return launch_kernel(combine_shared_kernel, grid, dim3(256), 0, stream, pdl, mixed, mixed_index, route_weights,
                         output, rows, hidden);
}

cudaError_t launch_rmsnorm(const std::uint16_t* input, const std::uint16_t* weight, std::uint16_t* output, int rows,
                           int elements, int input_stride, int output_stride, float epsilon, cudaStream_t stream, bool pdl) {
    if (input == nullptr || weight == nullptr || output == nullptr || rows <= 0 || elements <= 0 || elements > 24576 ||
        input_stride < elements || output_stride < elements || !(epsilon > 0.0F)) {
        return cudaErrorInvalidValue;
    }
    return launch_kernel(rmsnorm_rows_kernel, dim3(rows), dim3(256), static_cast<std::size_t>(elements) * 2, stream, pdl,
                         input, weight, output, elements, input_stride, output_stride, epsilon);
}

cudaError_t launch_retile_table(const p92b_expert_projection* device_table, int entries, int kind, std::uint8_t* chunks,
                                std::size_t entry_bytes, int rows, int k_bytes, int blocks_per_chunk, int slot,
                                float* alpha, cudaStream_t stream) {
    const long threads = static_cast<long>(rows) * (k_bytes / 16) +
                         static_cast<long>(rows / 128) * (k_bytes / 128) * (kChunkScaleBytes / 16);
    retile_table_kernel<<<dim3(blocks_for(threads, 256), entries), 256, 0, stream>>>(device_table, kind, chunks, entry_bytes,
                                                                                      rows, k_bytes, blocks_per_chunk, slot,
                                                                                      alpha);
    return cudaGetLastError();
}

}  // namespace p92b

using namespace p92b;

extern "C" {

int p92b_nvfp4_quantize(const uint16_t* input, uint8_t* output, uint8_t* scales, int elements,
                        float global_scale, void* stream) {
    if (elements <= 0 || elements % 16 != 0) return cudaErrorInvalidValue;
    return launch_quantize(input, output, scales, elements / 16, global_scale, static_cast<cudaStream_t>(stream));
}

size_t p92b_nvfp4_swizzled_scale_bytes(int rows, int scale_columns) {
    if (rows <= 0 || scale_columns <= 0) return 0;
    const size_t padded_rows = (static_cast<size_t>(rows) + 127) / 128 * 128;
    const size_t padded_columns = (static_cast<size_t>(scale_columns) + 3) / 4 * 4;
    return padded_rows * padded_columns;
}

int p92b_nvfp4_swizzle_scales(const uint8_t* linear, uint8_t* swizzled, int rows, int scale_columns,
                              void* stream) {
    if (linear == nullptr || swizzled == nullptr || rows <= 0 || scale_columns <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t st = cudaMemsetAsync(swizzled, 0, p92b_nvfp4_swizzled_scale_bytes(rows, scale_columns), s);
    if (st != cudaSuccess) return st;
    const long n = static_cast<long>(rows) * scale_columns;
    swizzle_kernel<<<blocks_for(n, 256), 256, 0, s>>>(linear, swizzled, rows, scale_columns, (scale_columns + 3) / 4);
    return cudaGetLastError();
}

int p92b_nvfp4_pack_weight(const uint16_t* input, uint8_t* packed, uint8_t* scales, size_t elements,
                           float* weight_scale_2, void* stream) {
    if (input == nullptr || packed == nullptr || scales == nullptr || weight_scale_2 == nullptr ||
        elements == 0 || elements % 16 != 0) {
        return cudaErrorInvalidValue;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the float slot doubles as the atomicMax cell (bit pattern of a non-negative float)
    cudaError_t st = cudaMemsetAsync(weight_scale_2, 0, sizeof(float), s);
    if (st != cudaSuccess) return st;
    const unsigned blocks = static_cast<unsigned>(std::min<size_t>((elements / 8 + 255) / 256, 148 * 16));
    amax_kernel<<<blocks, 256, 0, s>>>(input, elements, reinterpret_cast<unsigned*>(weight_scale_2));
    weight_scale_kernel<<<1, 32, 0, s>>>(reinterpret_cast<const unsigned*>(weight_scale_2), weight_scale_2, 1);
    const long groups = static_cast<long>(elements / 16);
    quantize_kernel<<<blocks_for(groups, 256), 256, 0, s>>>(input, packed, scales, groups, 0.0F, weight_scale_2);
    return cudaGetLastError();
}

int p92b_nvfp4_pack_weight_batch(const uint16_t* input, uint8_t* packed, uint8_t* scales, size_t elements_per_matrix,
                                 int matrices, float* weight_scale_2, void* stream) {
    if (input == nullptr || packed == nullptr || scales == nullptr || weight_scale_2 == nullptr || matrices <= 0 ||
        matrices > 65535 || elements_per_matrix == 0 || elements_per_matrix % 16 != 0) {
        return cudaErrorInvalidValue;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t st = cudaMemsetAsync(weight_scale_2, 0, sizeof(float) * matrices, s);
    if (st != cudaSuccess) return st;
    const unsigned blocks = static_cast<unsigned>(std::min<size_t>((elements_per_matrix / 8 + 255) / 256, 64));
    amax_batch_kernel<<<dim3(blocks, matrices), 256, 0, s>>>(input, elements_per_matrix,
                                                              reinterpret_cast<unsigned*>(weight_scale_2));
    weight_scale_kernel<<<(matrices + 255) / 256, 256, 0, s>>>(reinterpret_cast<const unsigned*>(weight_scale_2),
                                                                weight_scale_2, matrices);
    const long groups = static_cast<long>(elements_per_matrix / 16);
    quantize_batch_kernel<<<dim3(blocks_for(groups, 256), matrices), 256, 0, s>>>(input, packed, scales, groups,
                                                                                   weight_scale_2);
    return cudaGetLastError();
}

int p92b_swiglu(const uint16_t* gate, const uint16_t* up, uint16_t* output, int elements, void* stream) {
    if (gate == nullptr || up == nullptr || output == nullptr || elements <= 0) return cudaErrorInvalidValue;
    const long vectors = aligned16(gate, up, output) ? elements / 8 : 0;
    swiglu_kernel<<<blocks_for(vectors + (elements - vectors * 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        gate, up, output, elements, vectors);
    return cudaGetLastError();
}

int p92b_expert_combine_rows(const uint16_t* expert_rows, const float* route_weights, uint16_t* output,
                             int batch_rows, int experts, int elements, void* stream) {
    if (expert_rows == nullptr || route_weights == nullptr || output == nullptr || batch_rows <= 0 ||
        experts <= 0 || elements <= 0) {
        return cudaErrorInvalidValue;
    }
    const int vectors = aligned16(expert_rows, output) && elements % 8 == 0 ? elements / 8 : 0;
    dim3 grid(blocks_for(vectors + (elements - vectors * 8), 256), batch_rows);
    combine_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(expert_rows, route_weights, output,
                                                                            experts, elements, vectors);
    return cudaGetLastError();
}

int p92b_expert_combine(const uint16_t* expert_rows, const float* route_weights, uint16_t* output,
                        int experts, int elements, void* stream) {
    return p92b_expert_combine_rows(expert_rows, route_weights, output, 1, experts, elements, stream);
}

int p92b_rmsnorm(const uint16_t* input, const uint16_t* weight, uint16_t* output, int rows, int elements, float epsilon,
                 void* stream) {
    return launch_rmsnorm(input, weight, output, rows, elements, elements, elements, epsilon,
                          static_cast<cudaStream_t>(stream), false);
}

int p92b_rmsnorm_strided(const uint16_t* input, int input_stride, const uint16_t* weight, uint16_t* output,
                         int output_stride, int rows, int elements, float epsilon, void* stream) {
    return launch_rmsnorm(input, weight, output, rows, elements, input_stride, output_stride, epsilon,
                          static_cast<cudaStream_t>(stream), false);
}

int p92b_add_inplace(uint16_t* destination, const uint16_t* source, int elements, void* stream) {
    if (destination == nullptr || source == nullptr || elements <= 0) return cudaErrorInvalidValue;
    const long vectors = aligned16(destination, source) ? elements / 8 : 0;
    add_kernel<<<blocks_for(vectors + (elements - vectors * 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        destination, source, elements, vectors);
    return cudaGetLastError();
}

}  // extern "C"
