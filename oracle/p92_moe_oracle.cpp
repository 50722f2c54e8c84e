// CPU oracle for the openPangu-2.0-Flash MoE block.
//
// TEST INFRASTRUCTURE ONLY.  This file is a CPU restatement of the reference's
// arithmetic for the MoE path; it is the checker for the CUDA library and the
// timed CPU baseline.  Nothing in the shipped library links, loads or calls it.
//
// Every function names the reference source it follows (paths are relative to
// the reference project).  Summation orders, rounding points and tie rules are
// reproduced literally so that results which are pure comparison / integer work
// (expert ids, permutation, NVFP4 bytes) are bit-identical, and floating-point
// results are identical wherever the reference uses IEEE operations.  The one
// known difference: the reference's CUDA build uses --use_fast_math
// (CMakeLists.txt:98), so its expf and divisions are hardware approximations;
// here they are libm / IEEE.  Callers compare ids on margin-filtered tokens and
// use the GPU-compiled reference (oracle/_ref) for bit-exact id parity.
//
// Parity pin: E2M1/E4M3 conversions are pinned exhaustively against the CUDA
// toolkit's cuda_fp4.h / cuda_fp8.h host conversions (oracle/pin_cvt.cpp); the
// router tie rule, E2M1 table and UE4M3 decode are pinned against the known
// answers in the reference's own tests (tests/test_oracle_pins.py).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#if defined(_OPENMP)
#include <omp.h>
#endif

namespace {

inline float bf16_to_float(std::uint16_t bits) {
    std::uint32_t u = static_cast<std::uint32_t>(bits) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

// __float2bfloat16_rn: round to nearest even, NaN -> 0x7fff.
inline std::uint16_t float_to_bf16(float value) {
    std::uint32_t u;
    std::memcpy(&u, &value, 4);
    if ((u & 0x7fffffffU) > 0x7f800000U) return 0x7fffU;
    const std::uint32_t rounding = 0x7fffU + ((u >> 16) & 1U);
    return static_cast<std::uint16_t>((u + rounding) >> 16);
}

// E2M1 magnitudes (amd-gfx906/prefill/tests/p92_pf_moe_test.hip:15-20).
const float kE2m1[8] = {0.0F, 0.5F, 1.0F, 1.5F, 2.0F, 3.0F, 4.0F, 6.0F};

inline float decode_fp4(std::uint8_t nibble) {
    const float v = kE2m1[nibble & 7U];
    return (nibble & 8U) ? -v : v;
}

// E4M3 (sign, 4-bit exponent bias 7, 3-bit mantissa; 0x7f/0xff = NaN).
// Unsigned part follows amd-gfx906/prefill/tests/p92_pf_moe_test.hip:21-28.
inline float decode_e4m3(std::uint8_t bits) {
    const std::uint32_t e = (bits >> 3) & 15U;
    const std::uint32_t m = bits & 7U;
    float v;
    if (e == 0) {
        v = static_cast<float>(m) * 0.001953125F;
    } else if (e == 15 && m == 7) {
        v = NAN;
    } else {
        const std::uint32_t u = ((e + 120U) << 23) | (m << 20);
        std::memcpy(&v, &u, 4);
    }
    return (bits & 0x80U) ? -v : v;
}

// float -> E4M3, round-to-nearest-even, saturate-to-finite: what
// __nv_fp8_e4m3(float) does (cuda/nvfp4_ops.cu:828, cuda/nvfp4_pack.cu:162).
inline std::uint8_t encode_e4m3(float value) {
    std::uint32_t u;
    std::memcpy(&u, &value, 4);
    const std::uint8_t sign = static_cast<std::uint8_t>((u >> 24) & 0x80U);
    const float a = std::fabs(value);
    if (std::isnan(value)) return static_cast<std::uint8_t>(sign | 0x7fU);
    if (a >= 448.0F) return static_cast<std::uint8_t>(sign | 0x7eU);
    int exponent;
    (void)std::frexp(a, &exponent);              // a = f * 2^exponent, f in [0.5,1)
    int e = exponent - 1;                        // floor(log2 a)
    if (e < -6) e = -6;                          // subnormal range shares 2^-9 quantum
    const float quantum = std::ldexp(1.0F, e - 3);
    float q = std::nearbyint(a / quantum) * quantum;   // exact: power-of-two scaling
    if (q > 448.0F) q = 448.0F;
    if (q == 0.0F) return sign;
    (void)std::frexp(q, &exponent);
    e = exponent - 1;
    std::uint32_t field_e;
    std::uint32_t field_m;
    if (e < -6) {
        field_e = 0;
        field_m = static_cast<std::uint32_t>(q * 512.0F);
    } else {
        field_e = static_cast<std::uint32_t>(e + 7);
        field_m = static_cast<std::uint32_t>((q / std::ldexp(1.0F, e) - 1.0F) * 8.0F);
    }
    return static_cast<std::uint8_t>(sign | (field_e << 3) | field_m);
}

// float -> E2M1, round-to-nearest-even, saturate-to-finite: one half of
// __nv_fp4x2_e2m1(float2) (cuda/nvfp4_ops.cu:836-839).
inline std::uint8_t encode_e2m1(float value) {
    std::uint32_t u;
    std::memcpy(&u, &value, 4);
    const std::uint8_t sign = static_cast<std::uint8_t>((u >> 28) & 8U);
    float a = std::fabs(value);
    if (std::isnan(value)) return static_cast<std::uint8_t>(sign | 7U);
    if (a > 6.0F) a = 6.0F;
    const float quantum = a < 2.0F ? 0.5F : (a < 4.0F ? 1.0F : 2.0F);
    const float q = std::nearbyint(a / quantum) * quantum;
    std::uint8_t code = 0;
    for (std::uint8_t i = 0; i < 8; ++i) {
        if (kE2m1[i] == q) code = i;
    }
    return static_cast<std::uint8_t>(sign | code);
}

// cuda/nvfp4_ops.cu:38-51 block_sum for a 256-thread block: warp shuffle-down
// tree (offsets 16..1), then a second tree over the 8 warp sums held in lanes
// 0..7 of warp 0 (lanes 8..31 contribute 0).
inline float warp_tree(const float* lanes32) {
    float v[32];
    for (int i = 0; i < 32; ++i) v[i] = lanes32[i];
    for (int offset = 16; offset > 0; offset >>= 1) {
        for (int lane = 0; lane < offset; ++lane) v[lane] = v[lane] + v[lane + offset];
    }
    return v[0];
}

inline float block_sum_256(const float* threads256) {
    float lanes[32];
    for (int i = 0; i < 32; ++i) lanes[i] = 0.0F;
    for (int warp = 0; warp < 8; ++warp) lanes[warp] = warp_tree(threads256 + warp * 32);
    return warp_tree(lanes);
}

}  // namespace

extern "C" {

int orc_threads() {
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void orc_set_threads(int n) {
#if defined(_OPENMP)
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

void orc_float_to_bf16(const float* in, std::uint16_t* out, long n) {
    for (long i = 0; i < n; ++i) out[i] = float_to_bf16(in[i]);
}

void orc_bf16_to_float(const std::uint16_t* in, float* out, long n) {
    for (long i = 0; i < n; ++i) out[i] = bf16_to_float(in[i]);
}

std::uint8_t orc_encode_e4m3(float v) { return encode_e4m3(v); }
std::uint8_t orc_encode_e2m1(float v) { return encode_e2m1(v); }
float orc_decode_e4m3(std::uint8_t b) { return decode_e4m3(b); }
float orc_decode_e2m1(std::uint8_t b) { return decode_fp4(b); }

void orc_encode_e4m3_array(const float* in, std::uint8_t* out, long n) {
    for (long i = 0; i < n; ++i) out[i] = encode_e4m3(in[i]);
}

void orc_encode_e2m1_array(const float* in, std::uint8_t* out, long n) {
    for (long i = 0; i < n; ++i) out[i] = encode_e2m1(in[i]);
}

// Router logits.  batch_rows == 1 follows bf16_gemv_f32_kernel
// (cuda/nvfp4_ops.cu:161-176: thread t sums columns t, t+256, ... with fmaf,
// then block_sum); batch_rows > 1 follows bf16_gemm_kernel<true>
// (cuda/nvfp4_ops.cu:178-207: lane l sums columns l, l+32, ..., then the
// shuffle-down tree).  The caller picks by row count exactly as
// src/model.cpp:1488 / :1679 do.  gemv_order != 0 forces the T=1 order.
void orc_router_logits(const std::uint16_t* x, const std::uint16_t* w, float* out,
                       int batch_rows, int rows, int columns, int gemv_order) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int t = 0; t < batch_rows; ++t) {
        for (int r = 0; r < rows; ++r) {
            const std::uint16_t* xi = x + static_cast<std::size_t>(t) * columns;
            const std::uint16_t* wi = w + static_cast<std::size_t>(r) * columns;
            if (gemv_order) {
                float partial[256];
                for (int th = 0; th < 256; ++th) {
                    float v = 0.0F;
                    for (int c = th; c < columns; c += 256) {
                        v = std::fmaf(bf16_to_float(xi[c]), bf16_to_float(wi[c]), v);
                    }
                    partial[th] = v;
                }
                out[static_cast<std::size_t>(t) * rows + r] = block_sum_256(partial);
            } else {
                float partial[32];
                for (int lane = 0; lane < 32; ++lane) {
                    float v = 0.0F;
                    for (int c = lane; c < columns; c += 32) {
                        v = std::fmaf(bf16_to_float(xi[c]), bf16_to_float(wi[c]), v);
                    }
                    partial[lane] = v;
                }
                out[static_cast<std::size_t>(t) * rows + r] = warp_tree(partial);
            }
        }
    }
}

// cuda/nvfp4_ops.cu:357-433 router_top8_kernel: sigmoid, + correction bias,
// eight rounds of arg-max over the corrected score with ties to the lower id,
// weights = uncorrected sigmoid of the winners, renormalised to routed_scale
// with the total taken in slot order.  `margin` (optional) receives, per row,
// the smallest gap between consecutive ranks 1..9 of the corrected scores, so
// callers can tell which rows a 1-ulp sigmoid difference could reorder.
void orc_router_top8(const float* logits, const float* bias, std::int32_t* ids,
                     float* weights, float* margin, int rows, int experts,
                     float routed_scale) {
#pragma omp parallel for schedule(static)
    for (int row = 0; row < rows; ++row) {
        std::vector<float> raw(experts), corrected(experts);
        std::vector<char> used(experts, 0);
        const float* lg = logits + static_cast<std::size_t>(row) * experts;
        for (int e = 0; e < experts; ++e) {
            raw[e] = 1.0F / (1.0F + std::exp(-lg[e]));
            corrected[e] = raw[e] + bias[e];
        }
        float chosen[9];
        for (int slot = 0; slot < 9; ++slot) {
            int best = -1;
            for (int e = 0; e < experts; ++e) {
                if (used[e]) continue;
                if (best < 0 || corrected[e] > corrected[best]) best = e;   // ties keep lower id
            }
            chosen[slot] = best >= 0 ? corrected[best] : -INFINITY;
            if (slot < 8) {
                used[best] = 1;
                ids[static_cast<std::size_t>(row) * 8 + slot] = best;
                weights[static_cast<std::size_t>(row) * 8 + slot] = raw[best];
            }
        }
        float total = 0.0F;
        for (int slot = 0; slot < 8; ++slot) total += weights[static_cast<std::size_t>(row) * 8 + slot];
        const float multiplier = routed_scale / total;
        for (int slot = 0; slot < 8; ++slot) weights[static_cast<std::size_t>(row) * 8 + slot] *= multiplier;
        if (margin != nullptr) {
            float m = INFINITY;
            for (int slot = 0; slot < 8; ++slot) m = std::min(m, chosen[slot] - chosen[slot + 1]);
            margin[row] = m;
        }
    }
}

// The permutation into expert-contiguous order.  Position of assignment
// (t, k) = #{ids < id} + #{same id, flat index t*8+k smaller}: the ranking loop
// of prepare_grouped_pointers_kernel (cuda/nvfp4_grouped.cu:117-132, per
// projection kind) and the row-major / slot-minor host scan in
// src/model.cpp:1528-1540.  order[pos] = flat index; position[flat] = pos;
// counts[e] rows per expert; offsets[e] exclusive prefix (experts+1 entries).
void orc_permute(const std::int32_t* ids, int assignments, int experts,
                 std::int32_t* order, std::int32_t* position, std::int32_t* counts,
                 std::int32_t* offsets) {
    for (int e = 0; e < experts; ++e) counts[e] = 0;
    for (int i = 0; i < assignments; ++i) counts[ids[i]] += 1;
    offsets[0] = 0;
    for (int e = 0; e < experts; ++e) offsets[e + 1] = offsets[e] + counts[e];
    std::vector<std::int32_t> cursor(offsets, offsets + experts);
    for (int i = 0; i < assignments; ++i) {
        const int pos = cursor[ids[i]]++;
        order[pos] = i;
        if (position != nullptr) position[i] = pos;
    }
}

// The literal O(n^2) ranking of cuda/nvfp4_grouped.cu:117-132 for one
// projection kind; only used to pin orc_permute on small inputs.
void orc_permute_ranking(const std::int32_t* ids, int assignments, std::int32_t* position) {
    for (int g = 0; g < assignments; ++g) {
        int ordered = 0;
        for (int other = 0; other < assignments; ++other) {
            ordered += ids[other] < ids[g] || (ids[other] == ids[g] && other < g);
        }
        position[g] = ordered;
    }
}

// BF16 -> NVFP4 per 16-element block (cuda/nvfp4_ops.cu:818-841 `quantize`,
// identical arithmetic to cuda/nvfp4_pack.cu:151-176 `pack_weight`).
// Activations use global_scale = 1 (src/executor.cpp:54-55,89-91); weights use
// global_scale = 1 / weight_scale_2.
void orc_nvfp4_quantize(const std::uint16_t* input, std::uint8_t* packed,
                        std::uint8_t* scales, long groups, float global_scale) {
#pragma omp parallel for schedule(static)
    for (long g = 0; g < groups; ++g) {
        const std::uint16_t* block = input + g * 16;
        float maximum = 0.0F;
        for (int i = 0; i < 16; ++i) maximum = std::fmax(maximum, std::fabs(bf16_to_float(block[i])));
        const std::uint8_t scale = encode_e4m3(maximum * (global_scale / 6.0F));
        scales[g] = scale;
        const float decoded = decode_e4m3(scale);
        const float multiplier = decoded == 0.0F ? 0.0F : global_scale / decoded;
        for (int i = 0; i < 8; ++i) {
            const std::uint8_t lo = encode_e2m1(bf16_to_float(block[2 * i]) * multiplier);
            const std::uint8_t hi = encode_e2m1(bf16_to_float(block[2 * i + 1]) * multiplier);
            packed[g * 8 + i] = static_cast<std::uint8_t>(lo | (hi << 4));
        }
    }
}

// cuda/nvfp4_pack.cu:141-149,255-256: per-tensor amax, weight_scale_2 =
// amax / (6 * 448), then pack_weight with global_scale = 1 / weight_scale_2.
float orc_nvfp4_pack_weight(const std::uint16_t* input, std::uint8_t* packed,
                            std::uint8_t* scales, long elements) {
    float amax = 0.0F;
    for (long i = 0; i < elements; ++i) amax = std::fmax(amax, std::fabs(bf16_to_float(input[i])));
    const float weight_scale_2 = amax / (6.0F * 448.0F);
    const float global_scale = 1.0F / weight_scale_2;
    orc_nvfp4_quantize(input, packed, scales, elements / 16, global_scale);
    return weight_scale_2;
}

// cuda/nvfp4_ops.cu:1332-1353 size rule and :869-890 `swizzle`: linear
// [row][K/16] scales into 128-row x 4-column tiles, zero padded.
long orc_swizzled_scale_bytes(int rows, int scale_columns) {
    const long padded_rows = (static_cast<long>(rows) + 127) / 128 * 128;
    const long padded_columns = (static_cast<long>(scale_columns) + 3) / 4 * 4;
    return padded_rows * padded_columns;
}

void orc_swizzle_scales(const std::uint8_t* linear, std::uint8_t* swizzled, int rows,
                        int scale_columns) {
    const long bytes = orc_swizzled_scale_bytes(rows, scale_columns);
    std::memset(swizzled, 0, static_cast<std::size_t>(bytes));
    const int column_blocks = (scale_columns + 3) / 4;
    for (int row = 0; row < rows; ++row) {
        for (int column = 0; column < scale_columns; ++column) {
            const int row_block = row / 128;
            const int row_in_block = row % 128;
            const int row_quarter = row_in_block / 32;
            const int row_in_quarter = row_in_block % 32;
            const long destination =
                (static_cast<long>(row_block) * column_blocks + column / 4) * 512 +
                row_in_quarter * 16 + row_quarter * 4 + column % 4;
            swizzled[destination] = linear[static_cast<long>(row) * scale_columns + column];
        }
    }
}

// cuda/nvfp4_ops.cu:843-867 `gemv` (the reference's software NVFP4 product and
// its own parity yardstick, cuda/nvfp4_projection_test.cu:222-225): thread t of
// 256 walks elements t, t+256, ...; each term is
// fmaf(fp4(x)*e4m3(sx), fp4(w)*e4m3(sw), sum); block_sum; bf16(sum * alpha).
// Linear (un-swizzled) scales.  batch_rows inputs share the weight.
void orc_nvfp4_gemv(const std::uint8_t* input, const std::uint8_t* weight,
                    const std::uint8_t* input_scales, const std::uint8_t* weight_scales,
                    std::uint16_t* output, int batch_rows, int rows, int columns, float alpha) {
    const int groups = columns / 16;
    std::vector<float> wdec(static_cast<std::size_t>(rows) * columns);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const std::uint8_t* rw = weight + static_cast<std::size_t>(r) * (columns / 2);
        const std::uint8_t* rs = weight_scales + static_cast<std::size_t>(r) * groups;
        float* dst = wdec.data() + static_cast<std::size_t>(r) * columns;
        for (int c = 0; c < columns; ++c) {
            const int shift = (c & 1) * 4;
            dst[c] = decode_fp4(static_cast<std::uint8_t>(rw[c / 2] >> shift)) * decode_e4m3(rs[c / 16]);
        }
    }
    for (int b = 0; b < batch_rows; ++b) {
        std::vector<float> xdec(columns);
        const std::uint8_t* xi = input + static_cast<std::size_t>(b) * (columns / 2);
        const std::uint8_t* xs = input_scales + static_cast<std::size_t>(b) * groups;
        for (int c = 0; c < columns; ++c) {
            const int shift = (c & 1) * 4;
            xdec[c] = decode_fp4(static_cast<std::uint8_t>(xi[c / 2] >> shift)) * decode_e4m3(xs[c / 16]);
        }
#pragma omp parallel for schedule(static)
        for (int r = 0; r < rows; ++r) {
            const float* wr = wdec.data() + static_cast<std::size_t>(r) * columns;
            float partial[256];
            for (int th = 0; th < 256; ++th) {
                float sum = 0.0F;
                for (int c = th; c < columns; c += 256) sum = std::fmaf(xdec[c], wr[c], sum);
                partial[th] = sum;
            }
            output[static_cast<std::size_t>(b) * rows + r] = float_to_bf16(block_sum_256(partial) * alpha);
        }
    }
}

// cuda/nvfp4_ops.cu:97-105 swiglu_kernel (IEEE expf / division here).
void orc_swiglu(const std::uint16_t* gate, const std::uint16_t* up, std::uint16_t* out, long n) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; ++i) {
        const float value = bf16_to_float(gate[i]);
        out[i] = float_to_bf16((value / (1.0F + std::exp(-value))) * bf16_to_float(up[i]));
    }
}

// cuda/nvfp4_ops.cu:124-142 expert_combine_rows_kernel: FP32 fmaf over the
// eight slots in rank order, one BF16 rounding ("device law").
void orc_expert_combine_rows(const std::uint16_t* expert_rows, const float* route_weights,
                             std::uint16_t* output, int batch_rows, int experts, int elements) {
#pragma omp parallel for schedule(static)
    for (int row = 0; row < batch_rows; ++row) {
        for (int el = 0; el < elements; ++el) {
            float value = 0.0F;
            for (int slot = 0; slot < experts; ++slot) {
                const std::size_t base = static_cast<std::size_t>(row) * experts + slot;
                value = std::fmaf(bf16_to_float(expert_rows[base * elements + el]), route_weights[base], value);
            }
            output[static_cast<std::size_t>(row) * elements + el] = float_to_bf16(value);
        }
    }
}

// cuda/nvfp4_ops.cu:616-632 scatter_add_scaled_rows_kernel: BF16
// read-modify-write per selected row ("host law" step for one expert).
void orc_scatter_add_scaled_rows(std::uint16_t* destination, const std::uint16_t* source,
                                 const std::int32_t* row_indices, const float* scales,
                                 int selected_rows, int elements) {
    for (int s = 0; s < selected_rows; ++s) {
        std::uint16_t* dst = destination + static_cast<std::size_t>(row_indices[s]) * elements;
        for (int el = 0; el < elements; ++el) {
            dst[el] = float_to_bf16(bf16_to_float(dst[el]) +
                                    bf16_to_float(source[static_cast<std::size_t>(s) * elements + el]) * scales[s]);
        }
    }
}

// cuda/nvfp4_ops.cu:67-90 rmsnorm_kernel with 256 threads (:14, :907-918): thread t sums the squares of elements
// t, t+256, ... with fmaf; block_sum (:38-51) is a shuffle-down tree over each 32 threads, then the same tree over
// the eight warp results (lanes 8..31 contribute zeros); inverse = rsqrtf(sum / elements + epsilon); out =
// bf16(x * inverse * w).  The CUDA build's rsqrtf and fast-math division are hardware approximations, so this
// restatement (1 / sqrtf, IEEE division) agrees with the kernel to a BF16 last place, not bit for bit.
void orc_rmsnorm(const std::uint16_t* input, const std::uint16_t* weight, std::uint16_t* output, int rows, int elements,
                 float epsilon) {
    for (int row = 0; row < rows; ++row) {
        const std::uint16_t* in = input + static_cast<std::size_t>(row) * elements;
        float chain[256];
        for (int t = 0; t < 256; ++t) {
            float s = 0.0F;
            for (int i = t; i < elements; i += 256) {
                const float v = bf16_to_float(in[i]);
                s = std::fmaf(v, v, s);
            }
            chain[t] = s;
        }
        float warp_sum[32] = {};
        for (int w = 0; w < 8; ++w) {
            float lane[32];
            for (int l = 0; l < 32; ++l) lane[l] = chain[w * 32 + l];
            for (int offset = 16; offset > 0; offset >>= 1) {
                for (int l = 0; l < 32; ++l) lane[l] = lane[l] + (l + offset < 32 ? lane[l + offset] : lane[l]);
            }
            warp_sum[w] = lane[0];
        }
        for (int offset = 16; offset > 0; offset >>= 1) {
            for (int l = 0; l < 32; ++l) warp_sum[l] = warp_sum[l] + (l + offset < 32 ? warp_sum[l + offset] : warp_sum[l]);
        }
        const float inverse = 1.0F / std::sqrt(warp_sum[0] / static_cast<float>(elements) + epsilon);
        for (int i = 0; i < elements; ++i) {
            output[static_cast<std::size_t>(row) * elements + i] =
                float_to_bf16(bf16_to_float(in[i]) * inverse * bf16_to_float(weight[i]));
        }
    }
}

// cuda/nvfp4_ops.cu:92-95 add_kernel.
void orc_add_inplace(std::uint16_t* destination, const std::uint16_t* source, long n) {
    for (long i = 0; i < n; ++i) {
        destination[i] = float_to_bf16(bf16_to_float(destination[i]) + bf16_to_float(source[i]));
    }
}

// One NVFP4 projection the way ProjectionExecutor::project_rows does it
// (src/executor.cpp:148-179): quantise the BF16 rows with global_scale 1, then
// the NVFP4 product with alpha = weight_scale_2, BF16 out.  The tensor-core
// GEMM of the reference is replaced by its software gemv (see file header).
static void project_rows(const std::uint16_t* input, int batch_rows, const std::uint8_t* weight,
                         const std::uint8_t* weight_scales, float alpha, int rows, int columns,
                         std::uint16_t* output) {
    std::vector<std::uint8_t> packed(static_cast<std::size_t>(batch_rows) * columns / 2);
    std::vector<std::uint8_t> scales(static_cast<std::size_t>(batch_rows) * columns / 16);
    orc_nvfp4_quantize(input, packed.data(), scales.data(), static_cast<long>(batch_rows) * columns / 16, 1.0F);
    orc_nvfp4_gemv(packed.data(), weight, scales.data(), weight_scales, output, batch_rows, rows, columns, alpha);
}

// The whole block for `rows` tokens, following Model::Impl::run_moe_rows
// (src/model.cpp:1486-1573) with the device-grouped law for the routed experts
// (gate/up -> swiglu -> down -> expert_combine_rows) and the shared expert
// added afterwards (src/model.cpp:1565-1572).  rows == 1 follows run_moe
// (src/model.cpp:1677-1729), which differs only in the logits summation order.
//
// Expert bank: for expert e (0..experts-1 routed, index `experts` = shared) and
// kind k (0 gate, 1 up, 2 down) the packed weight is at
//   weights + (e*3 + k) * weight_stride, linear scales at
//   scales + (e*3 + k) * scale_stride, alpha at alphas[e*3 + k]
// (bank index expert*3 + kind: cuda/nvfp4_grouped.cu:133).
// host_law != 0 switches the routed combine to the host-scheduled law
// (src/model.cpp:1522-1563: zeroed BF16 output, experts in ascending id,
// scatter_add_scaled_rows).
// Optional outputs (may be null): logits [rows,experts], ids/route_weights
// [rows,8], mixed [rows*8, hidden] (BF16 down outputs per assignment).
void orc_moe_forward(const std::uint16_t* x, const std::uint16_t* router_w, const float* bias,
                     const std::uint8_t* weights, const std::uint8_t* scales, const float* alphas,
                     long weight_stride, long scale_stride, std::uint16_t* out, int rows,
                     int hidden, int intermediate, int experts, float routed_scale, int host_law,
                     float* logits_out, std::int32_t* ids_out, float* route_weights_out,
                     std::uint16_t* mixed_out) {
    const int top = 8;
    std::vector<float> logits(static_cast<std::size_t>(rows) * experts);
    std::vector<std::int32_t> ids(static_cast<std::size_t>(rows) * top);
    std::vector<float> rw(static_cast<std::size_t>(rows) * top);
    orc_router_logits(x, router_w, logits.data(), rows, experts, hidden, rows == 1);
    orc_router_top8(logits.data(), bias, ids.data(), rw.data(), nullptr, rows, experts, routed_scale);
    if (logits_out) std::memcpy(logits_out, logits.data(), logits.size() * 4);
    if (ids_out) std::memcpy(ids_out, ids.data(), ids.size() * 4);
    if (route_weights_out) std::memcpy(route_weights_out, rw.data(), rw.size() * 4);

    const int assignments = rows * top;
    std::vector<std::int32_t> order(assignments), counts(experts), offsets(experts + 1);
    orc_permute(ids.data(), assignments, experts, order.data(), nullptr, counts.data(), offsets.data());

    std::vector<std::uint16_t> mixed(static_cast<std::size_t>(assignments) * hidden);
    auto bank_w = [&](int e, int k) { return weights + static_cast<std::size_t>(e * 3 + k) * weight_stride; };
    auto bank_s = [&](int e, int k) { return scales + static_cast<std::size_t>(e * 3 + k) * scale_stride; };

    for (int e = 0; e < experts; ++e) {
        const int n = counts[e];
        if (n == 0) continue;
        std::vector<std::uint16_t> xin(static_cast<std::size_t>(n) * hidden);
        for (int j = 0; j < n; ++j) {
            const int token = order[offsets[e] + j] / top;
            std::memcpy(xin.data() + static_cast<std::size_t>(j) * hidden,
                        x + static_cast<std::size_t>(token) * hidden, static_cast<std::size_t>(hidden) * 2);
        }
        std::vector<std::uint16_t> gate(static_cast<std::size_t>(n) * intermediate), up(gate.size()),
            down(static_cast<std::size_t>(n) * hidden);
        project_rows(xin.data(), n, bank_w(e, 0), bank_s(e, 0), alphas[e * 3 + 0], intermediate, hidden, gate.data());
        project_rows(xin.data(), n, bank_w(e, 1), bank_s(e, 1), alphas[e * 3 + 1], intermediate, hidden, up.data());
        orc_swiglu(gate.data(), up.data(), gate.data(), static_cast<long>(n) * intermediate);
        project_rows(gate.data(), n, bank_w(e, 2), bank_s(e, 2), alphas[e * 3 + 2], hidden, intermediate, down.data());
        for (int j = 0; j < n; ++j) {
            std::memcpy(mixed.data() + static_cast<std::size_t>(order[offsets[e] + j]) * hidden,
                        down.data() + static_cast<std::size_t>(j) * hidden, static_cast<std::size_t>(hidden) * 2);
        }
    }
    if (mixed_out) std::memcpy(mixed_out, mixed.data(), mixed.size() * 2);

    if (!host_law) {
        orc_expert_combine_rows(mixed.data(), rw.data(), out, rows, top, hidden);
    } else {
        std::memset(out, 0, static_cast<std::size_t>(rows) * hidden * 2);
        for (int e = 0; e < experts; ++e) {
            for (int j = 0; j < counts[e]; ++j) {
                const std::int32_t flat = order[offsets[e] + j];
                const std::int32_t token = flat / top;
                const float scale = rw[flat];
                orc_scatter_add_scaled_rows(out, mixed.data() + static_cast<std::size_t>(flat) * hidden, &token,
                                            &scale, 1, hidden);
            }
        }
    }

    // shared expert: every row, weight 1, added after the routed combine.
    {
        const int e = experts;
        std::vector<std::uint16_t> gate(static_cast<std::size_t>(rows) * intermediate), up(gate.size()),
            down(static_cast<std::size_t>(rows) * hidden);
        project_rows(x, rows, bank_w(e, 0), bank_s(e, 0), alphas[e * 3 + 0], intermediate, hidden, gate.data());
        project_rows(x, rows, bank_w(e, 1), bank_s(e, 1), alphas[e * 3 + 1], intermediate, hidden, up.data());
        orc_swiglu(gate.data(), up.data(), gate.data(), static_cast<long>(rows) * intermediate);
        project_rows(gate.data(), rows, bank_w(e, 2), bank_s(e, 2), alphas[e * 3 + 2], hidden, intermediate, down.data());
        orc_add_inplace(out, down.data(), static_cast<long>(rows) * hidden);
    }
}

// Model::Impl::run_dense_rows (src/model.cpp:1476-1484): gate and up projections of the token rows, SwiGLU in
// BF16, down projection; each projection is project_rows above.  weights/scales: the three matrices (gate, up,
// down) back to back at `weight_stride` / `scale_stride`, linear scales.
void orc_dense_forward(const std::uint16_t* x, const std::uint8_t* weights, const std::uint8_t* scales,
                       const float* alphas, long weight_stride, long scale_stride, std::uint16_t* out, int rows,
                       int hidden, int intermediate) {
    std::vector<std::uint16_t> gate(static_cast<std::size_t>(rows) * intermediate), up(gate.size());
    project_rows(x, rows, weights, scales, alphas[0], intermediate, hidden, gate.data());
    project_rows(x, rows, weights + weight_stride, scales + scale_stride, alphas[1], intermediate, hidden, up.data());
    orc_swiglu(gate.data(), up.data(), gate.data(), static_cast<long>(rows) * intermediate);
    project_rows(gate.data(), rows, weights + 2 * weight_stride, scales + 2 * scale_stride, alphas[2], hidden, intermediate, out);
}

// FNV-1a over BF16 bytes, low byte first: the determinism hash of
// tests/moe_forward_test.cpp:61-70.
std::uint64_t orc_fnv1a_bf16(const std::uint16_t* values, long n) {
    std::uint64_t hash = 1469598103934665603ULL;
    for (long i = 0; i < n; ++i) {
        hash ^= values[i] & 0xffU;
        hash *= 1099511628211ULL;
        hash ^= values[i] >> 8;
        hash *= 1099511628211ULL;
    }
    return hash;
}

}  // extern "C"
