// C-ABI driver around the reference's own MoE kernels.  TEST INFRASTRUCTURE ONLY.
//
// Linked together with the reference's cuda/nvfp4_ops.cu, compiled unmodified
// for sm_100a straight from the reference tree (see Makefile target `ref`), so
// the checker runs the reference's own router, quantiser, software NVFP4
// product, SwiGLU and combine kernels on the same GPU as the library under
// test.  Only this driver is ours; it declares the reference operator API by
// including the reference header at build time.
//
// ref_moe_forward_rows restates the device-grouped branch of
// Model::Impl::run_moe_rows (src/model.cpp:1486-1508,1565-1572) /
// run_moe (src/model.cpp:1677-1698,1723-1728).  The reference's two tensor-core
// GEMMs (cuda/nvfp4_grouped.cu, cuda/nvfp4_tensorcore.cu) are Sm120-only and
// cannot execute on sm_100; each is replaced by the reference's software NVFP4
// product nvfp4_gemv (cuda/nvfp4_ops.cu:843-867), the kernel the reference's own
// tests use as the yardstick for those GEMMs
// (cuda/nvfp4_projection_test.cu:222-225,266-270).
#include "p92/kernels.h"

#include <cuda_runtime_api.h>

#include <cstdint>
#include <vector>

namespace ref = p92::cuda;

extern "C" {

int ref_bf16_gemv_f32(const std::uint16_t* x, const std::uint16_t* w, float* out, int rows,
                      int columns, cudaStream_t s) {
    return ref::bf16_gemv_f32(x, w, out, rows, columns, s);
}

int ref_bf16_gemm_f32(const std::uint16_t* x, const std::uint16_t* w, float* out, int batch_rows,
                      int rows, int columns, cudaStream_t s) {
    return ref::bf16_gemm_f32(x, w, out, batch_rows, rows, columns, s);
}

int ref_router_top8_rows(const float* logits, const float* bias, std::int32_t* ids, float* weights,
                         int rows, float routed_scale, cudaStream_t s) {
    return ref::router_top8_rows(logits, bias, ids, weights, rows, routed_scale, s);
}

int ref_router_top8(const float* logits, const float* bias, std::int32_t* ids, float* weights,
                    float routed_scale, cudaStream_t s) {
    return ref::router_top8(logits, bias, ids, weights, routed_scale, s);
}

int ref_nvfp4_quantize(const std::uint16_t* input, std::uint8_t* output, std::uint8_t* scales,
                       int elements, float global_scale, cudaStream_t s) {
    return ref::nvfp4_quantize(input, output, scales, elements, global_scale, s);
}

long ref_nvfp4_swizzled_scale_bytes(int rows, int scale_columns) {
    return static_cast<long>(ref::nvfp4_swizzled_scale_bytes(rows, scale_columns));
}

int ref_nvfp4_swizzle_scales(const std::uint8_t* linear, std::uint8_t* swizzled, int rows,
                             int scale_columns, cudaStream_t s) {
    return ref::nvfp4_swizzle_scales(linear, swizzled, rows, scale_columns, s);
}

int ref_nvfp4_gemv(const std::uint8_t* input, const std::uint8_t* weight,
                   const std::uint8_t* input_scales, const std::uint8_t* weight_scales,
                   std::uint16_t* output, int rows, int columns, float alpha, cudaStream_t s) {
    return ref::nvfp4_gemv(input, weight, input_scales, weight_scales, output, rows, columns, alpha, s);
}

int ref_swiglu(const std::uint16_t* gate, const std::uint16_t* up, std::uint16_t* out, int elements,
               cudaStream_t s) {
    return ref::swiglu(gate, up, out, elements, s);
}

int ref_expert_combine_rows(const std::uint16_t* expert_rows, const float* route_weights,
                            std::uint16_t* output, int batch_rows, int experts, int elements,
                            cudaStream_t s) {
    return ref::expert_combine_rows(expert_rows, route_weights, output, batch_rows, experts, elements, s);
}

int ref_rmsnorm(const std::uint16_t* input, const std::uint16_t* weight, std::uint16_t* output, int rows,
                int elements, float epsilon, cudaStream_t s) {
    return ref::rmsnorm(input, weight, output, rows, elements, epsilon, s);
}

int ref_add_inplace(std::uint16_t* destination, const std::uint16_t* source, int elements,
                    cudaStream_t s) {
    return ref::add_inplace(destination, source, elements, s);
}

// Whole block, reference kernels only.  All pointers are device pointers except
// host_alphas.  Bank addressing: entry (expert*3 + kind) lives at
// weights + entry*weight_stride / scales + entry*scale_stride (linear scales),
// kinds 0/1/2 = gate/up/down, entry `experts` = the shared expert.
// Optional device outputs (nullable): logits [rows,experts], ids [rows,8],
// route_weights [rows,8], mixed [rows*8,hidden].  Synchronises the stream.
int ref_moe_forward_rows(const std::uint16_t* x, const std::uint16_t* router_w, const float* bias,
                         const std::uint8_t* weights, const std::uint8_t* scales,
                         const float* host_alphas, long weight_stride, long scale_stride,
                         std::uint16_t* out, int rows, int hidden, int intermediate, int experts,
                         float routed_scale, float* logits_out, std::int32_t* ids_out,
                         float* route_weights_out, std::uint16_t* mixed_out, cudaStream_t s) {
    constexpr int kTop = 8;
    if (experts != 256) return cudaErrorInvalidValue;   // router_top8 is hard-wired to 256 experts
    float* logits = nullptr;
    std::int32_t* ids = nullptr;
    float* rw = nullptr;
    std::uint8_t *xq = nullptr, *xs = nullptr, *hq = nullptr, *hs = nullptr;
    std::uint16_t *gate = nullptr, *up = nullptr, *mixed = nullptr, *shared_down = nullptr;
    const std::size_t assignments = static_cast<std::size_t>(rows) * kTop;
    int status = cudaSuccess;
#define REF_TRY(call)                         \
    do {                                      \
        status = static_cast<int>(call);      \
        if (status != cudaSuccess) goto done; \
    } while (0)
    {
        REF_TRY(cudaMalloc(&logits, sizeof(float) * rows * experts));
        REF_TRY(cudaMalloc(&ids, sizeof(std::int32_t) * assignments));
        REF_TRY(cudaMalloc(&rw, sizeof(float) * assignments));
        REF_TRY(cudaMalloc(&xq, static_cast<std::size_t>(rows) * hidden / 2));
        REF_TRY(cudaMalloc(&xs, static_cast<std::size_t>(rows) * hidden / 16));
        REF_TRY(cudaMalloc(&hq, assignments * intermediate / 2));
        REF_TRY(cudaMalloc(&hs, assignments * intermediate / 16));
        REF_TRY(cudaMalloc(&gate, 2 * assignments * intermediate));
        REF_TRY(cudaMalloc(&up, 2 * assignments * intermediate));
        REF_TRY(cudaMalloc(&mixed, 2 * assignments * hidden));
        REF_TRY(cudaMalloc(&shared_down, 2 * static_cast<std::size_t>(rows) * hidden));

        // src/model.cpp:1679 (rows == 1) vs :1488 (rows > 1)
        if (rows == 1) REF_TRY(ref::bf16_gemv_f32(x, router_w, logits, experts, hidden, s));
        else REF_TRY(ref::bf16_gemm_f32(x, router_w, logits, rows, experts, hidden, s));
        REF_TRY(ref::router_top8_rows(logits, bias, ids, rw, rows, routed_scale, s));
        std::vector<std::int32_t> host_ids(assignments);
        REF_TRY(cudaMemcpyAsync(host_ids.data(), ids, sizeof(std::int32_t) * assignments,
                                cudaMemcpyDeviceToHost, s));
        REF_TRY(cudaStreamSynchronize(s));

        // src/executor.cpp:53-55: the token row is quantised once, shared by its 8 slots.
        REF_TRY(ref::nvfp4_quantize(x, xq, xs, rows * hidden, 1.0F, s));
        auto w_at = [&](int e, int k) { return weights + static_cast<std::size_t>(e * 3 + k) * weight_stride; };
        auto s_at = [&](int e, int k) { return scales + static_cast<std::size_t>(e * 3 + k) * scale_stride; };
        for (int row = 0; row < rows; ++row) {
            for (int slot = 0; slot < kTop; ++slot) {
                const std::size_t a = static_cast<std::size_t>(row) * kTop + slot;
                const int e = host_ids[a];
                const std::uint8_t* xin = xq + static_cast<std::size_t>(row) * hidden / 2;
                const std::uint8_t* xsc = xs + static_cast<std::size_t>(row) * hidden / 16;
                REF_TRY(ref::nvfp4_gemv(xin, w_at(e, 0), xsc, s_at(e, 0), gate + a * intermediate,
                                        intermediate, hidden, host_alphas[e * 3 + 0], s));
                REF_TRY(ref::nvfp4_gemv(xin, w_at(e, 1), xsc, s_at(e, 1), up + a * intermediate,
                                        intermediate, hidden, host_alphas[e * 3 + 1], s));
            }
        }
        REF_TRY(ref::swiglu(gate, up, gate, static_cast<int>(assignments) * intermediate, s));
        // src/executor.cpp:85-91: every (row, slot) intermediate row is re-quantised.
        REF_TRY(ref::nvfp4_quantize(gate, hq, hs, static_cast<int>(assignments) * intermediate, 1.0F, s));
        for (std::size_t a = 0; a < assignments; ++a) {
            const int e = host_ids[a];
            REF_TRY(ref::nvfp4_gemv(hq + a * intermediate / 2, w_at(e, 2), hs + a * intermediate / 16,
                                    s_at(e, 2), mixed + a * hidden, hidden, intermediate,
                                    host_alphas[e * 3 + 2], s));
        }
        REF_TRY(ref::expert_combine_rows(mixed, rw, out, rows, kTop, hidden, s));

        // shared expert (src/model.cpp:1565-1572): its own quantise of x is
        // bit-identical to xq, so xq is reused.
        const int e = experts;
        for (int row = 0; row < rows; ++row) {
            const std::uint8_t* xin = xq + static_cast<std::size_t>(row) * hidden / 2;
            const std::uint8_t* xsc = xs + static_cast<std::size_t>(row) * hidden / 16;
            REF_TRY(ref::nvfp4_gemv(xin, w_at(e, 0), xsc, s_at(e, 0), gate + static_cast<std::size_t>(row) * intermediate,
                                    intermediate, hidden, host_alphas[e * 3 + 0], s));
            REF_TRY(ref::nvfp4_gemv(xin, w_at(e, 1), xsc, s_at(e, 1), up + static_cast<std::size_t>(row) * intermediate,
                                    intermediate, hidden, host_alphas[e * 3 + 1], s));
        }
        REF_TRY(ref::swiglu(gate, up, gate, rows * intermediate, s));
        REF_TRY(ref::nvfp4_quantize(gate, hq, hs, rows * intermediate, 1.0F, s));
        for (int row = 0; row < rows; ++row) {
            REF_TRY(ref::nvfp4_gemv(hq + static_cast<std::size_t>(row) * intermediate / 2, w_at(e, 2),
                                    hs + static_cast<std::size_t>(row) * intermediate / 16, s_at(e, 2),
                                    shared_down + static_cast<std::size_t>(row) * hidden, hidden, intermediate,
                                    host_alphas[e * 3 + 2], s));
        }
        REF_TRY(ref::add_inplace(out, shared_down, rows * hidden, s));

        if (logits_out) REF_TRY(cudaMemcpyAsync(logits_out, logits, sizeof(float) * rows * experts, cudaMemcpyDeviceToDevice, s));
        if (ids_out) REF_TRY(cudaMemcpyAsync(ids_out, ids, sizeof(std::int32_t) * assignments, cudaMemcpyDeviceToDevice, s));
        if (route_weights_out) REF_TRY(cudaMemcpyAsync(route_weights_out, rw, sizeof(float) * assignments, cudaMemcpyDeviceToDevice, s));
        if (mixed_out) REF_TRY(cudaMemcpyAsync(mixed_out, mixed, 2 * assignments * hidden, cudaMemcpyDeviceToDevice, s));
        REF_TRY(cudaStreamSynchronize(s));
    }
done:
#undef REF_TRY
    cudaFree(logits); cudaFree(ids); cudaFree(rw); cudaFree(xq); cudaFree(xs); cudaFree(hq); cudaFree(hs);
    cudaFree(gate); cudaFree(up); cudaFree(mixed); cudaFree(shared_down);
    return status;
}

}  // extern "C"
