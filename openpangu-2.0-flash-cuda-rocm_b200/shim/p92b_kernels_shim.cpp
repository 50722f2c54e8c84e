// Drop-in definitions of the reference engine's MoE operator entry points on top of libp92moe_b200.so.
//
// The reference calls its kernels through free functions in namespace p92::cuda, declared in its own header
// include/p92/kernels.h.  This translation unit includes THAT header (from the reference checkout, -I<reference>/include)
// and defines the MoE-path functions of it by forwarding to the C ABI of include/p92b_moe.h; a maintainer compiles it
// into the engine's kernel library in place of cuda/nvfp4_grouped.cu and in front of the MoE functions of
// cuda/nvfp4_ops.cu, and links -lp92moe_b200.  Because the signatures come from the reference's header, a drift between
// the two sides is a compile error here (tests/test_shim_compiles.py runs the compiler over this file whenever the
// reference checkout is present).
//
// Every function keeps the reference's contract: asynchronous on `stream`, cudaError_t result that the executor's
// check() turns into std::runtime_error (src/executor.cpp:12-16), *_destroy null-safe and noexcept.
#include "p92/kernels.h"

#include "p92b_moe.h"

#include <new>

namespace p92::cuda {

namespace {
inline cudaError_t rc(int code) { return static_cast<cudaError_t>(code); }
}  // namespace

// The reference's plan is an opaque struct (include/p92/kernels.h:18); here it wraps the library's.
struct Nvfp4GroupedPlan {
    p92b_grouped_plan* impl = nullptr;
};

static_assert(sizeof(Nvfp4ExpertProjection) == sizeof(p92b_expert_projection), "expert table entries are passed through as they are");

cudaError_t nvfp4_grouped_plan_create(Nvfp4GroupedPlan** plan, int groups, int rows, int columns) {
    if (plan == nullptr) return cudaErrorInvalidValue;
    *plan = nullptr;
    Nvfp4GroupedPlan* created = new (std::nothrow) Nvfp4GroupedPlan();
    if (created == nullptr) return cudaErrorMemoryAllocation;
    const cudaError_t status = rc(p92b_nvfp4_grouped_plan_create(&created->impl, groups, rows, columns));
    if (status != cudaSuccess) {
        delete created;
        return status;
    }
    *plan = created;
    return cudaSuccess;
}

void nvfp4_grouped_plan_destroy(Nvfp4GroupedPlan* plan) noexcept {
    if (plan == nullptr) return;
    p92b_nvfp4_grouped_plan_destroy(plan->impl);
    delete plan;
}

cudaError_t nvfp4_grouped_m1(Nvfp4GroupedPlan* plan, const std::uint8_t* packed_input,
                             const std::uint8_t* input_scales_swizzled, const Nvfp4ExpertProjection* expert_bank,
                             const std::int32_t* expert_ids, BFloat16* first_output, BFloat16* second_output,
                             int projection_kind, bool distinct_input_rows, cudaStream_t stream) {
    if (plan == nullptr) return cudaErrorInvalidValue;
    return rc(p92b_nvfp4_grouped_m1(plan->impl, packed_input, input_scales_swizzled,
                                    reinterpret_cast<const p92b_expert_projection*>(expert_bank), expert_ids, first_output,
                                    second_output, projection_kind, distinct_input_rows ? 1 : 0, stream));
}

cudaError_t nvfp4_grouped_rows(Nvfp4GroupedPlan* plan, const std::uint8_t* packed_input,
                               const std::uint8_t* input_scales_swizzled, const Nvfp4ExpertProjection* expert_bank,
                               const std::int32_t* expert_ids, BFloat16* first_output, BFloat16* second_output,
                               int projection_kind, int batch_rows, bool expert_distinct_input_rows,
                               cudaStream_t stream) {
    if (plan == nullptr) return cudaErrorInvalidValue;
    return rc(p92b_nvfp4_grouped_rows(plan->impl, packed_input, input_scales_swizzled,
                                      reinterpret_cast<const p92b_expert_projection*>(expert_bank), expert_ids, first_output,
                                      second_output, projection_kind, batch_rows, expert_distinct_input_rows ? 1 : 0, stream));
}

cudaError_t bf16_gemv_f32(const BFloat16* input, const BFloat16* weight, float* output, int rows, int columns,
                          cudaStream_t stream) {
    return rc(p92b_bf16_gemv_f32(input, weight, output, rows, columns, stream));
}

cudaError_t bf16_gemm_f32(const BFloat16* input, const BFloat16* weight, float* output, int batch_rows, int rows,
                          int columns, cudaStream_t stream) {
    return rc(p92b_bf16_gemm_f32(input, weight, output, batch_rows, rows, columns, stream));
}

cudaError_t router_top8(const float* logits, const float* correction_bias, std::int32_t* expert_ids,
                        float* expert_weights, float routed_scale, cudaStream_t stream) {
    return rc(p92b_router_top8(logits, correction_bias, expert_ids, expert_weights, routed_scale, stream));
}

cudaError_t router_top8_rows(const float* logits, const float* correction_bias, std::int32_t* expert_ids,
                             float* expert_weights, int rows, float routed_scale, cudaStream_t stream) {
    return rc(p92b_router_top8_rows(logits, correction_bias, expert_ids, expert_weights, rows, routed_scale, stream));
}

cudaError_t nvfp4_quantize(const BFloat16* input, std::uint8_t* output, std::uint8_t* scales, int elements,
                           float global_scale, cudaStream_t stream) {
    return rc(p92b_nvfp4_quantize(input, output, scales, elements, global_scale, stream));
}

std::size_t nvfp4_swizzled_scale_bytes(int rows, int scale_columns) {
    return p92b_nvfp4_swizzled_scale_bytes(rows, scale_columns);
}

cudaError_t nvfp4_swizzle_scales(const std::uint8_t* linear, std::uint8_t* swizzled, int rows, int scale_columns,
                                 cudaStream_t stream) {
    return rc(p92b_nvfp4_swizzle_scales(linear, swizzled, rows, scale_columns, stream));
}

cudaError_t swiglu(const BFloat16* gate, const BFloat16* up, BFloat16* output, int elements, cudaStream_t stream) {
    return rc(p92b_swiglu(gate, up, output, elements, stream));
}

cudaError_t expert_combine(const BFloat16* expert_rows, const float* route_weights, BFloat16* output, int experts,
                           int elements, cudaStream_t stream) {
    return rc(p92b_expert_combine(expert_rows, route_weights, output, experts, elements, stream));
}

cudaError_t expert_combine_rows(const BFloat16* expert_rows, const float* route_weights, BFloat16* output,
                                int batch_rows, int experts, int elements, cudaStream_t stream) {
    return rc(p92b_expert_combine_rows(expert_rows, route_weights, output, batch_rows, experts, elements, stream));
}

cudaError_t add_inplace(BFloat16* destination, const BFloat16* source, int elements, cudaStream_t stream) {
    return rc(p92b_add_inplace(destination, source, elements, stream));
}

cudaError_t rmsnorm(const BFloat16* input, const BFloat16* weight, BFloat16* output, int rows, int elements,
                    float epsilon, cudaStream_t stream) {
    return rc(p92b_rmsnorm(input, weight, output, rows, elements, epsilon, stream));
}

cudaError_t rmsnorm_strided(const BFloat16* input, int input_stride, const BFloat16* weight, BFloat16* output,
                            int output_stride, int rows, int elements, float epsilon, cudaStream_t stream) {
    return rc(p92b_rmsnorm_strided(input, input_stride, weight, output, output_stride, rows, elements, epsilon, stream));
}

}  // namespace p92::cuda
