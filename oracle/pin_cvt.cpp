// Conversion pin for the CPU oracle.  TEST INFRASTRUCTURE ONLY.
//
// Wraps the CUDA toolkit's own host-side E2M1 / E4M3 conversions (cuda_fp4.h,
// cuda_fp8.h: the constructors the reference calls at cuda/nvfp4_ops.cu:828,
// :836-839 and :26-36) behind a C ABI so the tests can compare the oracle's
// hand-written encoders and decoders against them value by value.
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include <cstdint>

extern "C" {

void pin_encode_e4m3_array(const float* in, std::uint8_t* out, long n) {
    for (long i = 0; i < n; ++i) out[i] = __nv_fp8_e4m3(in[i]).__x;
}

// Low nibble = first value, high nibble = second value of the pair.
void pin_encode_e2m1x2_array(const float* in, std::uint8_t* out, long pairs) {
    for (long i = 0; i < pairs; ++i) {
        out[i] = __nv_fp4x2_e2m1(make_float2(in[2 * i], in[2 * i + 1])).__x;
    }
}

float pin_decode_e4m3(std::uint8_t bits) {
    __nv_fp8_e4m3 value;
    value.__x = bits;
    return static_cast<float>(value);
}

float pin_decode_e2m1(std::uint8_t bits) {
    __nv_fp4_e2m1 value;
    value.__x = bits & 0x0fU;
    return static_cast<float>(value);
}

}  // extern "C"
