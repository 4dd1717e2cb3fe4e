// Device-side helpers shared by every kernel: bf16 <-> f32 with the exact
// rounding the reference shaders use, e4m3 conversion, warp reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nerve {

// (bits + 0x7fff + lsb) >> 16, no NaN special case: every shader's f32_to_bf16
// (e.g. runtime-rs/shaders/rms_norm_bf16.comp.template:30-35).
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float value) {
    uint32_t bits = __float_as_uint(value);
    uint32_t lsb = (bits >> 16) & 1u;
    return (bits + 0x7fffu + lsb) >> 16;
}
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits) { return __uint_as_float((bits & 0xffffu) << 16); }
__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }
__device__ __forceinline__ float round_bf16(float value) { return __uint_as_float(f32_to_bf16_bits(value) << 16); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    return (f32_to_bf16_bits(hi) << 16) | f32_to_bf16_bits(lo);
}

// SiLU rounded to bf16 before it is used (silu_multiply_bf16.comp.template:26-29).
__device__ __forceinline__ float rounded_silu(float value) { return round_bf16(value / (1.0f + expf(-value))); }

__device__ __forceinline__ float warp_sum(float value) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_xor_sync(0xffffffffu, value, offset);
    return value;
}
__device__ __forceinline__ float warp_max(float value) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) value = fmaxf(value, __shfl_xor_sync(0xffffffffu, value, offset));
    return value;
}

// e4m3fn byte -> f32 (exact).
__device__ __forceinline__ float e4m3_to_f32(uint8_t code) {
    __half_raw raw = __nv_cvt_fp8_to_halfraw(code, __NV_E4M3);
    return __half2float(__half(raw));
}
// f32 -> e4m3fn, round-to-nearest-even, saturating.
__device__ __forceinline__ uint8_t f32_to_e4m3(float value) {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(value, __NV_SATFINITE, __NV_E4M3));
}

// Programmatic dependent launch: a kernel may start while its predecessor in
// the stream drains; everything before grid_dependency_wait() must not read
// data the predecessor writes (weight prefetch is fine).
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

}  // namespace nerve
