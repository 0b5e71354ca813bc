// Exposes the HOST paths of the CUDA toolkit converters that the reference
// kernels call (__nv_cvt_float_to_fp8 / __nv_cvt_float_to_fp4) so the oracle's
// own software encoders can be pinned against them.  Test infrastructure only.
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include <cstdint>

extern "C" {

uint8_t pin_e4m3_satfinite(float value) {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(value, __NV_SATFINITE, __NV_E4M3));
}

uint8_t pin_e2m1_rn(float value) {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp4(value, __NV_E2M1, cudaRoundNearest));
}

void pin_e4m3_satfinite_many(const float *in, uint8_t *out, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) out[i] = pin_e4m3_satfinite(in[i]);
}

void pin_e2m1_rn_many(const float *in, uint8_t *out, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) out[i] = pin_e2m1_rn(in[i]);
}

}
