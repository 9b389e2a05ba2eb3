// Host-side wrapper around the REFERENCE's own E4M3 codec, compiled from the
// reference tree where it lies (never copied): include/ida_native/fp8_e4m3.hpp.
// Output goes to oracle/_ref/libref_host.so. Test infrastructure only.
//
// g++ needs the two using-declarations because the header calls signbit /
// isfinite unqualified (fp8_e4m3.hpp:32,34).
#include <cmath>
#include <cstdint>
using std::signbit;
using std::isfinite;
#include "ida_native/fp8_e4m3.hpp"

// cuda_fp8.h's host conversion is the routine __nv_fp8_e4m3(float) and
// __nv_fp8_e5m2(float) run on the host, i.e. what kernels/fp8.cu:49,59 encode with.
#include <cuda_fp8.h>

extern "C" {
uint8_t ref_e4m3_pack(float x, int* finite) {
    const auto p = ida_native::fp8_e4m3::pack(x);
    *finite = p.finite ? 1 : 0;
    return p.bits;
}
float ref_e4m3_unpack(uint8_t b) { return ida_native::fp8_e4m3::unpack(b); }
uint8_t ref_nv_e4m3(float x) { return __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3); }
uint8_t ref_nv_e5m2(float x) { return __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E5M2); }
void ref_e4m3_pack_array(const float* x, uint8_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = ida_native::fp8_e4m3::pack(x[i]).bits;
}
void ref_nv_array(const float* x, uint8_t* out, int64_t n, int is_e5m2) {
    for (int64_t i = 0; i < n; ++i)
        out[i] = __nv_cvt_float_to_fp8(x[i], __NV_SATFINITE, is_e5m2 ? __NV_E5M2 : __NV_E4M3);
}
}
