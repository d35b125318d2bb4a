// Stand-in for <hip/hip_fp16.h>: IEEE binary16 storage with round-to-nearest-even conversions,
// which is what __float2half / __half2float do on the GPU.  TEST INFRASTRUCTURE ONLY.
#pragma once
typedef _Float16 __half;
inline float __half2float(__half h) { return (float)h; }
inline __half __float2half(float f) { return (__half)f; }
