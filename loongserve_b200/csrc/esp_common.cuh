// Shared helpers for the ESP attention kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/esp_attention.h"

namespace esp {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this

// Last CUDA error text, per host thread.
char* last_cuda_error_buf();

inline int cuda_fail(cudaError_t e, const char* what) {
    snprintf(last_cuda_error_buf(), 256, "%s: %s", what, cudaGetErrorString(e));
    return ESP_ERR_CUDA;
}

#define ESP_CUDA_TRY(expr)                                   \
    do {                                                     \
        cudaError_t _e = (expr);                             \
        if (_e != cudaSuccess) return ::esp::cuda_fail(_e, #expr); \
    } while (0)

#define ESP_LAUNCH_CHECK(name)                               \
    do {                                                     \
        cudaError_t _e = cudaGetLastError();                 \
        if (_e != cudaSuccess) return ::esp::cuda_fail(_e, name); \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

__device__ __forceinline__ void st_cs_v4(void* p, uint4 v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <typename T> struct Cvt;
template <> struct Cvt<__half> {
    static __device__ __forceinline__ float2 to_f2(uint32_t u) {
        return __half22float2(*reinterpret_cast<const __half2*>(&u));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};
template <> struct Cvt<__nv_bfloat16> {
    static __device__ __forceinline__ float2 to_f2(uint32_t u) {
        // bf16 -> fp32 is a 16-bit shift
        return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};

}  // namespace esp
