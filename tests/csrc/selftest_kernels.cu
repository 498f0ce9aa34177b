// Test-only kernels, built into their own library by the test-suite (not part of the product library or its ABI).
//
// esp_selftest_umma: building-block check for the tcgen05.mma operand forms used by the prefill kernel: one CTA
// computes D[128,128] fp32 = A[128,128] * B^T through an 8-step K=16 MMA chain.
//   mode 0: A and B K-major in shared memory (the Q*K^T form);
//   mode 1: A K-major, B MN-major in shared memory (B given as [K=128, N=128] row-major, the P*V form);
//   mode 2: A converted to 16-bit and staged in tensor memory, B MN-major (the P*V form actually used).
// esp_selftest_bounded_wait: the product's own bounded mbarrier wait (mbar_wait_bounded, the function every wait of
// the prefill kernel goes through) on a barrier nothing ever completes: it must give up after `limit_cycles`, write 1
// to *result_dev and return normally, leaving the context usable.  (2 would mean the barrier completed.)
#include <type_traits>

#include "../../loongserve_b200/csrc/esp_common.cuh"
#include "../../loongserve_b200/csrc/sm100_ptx.cuh"

namespace esp {
using namespace ptx;

// Store one 16-byte chunk (8 elements) of row `r`, chunk `c` (0..15) into a [128 rows x 128 cols]
// 16-bit tile kept as two 64-column panels of 128-byte rows with the 128-byte swizzle.
__device__ __forceinline__ void store_swizzled(uint8_t* tile, int r, int c, uint4 v) {
    const int panel = c >> 3, cc = c & 7;
    *reinterpret_cast<uint4*>(tile + panel * 16384 + r * 128 + ((cc ^ (r & 7)) << 4)) = v;
}

template <typename T>
__global__ void __launch_bounds__(128, 1) selftest_umma_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                              float* __restrict__ d, int mode) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    uint8_t* sA = gen; uint8_t* sB = gen + 32768;
    const uint32_t bar = base + 65536;
    volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(gen + 65536 + 8);
    const int warp = threadIdx.x >> 5, r = threadIdx.x;

    if (threadIdx.x == 0) { mbar_init(bar, 1); fence_barrier_init(); }
    if (warp == 0) { tmem_alloc(base + 65536 + 8, 256); tmem_relinquish(); }
    // row r of A (K contiguous) and row r of B.  For modes 1/2, B is [K, N] row-major, i.e. its rows
    // are K indices and the tile is used as an MN-major operand; the smem image is the same.
    for (int c = 0; c < 16; ++c) {
        store_swizzled(sA, r, c, *reinterpret_cast<const uint4*>(a + r * 128 + c * 8));
        store_swizzled(sB, r, c, *reinterpret_cast<const uint4*>(b + r * 128 + c * 8));
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    if (mode == 2) {
        // stage A in tensor memory: lane = row, 32-bit column c holds elements (2c, 2c+1)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint4 v = *reinterpret_cast<const uint4*>(a + r * 128 + h * 64 + i * 8);
                pk[4 * i] = v.x; pk[4 * i + 1] = v.y; pk[4 * i + 2] = v.z; pk[4 * i + 3] = v.w;
            }
            tmem_st32(tmem + lane_base + 128 + h * 32, pk);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
    }
    constexpr uint32_t fmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
    if (threadIdx.x == 0) {
        const uint32_t idesc = make_idesc(fmt, mode == 0 ? 0u : 1u, 128, 128);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t koff = (k >> 2) * 16384 + (k & 3) * 32;
            if (mode == 0)
                umma_ss(tmem, desc_kmajor_sw128(base + koff), desc_kmajor_sw128(base + 32768 + koff), idesc, k > 0);
            else if (mode == 1)
                umma_ss(tmem, desc_kmajor_sw128(base + koff), desc_mnmajor_sw128(base + 32768 + k * 2048, 16384), idesc, k > 0);
            else
                umma_ts(tmem, tmem + 128 + k * 8, desc_mnmajor_sw128(base + 32768 + k * 2048, 16384), idesc, k > 0);
        }
        umma_commit(bar);
    }
    // bounded wait for the MMA chain
    bool ok = false;
    for (int it = 0; it < (1 << 22); ++it) { if (mbar_try_wait(bar, 0)) { ok = true; break; } }
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t x[32];
            tmem_ld32(tmem + lane_base + c * 32, x);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) d[r * 128 + c * 32 + i] = __uint_as_float(x[i]);
        }
    } else {
        for (int i = 0; i < 128; ++i) d[r * 128 + i] = __int_as_float(0x7fc00000);   // NaN marks a timeout
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 256); }
}

__device__ long long g_selftest_limit;

__global__ void selftest_bounded_wait_kernel(int* result) {
    __shared__ __align__(8) unsigned long long s_bar;
    const uint32_t bar = smem_u32(&s_bar);
    if (threadIdx.x == 0) { mbar_init(bar, 1); fence_barrier_init(); }
    __syncthreads();
    if (threadIdx.x == 0) {
        const int r = mbar_wait_bounded(bar, 0, &g_selftest_limit, nullptr);
        *result = r == 2 ? 1 : 2;
    }
}

}  // namespace esp

using namespace esp;

extern "C" int esp_selftest_bounded_wait(int64_t limit_cycles, int32_t* result_dev, void* stream) {
    if (!result_dev || limit_cycles <= 0 || limit_cycles > 4000000000LL) return ESP_ERR_BAD_ARG;
    const long long v = limit_cycles;
    if (cudaMemcpyToSymbol(g_selftest_limit, &v, sizeof(v)) != cudaSuccess) return ESP_ERR_CUDA;
    selftest_bounded_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(result_dev);
    return cudaGetLastError() == cudaSuccess ? ESP_OK : ESP_ERR_CUDA;
}

extern "C" int esp_selftest_umma(const void* a, const void* b, float* d, int32_t mode, int32_t dtype, void* stream) {
    if (!a || !b || !d || mode < 0 || mode > 2) return ESP_ERR_BAD_ARG;
    const int smem = 65536 + 64 + 1024;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ESP_DTYPE_F16) {
        if (cudaFuncSetAttribute(selftest_umma_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return ESP_ERR_CUDA;
        selftest_umma_kernel<__half><<<1, 128, smem, s>>>((const __half*)a, (const __half*)b, d, mode);
    } else if (dtype == ESP_DTYPE_BF16) {
        if (cudaFuncSetAttribute(selftest_umma_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return ESP_ERR_CUDA;
        selftest_umma_kernel<__nv_bfloat16><<<1, 128, smem, s>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, d, mode);
    } else {
        return ESP_ERR_BAD_ARG;
    }
    return cudaGetLastError() == cudaSuccess ? ESP_OK : ESP_ERR_CUDA;
}
