// Element-wise layer kernels needed to run a whole Llama layer around the attention path: RMSNorm,
// in-place rotate-half RoPE, SiLU(gate)*up.  All HBM-bound: 16-byte accesses, fp32 math, one rounding.
// Algorithmic bytes: RMSNorm 2 x tokens x hidden x 2 B (+ weight once); RoPE 2 x tokens x heads x D x 2 B
// (+ cos/sin rows); SiLU*mul tokens x F x 2 B x 3.
#include "esp_common.cuh"

namespace esp {

constexpr int kNormThreads = 256;
constexpr int kNormCache = 4;     // 16-byte vectors cached per thread: rows up to 256*4*8 = 8192 elements stay in registers

template <typename T>
__global__ void __launch_bounds__(kNormThreads) rms_norm_kernel(T* __restrict__ out, const T* __restrict__ in,
                                                                const T* __restrict__ w, int hidden, float eps) {
    const int64_t row = blockIdx.x;
    const uint4* src = reinterpret_cast<const uint4*>(in + row * hidden);
    const uint4* wv = reinterpret_cast<const uint4*>(w);
    uint4* dst = reinterpret_cast<uint4*>(out + row * hidden);
    const int nvec = hidden >> 3;
    uint4 cache[kNormCache];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < kNormCache; ++c) {
        const int i = threadIdx.x + c * kNormThreads;
        if (i < nvec) {
            cache[c] = src[i];
            const uint32_t u[4] = {cache[c].x, cache[c].y, cache[c].z, cache[c].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) { const float2 f = Cvt<T>::to_f2(u[k]); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss); }
        }
    }
    for (int i = threadIdx.x + kNormCache * kNormThreads; i < nvec; i += kNormThreads) {
        const uint4 v = src[i];
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) { const float2 f = Cvt<T>::to_f2(u[k]); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss); }
    }
    __shared__ float s_part[kNormThreads / 32];
    __shared__ float s_inv;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < kNormThreads / 32; ++i) t += s_part[i];
        s_inv = rsqrtf(t / (float)hidden + eps);
    }
    __syncthreads();
    const float inv = s_inv;
    auto emit = [&](int i, uint4 v) {
        const uint4 ww = wv[i];
        const uint32_t u[4] = {v.x, v.y, v.z, v.w}, g[4] = {ww.x, ww.y, ww.z, ww.w};
        uint32_t r[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = Cvt<T>::to_f2(u[k]), h = Cvt<T>::to_f2(g[k]);
            r[k] = Cvt<T>::pack(f.x * inv * h.x, f.y * inv * h.y);
        }
        dst[i] = make_uint4(r[0], r[1], r[2], r[3]);
    };
#pragma unroll
    for (int c = 0; c < kNormCache; ++c) {
        const int i = threadIdx.x + c * kNormThreads;
        if (i < nvec) emit(i, cache[c]);
    }
    for (int i = threadIdx.x + kNormCache * kNormThreads; i < nvec; i += kNormThreads) emit(i, src[i]);
}

// grid (token chunks); each thread rotates 8 dims of the first half with the matching 8 of the second half.
template <typename T>
__global__ void __launch_bounds__(256) rotary_kernel(T* __restrict__ x, const T* __restrict__ cosv, const T* __restrict__ sinv,
                                                     int64_t stride_t, int64_t stride_h, int64_t tokens, int heads, int head_dim) {
    const int vec_per_head = head_dim >> 4;                  // 16-byte vectors in half a head
    const int64_t total = tokens * heads * vec_per_head;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    // two work items per thread and iteration: eight 16-byte loads in flight before the first store
    for (int64_t idx0 = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx0 < total; idx0 += 2 * stride) {
        T* base[2]; uint4 a[2], b[2], c[2], sn[2]; bool on[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int64_t idx = idx0 + u * stride;
            on[u] = idx < total;
            if (on[u]) {
                const int v = (int)(idx % vec_per_head);
                const int64_t th = idx / vec_per_head;
                const int h = (int)(th % heads);
                const int64_t t = th / heads;
                base[u] = x + t * stride_t + (int64_t)h * stride_h + v * 8;
                a[u] = *reinterpret_cast<const uint4*>(base[u]);
                b[u] = *reinterpret_cast<const uint4*>(base[u] + head_dim / 2);
                c[u] = *reinterpret_cast<const uint4*>(cosv + t * (head_dim / 2) + v * 8);
                sn[u] = *reinterpret_cast<const uint4*>(sinv + t * (head_dim / 2) + v * 8);
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (!on[u]) continue;
            const uint32_t ua[4] = {a[u].x, a[u].y, a[u].z, a[u].w}, ub[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
            const uint32_t uc[4] = {c[u].x, c[u].y, c[u].z, c[u].w}, us[4] = {sn[u].x, sn[u].y, sn[u].z, sn[u].w};
            uint32_t ra[4], rb[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 x1 = Cvt<T>::to_f2(ua[k]), x2 = Cvt<T>::to_f2(ub[k]), cc = Cvt<T>::to_f2(uc[k]), ss = Cvt<T>::to_f2(us[k]);
                ra[k] = Cvt<T>::pack(x1.x * cc.x - x2.x * ss.x, x1.y * cc.y - x2.y * ss.y);
                rb[k] = Cvt<T>::pack(x1.x * ss.x + x2.x * cc.x, x1.y * ss.y + x2.y * cc.y);
            }
            *reinterpret_cast<uint4*>(base[u]) = make_uint4(ra[0], ra[1], ra[2], ra[3]);
            *reinterpret_cast<uint4*>(base[u] + head_dim / 2) = make_uint4(rb[0], rb[1], rb[2], rb[3]);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) silu_mul_kernel(T* __restrict__ io, int64_t tokens, int ffn) {
    const int vec = ffn >> 3;
    const int64_t total = tokens * vec;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    // two independent vectors per thread and iteration: four 16-byte loads in flight before the first store
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += 2 * stride) {
        T* g[2]; uint4 a[2], b[2]; bool on[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int64_t id = idx + u * stride;
            on[u] = id < total;
            if (on[u]) {
                const int64_t t = id / vec;
                const int v = (int)(id - t * vec);
                g[u] = io + t * (2 * (int64_t)ffn) + v * 8;
                a[u] = *reinterpret_cast<const uint4*>(g[u]);
                b[u] = *reinterpret_cast<const uint4*>(g[u] + ffn);
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (!on[u]) continue;
            const uint32_t ua[4] = {a[u].x, a[u].y, a[u].z, a[u].w}, ub[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
            uint32_t r[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 x = Cvt<T>::to_f2(ua[k]), up = Cvt<T>::to_f2(ub[k]);
                r[k] = Cvt<T>::pack(x.x / (1.f + __expf(-x.x)) * up.x, x.y / (1.f + __expf(-x.y)) * up.y);
            }
            *reinterpret_cast<uint4*>(g[u]) = make_uint4(r[0], r[1], r[2], r[3]);
        }
    }
}

static inline int ew_grid(int64_t work_items) {
    const int64_t blocks = (work_items + 255) / 256;
    const int64_t cap = (int64_t)kNumSMs * 8;
    return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace esp

using namespace esp;

extern "C" int esp_rms_norm(void* out, const void* in, const void* weight, int64_t tokens, int32_t hidden, float eps,
                            int32_t dtype, void* stream) {
    if (tokens == 0) return ESP_OK;
    if (!out || !in || !weight || tokens < 0 || hidden <= 0) return ESP_ERR_BAD_ARG;
    if (hidden % 8 || !aligned16(out) || !aligned16(in) || !aligned16(weight)) return ESP_ERR_ALIGNMENT;
    if (tokens > 2147483647LL) return ESP_ERR_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ESP_DTYPE_F16)
        rms_norm_kernel<__half><<<(unsigned)tokens, kNormThreads, 0, s>>>((__half*)out, (const __half*)in, (const __half*)weight, hidden, eps);
    else if (dtype == ESP_DTYPE_BF16)
        rms_norm_kernel<__nv_bfloat16><<<(unsigned)tokens, kNormThreads, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)in,
                                                                                 (const __nv_bfloat16*)weight, hidden, eps);
    else return ESP_ERR_BAD_ARG;
    ESP_LAUNCH_CHECK("rms_norm_kernel");
    return ESP_OK;
}

extern "C" int esp_rotary_emb(void* x, const void* cosv, const void* sinv, int64_t x_stride_t, int64_t x_stride_h,
                              int64_t tokens, int32_t heads, int32_t head_dim, int32_t dtype, void* stream) {
    if (tokens == 0 || heads == 0) return ESP_OK;
    if (!x || !cosv || !sinv || tokens < 0 || heads < 0 || head_dim <= 0) return ESP_ERR_BAD_ARG;
    if (head_dim % 16 || (x_stride_t % 8) || (x_stride_h % 8) || !aligned16(x) || !aligned16(cosv) || !aligned16(sinv))
        return ESP_ERR_ALIGNMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int grid = ew_grid(tokens * heads * (head_dim >> 4));
    if (dtype == ESP_DTYPE_F16)
        rotary_kernel<__half><<<grid, 256, 0, s>>>((__half*)x, (const __half*)cosv, (const __half*)sinv, x_stride_t, x_stride_h, tokens, heads, head_dim);
    else if (dtype == ESP_DTYPE_BF16)
        rotary_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((__nv_bfloat16*)x, (const __nv_bfloat16*)cosv, (const __nv_bfloat16*)sinv,
                                                          x_stride_t, x_stride_h, tokens, heads, head_dim);
    else return ESP_ERR_BAD_ARG;
    ESP_LAUNCH_CHECK("rotary_kernel");
    return ESP_OK;
}

extern "C" int esp_silu_and_mul_inplace(void* io, int64_t tokens, int32_t ffn_inter_dim, int32_t dtype, void* stream) {
    if (tokens == 0) return ESP_OK;
    if (!io || tokens < 0 || ffn_inter_dim <= 0) return ESP_ERR_BAD_ARG;
    if (ffn_inter_dim % 8 || !aligned16(io)) return ESP_ERR_ALIGNMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int grid = ew_grid(tokens * (ffn_inter_dim >> 3));
    if (dtype == ESP_DTYPE_F16) silu_mul_kernel<__half><<<grid, 256, 0, s>>>((__half*)io, tokens, ffn_inter_dim);
    else if (dtype == ESP_DTYPE_BF16) silu_mul_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((__nv_bfloat16*)io, tokens, ffn_inter_dim);
    else return ESP_ERR_BAD_ARG;
    ESP_LAUNCH_CHECK("silu_mul_kernel");
    return ESP_OK;
}
