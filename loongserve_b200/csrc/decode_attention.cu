// Distributed flash-decoding for a token-indexed (page size 1) KV pool.
//
// Stage 1 (split-KV partial attention) is HBM-bound: every local K and V head row (D x 2 B = 256 B)
// is read exactly once per kv head with 16-byte non-allocating loads; a half-warp covers one row, so
// a warp instruction fetches two whole rows, and each lane keeps 2 x UNROLL such loads in flight.
// All q heads that share a kv head are served by the same loaded rows.  One pass (online softmax in
// base 2), warp-shuffle reductions, no atomics.  Algorithmic bytes per local token per kv head:
// 512 B of K+V + 4 B slot id per CTA that visits it; plus q and the fp32 partial (o, lse) per block.
//
// Stage 2 merges the partials of one (request, head) with one warp: weights exp(lse_j - max) are
// computed lane-parallel, then the [D] rows are accumulated with float4 loads.
#include "esp_common.cuh"

namespace esp {

constexpr int kDecThreads = 128;          // 4 warps, 8 half-warps
constexpr int kDecUnroll = 4;             // tokens per half-warp per step
constexpr int kDecChunk = 1024;           // slot ids staged in shared memory per chunk
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
// Bound of every cross-GPU flag wait in SM cycles (about a second by default); esp_set_wait_limit_cycles changes it.
__device__ long long g_gate_limit_cycles = 2000000000LL;

// Status of this file's kernels: {code, block, which, value}.  code ESP_ERR_DEVICE_TIMEOUT: a bounded flag wait gave up
// (which = 1 stage-1 gate, 2 merge gate, >= 16 caller-chosen ids of esp_flag_wait; value = the awaited flag value);
// code ESP_ERR_BAD_SLOT: stage 1 met a slot id outside the pool (which = 0, value = the id) and skipped that token.
__device__ int g_decode_status[4];

__device__ __forceinline__ int ld_acquire_sys(const int32_t* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int32_t* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {      // bypass L1: the data was written by another GPU
    uint4 r;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
// One thread waits until *flag >= value (flags only ever grow).  Gives up after kGateLimitCycles, or at once
// when an earlier wait on this device already failed; then records the failure and returns false.
__device__ __noinline__ bool gate_wait(const int32_t* flag, int value, int which, int patience = 1) {
    if (ld_acquire_sys(flag) >= value) return true;
    const long long t0 = clock64();
    unsigned spins = 0;
    while (ld_acquire_sys(flag) < value) {
        if ((++spins & 255u) == 0) {
            if (*reinterpret_cast<volatile int*>(&g_decode_status[0]) != 0) return false;
            if (clock64() - t0 > *reinterpret_cast<volatile long long*>(&g_gate_limit_cycles) * patience) {
                if (atomicCAS(&g_decode_status[0], 0, ESP_ERR_DEVICE_TIMEOUT) == 0) {
                    g_decode_status[1] = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
                    g_decode_status[2] = which;
                    g_decode_status[3] = value;
                }
                return false;
            }
        }
    }
    return true;
}

template <typename T, int G>
__global__ void __launch_bounds__(kDecThreads) decode_stage1_kernel(
    float* __restrict__ mid_o, float* __restrict__ mid_lse, const T* __restrict__ q,
    const T* __restrict__ k, const T* __restrict__ v, int64_t k_stride_t, int64_t k_stride_h,
    int64_t v_stride_t, int64_t v_stride_h, const int32_t* __restrict__ req_to_tokens,
    int64_t rtt_stride, const int32_t* __restrict__ b_req_idx, const int32_t* __restrict__ b_seqlen,
    int batch, int num_q_heads, int group /* q heads per kv head */, int seq_block_size,
    float scale_log2, const int32_t* __restrict__ wait_flag, int wait_value, const int32_t* __restrict__ value_base,
    int64_t pool_rows) {
    const int blk = blockIdx.x;
    const int hg = blockIdx.y;            // group of G consecutive q heads
    const int b = blockIdx.z;
    const int len = b_seqlen[b];
    const int t0 = blk * seq_block_size;
    const int t1 = min(t0 + seq_block_size, len);
    if (t1 <= t0) return;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = lane >> 4, hl = lane & 15;
    const int slot_in_cta = warp * 2 + half;          // 0..7: which token of each group of 8
    const int h0 = hg * G;
    const int kvh = h0 / group;

    __shared__ int32_t s_slots[kDecChunk];
    __shared__ float s_red[4][G][128 + 2];

    // Gated form: q is pushed into this GPU's memory by the master; wait (bounded) until it has arrived.
    const bool gated = wait_flag != nullptr;
    if (gated) {
        __shared__ int s_go;
        if (threadIdx.x == 0) s_go = gate_wait(wait_flag, wait_value + (value_base ? *value_base : 0), 1) ? 1 : 0;
        __syncthreads();
        if (!s_go) return;
    }

    // q (pre-scaled into the log2 domain), 8 dims per lane
    float qf[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const T* qp = q + ((int64_t)b * num_q_heads + h0 + g) * 128 + hl * 8;
        const uint4 qv = gated ? ld_cg_v4(qp) : *reinterpret_cast<const uint4*>(qp);
        const uint32_t w[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = Cvt<T>::to_f2(w[i]);
            qf[g][2 * i] = f.x * scale_log2;
            qf[g][2 * i + 1] = f.y * scale_log2;
        }
    }

    float m_run[G], l_run[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m_run[g] = -INFINITY; l_run[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
    }

    const int32_t* rtt = req_to_tokens + (int64_t)b_req_idx[b] * rtt_stride;
    const T* kbase = k + (int64_t)kvh * k_stride_h + hl * 8;
    const T* vbase = v + (int64_t)kvh * v_stride_h + hl * 8;

    for (int c0 = t0; c0 < t1; c0 += kDecChunk) {
        const int cn = min(kDecChunk, t1 - c0);
        __syncthreads();
        for (int i = threadIdx.x; i < cn; i += kDecThreads) {
            int32_t slot = rtt[c0 + i];
            if (pool_rows > 0 && (slot < 0 || slot >= pool_rows)) {
                // never dereferenced: the token is left out of the softmax and the id is reported
                if (atomicCAS(&g_decode_status[0], 0, ESP_ERR_BAD_SLOT) == 0) {
                    g_decode_status[1] = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
                    g_decode_status[2] = 0;
                    g_decode_status[3] = slot;
                }
                slot = -1;
            }
            s_slots[i] = slot;
        }
        __syncthreads();
        // each step covers 8 * kDecUnroll tokens of the chunk
        for (int base = 0; base < cn; base += 8 * kDecUnroll) {
            uint4 kr[kDecUnroll], vr[kDecUnroll];
            bool valid[kDecUnroll];
#pragma unroll
            for (int u = 0; u < kDecUnroll; ++u) {
                const int ti = base + u * 8 + slot_in_cta;
                int64_t slot = s_slots[ti < cn ? ti : cn - 1];
                valid[u] = ti < cn && slot >= 0;
                slot = slot >= 0 ? slot : 0;
                kr[u] = ld_nc_v4(kbase + slot * k_stride_t);
                vr[u] = ld_nc_v4(vbase + slot * v_stride_t);
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float s[kDecUnroll];
#pragma unroll
                for (int u = 0; u < kDecUnroll; ++u) {
                    const uint32_t w[4] = {kr[u].x, kr[u].y, kr[u].z, kr[u].w};
                    float d = 0.f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = Cvt<T>::to_f2(w[i]);
                        d = fmaf(qf[g][2 * i], f.x, d);
                        d = fmaf(qf[g][2 * i + 1], f.y, d);
                    }
                    s[u] = d;
                }
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) {
#pragma unroll
                    for (int u = 0; u < kDecUnroll; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
                }
                float m_new = m_run[g];
#pragma unroll
                for (int u = 0; u < kDecUnroll; ++u) {
                    s[u] = valid[u] ? s[u] : -INFINITY;
                    m_new = fmaxf(m_new, s[u]);
                }
                const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
                const float alpha = exp2f(m_run[g] - m_use);
                float p[kDecUnroll], psum = 0.f;
#pragma unroll
                for (int u = 0; u < kDecUnroll; ++u) { p[u] = exp2f(s[u] - m_use); psum += p[u]; }
                l_run[g] = l_run[g] * alpha + psum;
                m_run[g] = m_new;
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[g][i] *= alpha;
#pragma unroll
                for (int u = 0; u < kDecUnroll; ++u) {
                    const uint32_t w[4] = {vr[u].x, vr[u].y, vr[u].z, vr[u].w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = Cvt<T>::to_f2(w[i]);
                        acc[g][2 * i] = fmaf(p[u], f.x, acc[g][2 * i]);
                        acc[g][2 * i + 1] = fmaf(p[u], f.y, acc[g][2 * i + 1]);
                    }
                }
            }
        }
    }

    // combine the two half-warps, then the four warps
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float m_o = __shfl_xor_sync(0xffffffffu, m_run[g], 16);
        const float l_o = __shfl_xor_sync(0xffffffffu, l_run[g], 16);
        const float m_new = fmaxf(m_run[g], m_o);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float a_self = exp2f(m_run[g] - m_use), a_oth = exp2f(m_o - m_use);
        l_run[g] = l_run[g] * a_self + l_o * a_oth;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float other = __shfl_xor_sync(0xffffffffu, acc[g][i], 16);
            acc[g][i] = acc[g][i] * a_self + other * a_oth;
        }
        m_run[g] = m_new;
        if (half == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) s_red[warp][g][hl * 8 + i] = acc[g][i];
            if (hl == 0) { s_red[warp][g][128] = m_run[g]; s_red[warp][g][129] = l_run[g]; }
        }
    }
    __syncthreads();
    const int d = threadIdx.x;   // 128 threads == 128 dims
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, s_red[w][g][128]);
        const float Mu = (M == -INFINITY) ? 0.f : M;       // -inf only if every token of the block was skipped
        float L = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float a = exp2f(s_red[w][g][128] - Mu);
            L += s_red[w][g][129] * a;
            o += s_red[w][g][d] * a;
        }
        const int64_t row = ((int64_t)blk * batch + b) * num_q_heads + h0 + g;
        mid_o[row * 128 + d] = L > 0.f ? o / L : 0.f;
        if (d == 0) mid_lse[row] = L > 0.f ? (M + log2f(L)) * kLn2 : -INFINITY;
    }
}

template <typename OT> __device__ __forceinline__ void store4(OT* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<__half>(__half* p, float4 v) {
    uint2 u = make_uint2(Cvt<__half>::pack(v.x, v.y), Cvt<__half>::pack(v.z, v.w));
    *reinterpret_cast<uint2*>(p) = u;
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
    uint2 u = make_uint2(Cvt<__nv_bfloat16>::pack(v.x, v.y), Cvt<__nv_bfloat16>::pack(v.z, v.w));
    *reinterpret_cast<uint2*>(p) = u;
}

// One warp per (request, head); D = 128 -> 4 dims per lane.  4 warps per CTA.
template <typename OT>
__global__ void __launch_bounds__(128) decode_merge_kernel(
    OT* __restrict__ o, float* __restrict__ out_lse, const int32_t* __restrict__ b_seqlen,
    const float* __restrict__ mid_o, const float* __restrict__ mid_lse, int batch, int num_heads,
    int num_blocks, int block_seq, const int32_t* __restrict__ wait_flags, int n_wait, int wait_value,
    const int32_t* __restrict__ value_base) {
    // Gated form: the first n_wait partials are written into this GPU's memory by the peers; each peer raises
    // its flag when its partial is complete.
    if (wait_flags != nullptr) {
        __shared__ int s_go;
        if (threadIdx.x == 0) {
            int okf = 1;
            const int want = wait_value + (value_base ? *value_base : 0);
            for (int i = 0; i < n_wait && okf; ++i) okf = gate_wait(wait_flags + i, want, 2) ? 1 : 0;
            s_go = okf;
        }
        __syncthreads();
        if (!s_go) return;
    }
    const int lane = threadIdx.x & 31;
    const int64_t pair = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (pair >= (int64_t)batch * num_heads) return;
    const int b = (int)(pair / num_heads);
    const int len = b_seqlen[b];
    int n = len <= 0 ? 0 : (len + block_seq - 1) / block_seq;
    if (n > num_blocks) n = num_blocks;
    const int64_t bh = (int64_t)batch * num_heads;
    float M = -INFINITY;
    for (int j = lane; j < n; j += 32) M = fmaxf(M, __ldcg(mid_lse + j * bh + pair));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float wsum = 0.f;
    if (M > -INFINITY) {
        for (int j0 = 0; j0 < n; j0 += 32) {
            const int j = j0 + lane;
            const float wl = j < n ? __expf(__ldcg(mid_lse + j * bh + pair) - M) : 0.f;
            wsum += wl;
            const int cnt = min(32, n - j0);
#pragma unroll 4
            for (int jj = 0; jj < cnt; ++jj) {
                const float w = __shfl_sync(0xffffffffu, wl, jj);
                if (w > 0.f) {
                    const float4 x = __ldcg(reinterpret_cast<const float4*>(mid_o + ((j0 + jj) * bh + pair) * 128 + lane * 4));
                    acc.x = fmaf(w, x.x, acc.x); acc.y = fmaf(w, x.y, acc.y);
                    acc.z = fmaf(w, x.z, acc.z); acc.w = fmaf(w, x.w, acc.w);
                }
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, off);
        const float inv = 1.f / wsum;
        acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    }
    store4<OT>(o + pair * 128 + lane * 4, acc);
    if (lane == 0) out_lse[pair] = (M > -INFINITY) ? M + __logf(wsum) : -INFINITY;
}

template <typename T>
static int launch_stage1(float* mid_o, float* mid_lse, const void* q, const void* k, const void* v,
                         int64_t kst, int64_t ksh, int64_t vst, int64_t vsh, const int32_t* rtt,
                         int64_t rtt_stride, const int32_t* b_req_idx, const int32_t* b_seqlen,
                         int batch, int Hq, int Hkv, int max_len, int bs, float scale_log2,
                         cudaStream_t s, int64_t pool_rows, const int32_t* wait_flag = nullptr, int wait_value = 0,
                         const int32_t* value_base = nullptr) {
    const int group = Hq / Hkv;
    const int nblk = (max_len + bs - 1) / bs;
    int G = 1;
    if (group % 8 == 0) G = 8; else if (group % 4 == 0) G = 4; else if (group % 2 == 0) G = 2;
    dim3 grid(nblk, Hq / G, batch);
#define ESP_S1(GG) decode_stage1_kernel<T, GG><<<grid, kDecThreads, 0, s>>>(mid_o, mid_lse, (const T*)q, \
        (const T*)k, (const T*)v, kst, ksh, vst, vsh, rtt, rtt_stride, b_req_idx, b_seqlen, batch, Hq, \
        group, bs, scale_log2, wait_flag, wait_value, value_base, pool_rows)
    switch (G) {
        case 8: ESP_S1(8); break;
        case 4: ESP_S1(4); break;
        case 2: ESP_S1(2); break;
        default: ESP_S1(1); break;
    }
#undef ESP_S1
    ESP_LAUNCH_CHECK("decode_stage1_kernel");
    return ESP_OK;
}

}  // namespace esp

using namespace esp;

static int decode_stage1_impl(float* mid_o, float* mid_lse, const void* q, const void* k,
                                 const void* v, int64_t k_stride_t, int64_t k_stride_h,
                                 int64_t v_stride_t, int64_t v_stride_h, const int32_t* req_to_tokens,
                                 int64_t req_to_tokens_stride, const int32_t* b_req_idx,
                                 const int32_t* b_seqlen, int32_t batch, int32_t num_q_heads,
                                 int32_t num_kv_heads, int32_t head_dim, int32_t max_len_in_batch,
                                 int32_t seq_block_size, int32_t dtype, float sm_scale, int64_t pool_rows, void* stream,
                                 const int32_t* wait_flag, int32_t wait_value, const int32_t* value_base = nullptr) {
    if (batch == 0 || max_len_in_batch <= 0) return ESP_OK;
    if (!mid_o || !mid_lse || !q || !k || !v || !req_to_tokens || !b_req_idx || !b_seqlen || batch < 0 ||
        num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads || seq_block_size <= 0)
        return ESP_ERR_BAD_ARG;
    if (head_dim != 128) return ESP_ERR_UNSUPPORTED;
    if (batch > 65535 || num_q_heads > 65535) return ESP_ERR_TOO_LARGE;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || (k_stride_t % 8) || (k_stride_h % 8) ||
        (v_stride_t % 8) || (v_stride_h % 8))
        return ESP_ERR_ALIGNMENT;
    const float scale = (sm_scale > 0.f ? sm_scale : 1.0f / sqrtf((float)head_dim)) * kLog2e;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ESP_DTYPE_F16)
        return launch_stage1<__half>(mid_o, mid_lse, q, k, v, k_stride_t, k_stride_h, v_stride_t,
                                     v_stride_h, req_to_tokens, req_to_tokens_stride, b_req_idx,
                                     b_seqlen, batch, num_q_heads, num_kv_heads, max_len_in_batch,
                                     seq_block_size, scale, s, pool_rows, wait_flag, wait_value, value_base);
    if (dtype == ESP_DTYPE_BF16)
        return launch_stage1<__nv_bfloat16>(mid_o, mid_lse, q, k, v, k_stride_t, k_stride_h, v_stride_t,
                                            v_stride_h, req_to_tokens, req_to_tokens_stride, b_req_idx,
                                            b_seqlen, batch, num_q_heads, num_kv_heads,
                                            max_len_in_batch, seq_block_size, scale, s, pool_rows, wait_flag, wait_value, value_base);
    return ESP_ERR_BAD_ARG;
}

extern "C" int esp_decode_stage1(float* mid_o, float* mid_lse, const void* q, const void* k,
                                 const void* v, int64_t k_stride_t, int64_t k_stride_h,
                                 int64_t v_stride_t, int64_t v_stride_h, const int32_t* req_to_tokens,
                                 int64_t req_to_tokens_stride, const int32_t* b_req_idx,
                                 const int32_t* b_seqlen, int32_t batch, int32_t num_q_heads,
                                 int32_t num_kv_heads, int32_t head_dim, int32_t max_len_in_batch,
                                 int32_t seq_block_size, int32_t dtype, float sm_scale, int64_t pool_rows, void* stream) {
    return decode_stage1_impl(mid_o, mid_lse, q, k, v, k_stride_t, k_stride_h, v_stride_t, v_stride_h, req_to_tokens,
                              req_to_tokens_stride, b_req_idx, b_seqlen, batch, num_q_heads, num_kv_heads, head_dim,
                              max_len_in_batch, seq_block_size, dtype, sm_scale, pool_rows, stream, nullptr, 0);
}

extern "C" int esp_decode_stage1_gated(float* mid_o, float* mid_lse, const void* q, const void* k,
                                       const void* v, int64_t k_stride_t, int64_t k_stride_h,
                                       int64_t v_stride_t, int64_t v_stride_h, const int32_t* req_to_tokens,
                                       int64_t req_to_tokens_stride, const int32_t* b_req_idx,
                                       const int32_t* b_seqlen, int32_t batch, int32_t num_q_heads,
                                       int32_t num_kv_heads, int32_t head_dim, int32_t max_len_in_batch,
                                       int32_t seq_block_size, int32_t dtype, float sm_scale, int64_t pool_rows,
                                       const int32_t* wait_flag, int32_t wait_value, const int32_t* value_base, void* stream) {
    if (!wait_flag) return ESP_ERR_BAD_ARG;
    return decode_stage1_impl(mid_o, mid_lse, q, k, v, k_stride_t, k_stride_h, v_stride_t, v_stride_h, req_to_tokens,
                              req_to_tokens_stride, b_req_idx, b_seqlen, batch, num_q_heads, num_kv_heads, head_dim,
                              max_len_in_batch, seq_block_size, dtype, sm_scale, pool_rows, stream, wait_flag, wait_value, value_base);
}

static int decode_merge_impl(void* o, float* out_lse, const int32_t* b_seqlen, const float* mid_o,
                                const float* mid_lse, int32_t batch, int32_t num_heads,
                                int32_t head_dim, int32_t num_blocks, int32_t block_seq,
                                int32_t o_dtype, void* stream, const int32_t* wait_flags, int32_t n_wait,
                                int32_t wait_value, const int32_t* value_base = nullptr) {
    if (batch == 0) return ESP_OK;
    if (!o || !out_lse || !b_seqlen || !mid_o || !mid_lse || batch < 0 || num_heads <= 0 ||
        num_blocks < 0 || block_seq <= 0)
        return ESP_ERR_BAD_ARG;
    if (head_dim != 128) return ESP_ERR_UNSUPPORTED;
    if (!aligned16(mid_o) || !aligned16(o)) return ESP_ERR_ALIGNMENT;
    const int64_t pairs = (int64_t)batch * num_heads;
    const unsigned grid = (unsigned)((pairs + 3) / 4);
    cudaStream_t s = (cudaStream_t)stream;
    switch (o_dtype) {
        case ESP_DTYPE_F32:
            decode_merge_kernel<float><<<grid, 128, 0, s>>>((float*)o, out_lse, b_seqlen, mid_o, mid_lse,
                                                           batch, num_heads, num_blocks, block_seq, wait_flags, n_wait, wait_value, value_base);
            break;
        case ESP_DTYPE_F16:
            decode_merge_kernel<__half><<<grid, 128, 0, s>>>((__half*)o, out_lse, b_seqlen, mid_o,
                                                            mid_lse, batch, num_heads, num_blocks, block_seq, wait_flags, n_wait, wait_value, value_base);
            break;
        case ESP_DTYPE_BF16:
            decode_merge_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>((__nv_bfloat16*)o, out_lse, b_seqlen,
                                                                   mid_o, mid_lse, batch, num_heads,
                                                                   num_blocks, block_seq, wait_flags, n_wait, wait_value, value_base);
            break;
        default: return ESP_ERR_BAD_ARG;
    }
    ESP_LAUNCH_CHECK("decode_merge_kernel");
    return ESP_OK;
}

extern "C" int esp_decode_merge(void* o, float* out_lse, const int32_t* b_seqlen, const float* mid_o,
                                const float* mid_lse, int32_t batch, int32_t num_heads,
                                int32_t head_dim, int32_t num_blocks, int32_t block_seq,
                                int32_t o_dtype, void* stream) {
    return decode_merge_impl(o, out_lse, b_seqlen, mid_o, mid_lse, batch, num_heads, head_dim, num_blocks, block_seq,
                             o_dtype, stream, nullptr, 0, 0);
}

extern "C" int esp_decode_merge_gated(void* o, float* out_lse, const int32_t* b_seqlen, const float* mid_o,
                                      const float* mid_lse, int32_t batch, int32_t num_heads,
                                      int32_t head_dim, int32_t num_blocks, int32_t block_seq,
                                      int32_t o_dtype, const int32_t* wait_flags, int32_t n_wait,
                                      int32_t wait_value, const int32_t* value_base, void* stream) {
    if (n_wait < 0 || (n_wait > 0 && !wait_flags)) return ESP_ERR_BAD_ARG;
    return decode_merge_impl(o, out_lse, b_seqlen, mid_o, mid_lse, batch, num_heads, head_dim, num_blocks, block_seq,
                             o_dtype, stream, n_wait > 0 ? wait_flags : nullptr, n_wait, wait_value, value_base);
}

// ------------------------------------------------------------------------------------------------
// Peer memory: buffers other GPUs of the node can store into directly over NVLink, a push kernel that
// copies a block into every peer's buffer and then raises a flag there, and a one-word signal.
namespace esp {
constexpr int kMaxPushPeers = 16;
struct PushTargets { void* dst[kMaxPushPeers]; int32_t* flag[kMaxPushPeers]; };

// grid = number of peers; one CTA copies `bytes` (multiple of 16) into one peer and then publishes the flag
__global__ void __launch_bounds__(1024) peer_push_kernel(const uint4* __restrict__ src, PushTargets tg, int64_t nvec, int value,
                                                         const int32_t* __restrict__ value_base) {
    uint4* dst = reinterpret_cast<uint4*>(tg.dst[blockIdx.x]);
    for (int64_t i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = src[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(tg.flag[blockIdx.x], value + (value_base ? *value_base : 0));
}
// After a wait on this device has timed out the kernels behind it returned without writing their results, so the
// flag that would announce those results is not raised: the other side then times out too instead of reading garbage.
__global__ void peer_signal_kernel(int32_t* flag, int value, const int32_t* __restrict__ value_base) {
    if (*reinterpret_cast<volatile int*>(&g_decode_status[0]) == ESP_ERR_DEVICE_TIMEOUT) return;
    __threadfence_system();
    st_release_sys(flag, value + (value_base ? *value_base : 0));
}
// One thread waits (bounded) until *flag >= value.
__global__ void flag_wait_kernel(const int32_t* flag, int value, const int32_t* __restrict__ value_base, int which,
                                 int patience) {
    gate_wait(flag, value + (value_base ? *value_base : 0), which, patience);
}
}  // namespace esp

extern "C" int esp_peer_buffer_create(int64_t bytes, void** dev_ptr, uint8_t handle_out[64]) {
    if (bytes <= 0 || !dev_ptr || !handle_out) return ESP_ERR_BAD_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "unexpected IPC handle size");
    void* p = nullptr;
    ESP_CUDA_TRY(cudaMalloc(&p, (size_t)bytes));
    cudaError_t e = cudaMemset(p, 0, (size_t)bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) { cudaFree(p); return cuda_fail(e, "esp_peer_buffer_create"); }
    memcpy(handle_out, &h, 64);
    *dev_ptr = p;
    return ESP_OK;
}

extern "C" int esp_peer_buffer_open(const uint8_t handle[64], void** dev_ptr) {
    if (!handle || !dev_ptr) return ESP_ERR_BAD_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    ESP_CUDA_TRY(cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return ESP_OK;
}

extern "C" int esp_peer_buffer_close(void* dev_ptr) {
    if (!dev_ptr) return ESP_ERR_BAD_ARG;
    ESP_CUDA_TRY(cudaIpcCloseMemHandle(dev_ptr));
    return ESP_OK;
}

extern "C" int esp_peer_buffer_destroy(void* dev_ptr) {
    if (!dev_ptr) return ESP_ERR_BAD_ARG;
    ESP_CUDA_TRY(cudaFree(dev_ptr));
    return ESP_OK;
}

extern "C" int esp_peer_push(const void* src, void* const* peer_dst, int32_t* const* peer_flags, int32_t n_peers,
                             int64_t bytes, int32_t flag_value, const int32_t* value_base, void* stream) {
    if (n_peers == 0) return ESP_OK;
    if (!src || !peer_dst || !peer_flags || n_peers < 0 || bytes < 0) return ESP_ERR_BAD_ARG;
    if (n_peers > kMaxPushPeers) return ESP_ERR_TOO_LARGE;
    if (bytes % 16 || !aligned16(src)) return ESP_ERR_ALIGNMENT;
    PushTargets tg;
    for (int i = 0; i < n_peers; ++i) {
        if (!peer_dst[i] || !peer_flags[i] || !aligned16(peer_dst[i])) return ESP_ERR_BAD_ARG;
        tg.dst[i] = peer_dst[i]; tg.flag[i] = peer_flags[i];
    }
    peer_push_kernel<<<n_peers, 1024, 0, (cudaStream_t)stream>>>((const uint4*)src, tg, bytes / 16, flag_value, value_base);
    ESP_LAUNCH_CHECK("peer_push_kernel");
    return ESP_OK;
}

extern "C" int esp_peer_signal(int32_t* remote_flag, int32_t value, const int32_t* value_base, void* stream) {
    if (!remote_flag) return ESP_ERR_BAD_ARG;
    peer_signal_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(remote_flag, value, value_base);
    ESP_LAUNCH_CHECK("peer_signal_kernel");
    return ESP_OK;
}

extern "C" int esp_flag_wait(const int32_t* flag, int32_t value, const int32_t* value_base, int32_t wait_id,
                             int32_t patience, void* stream) {
    if (!flag || wait_id < 16 || patience < 1 || patience > 1000) return ESP_ERR_BAD_ARG;
    flag_wait_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(flag, value, value_base, wait_id, patience);
    ESP_LAUNCH_CHECK("flag_wait_kernel");
    return ESP_OK;
}

namespace esp { int set_prefill_wait_limit(long long cycles); }

extern "C" int esp_set_wait_limit_cycles(int64_t cycles) {
    if (cycles <= 0) return ESP_ERR_BAD_ARG;
    const long long v = cycles;
    ESP_CUDA_TRY(cudaMemcpyToSymbol(g_gate_limit_cycles, &v, sizeof(v)));
    return set_prefill_wait_limit(v);
}

extern "C" int esp_decode_device_status(int32_t out[4], int32_t clear) {
    if (!out) return ESP_ERR_BAD_ARG;
    ESP_CUDA_TRY(cudaDeviceSynchronize());
    ESP_CUDA_TRY(cudaMemcpyFromSymbol(out, g_decode_status, sizeof(int) * 4));
    if (clear) {
        int zero[4] = {0, 0, 0, 0};
        ESP_CUDA_TRY(cudaMemcpyToSymbol(g_decode_status, zero, sizeof(zero)));
    }
    return ESP_OK;
}

// ------------------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc on the serving path: a worker whose memory pool was
// sized once at start-up and handed over entirely to the KV cache, or a caller replaying a fixed launch
// sequence that must not touch the allocator.  The split-KV decode needs scratch for the per-split
// partial (o, lse) between its two kernels; here that scratch is a fixed array inside the library image,
// so the call needs nothing beyond its inputs and outputs.
//
// Capacity: kNoAllocScratchFloats fp32 values (16 MiB), resident on every GPU that loads the library for
// the life of the process.  The split size is chosen so the partials fit; a batch whose single split
// already exceeds the capacity (batch * q heads * 129 > capacity) is rejected with ESP_ERR_TOO_LARGE.
// All calls on a device share the array: two calls that overlap on the GPU (different streams) race.
// Nothing needs clearing between calls: stage 1 writes every partial that the merge later reads.
constexpr long long kNoAllocScratchFloats = 4ll * 1024 * 1024;
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];

namespace esp {
constexpr int kMaxDevices = 64;
// Device addresses of g_noalloc_scratch, one per device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel can use; the address comes from the runtime, once per
// device, with that device current.
static float* g_noalloc_addr[kMaxDevices] = {nullptr};

static int noalloc_scratch(float** out) {
    int dev = -1;
    ESP_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return ESP_ERR_UNSUPPORTED;
    float* p = g_noalloc_addr[dev];
    if (!p) {
        ESP_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch));
        g_noalloc_addr[dev] = p;      // racing host threads would store the same value
    }
    *out = p;
    return ESP_OK;
}
}  // namespace esp

extern "C" int esp_decode_attention_noalloc(void* o, float* out_lse, const void* q, const void* k,
                                            const void* v, int64_t k_stride_t, int64_t k_stride_h,
                                            int64_t v_stride_t, int64_t v_stride_h,
                                            const int32_t* req_to_tokens, int64_t req_to_tokens_stride,
                                            const int32_t* b_req_idx, const int32_t* b_seqlen,
                                            int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                                            int32_t head_dim, int32_t max_len_in_batch, int32_t dtype,
                                            int32_t o_dtype, float sm_scale, int64_t pool_rows, void* stream) {
    if (batch == 0) return ESP_OK;
    if (!o || !out_lse || !q || !k || !v || !req_to_tokens || !b_req_idx || !b_seqlen || batch < 0 ||
        num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads || max_len_in_batch < 0)
        return ESP_ERR_BAD_ARG;
    if (head_dim != 128) return ESP_ERR_UNSUPPORTED;
    const long long per_split = (long long)batch * num_q_heads * (head_dim + 1);
    if (per_split > kNoAllocScratchFloats) {
        snprintf(last_cuda_error_buf(), 256,
                 "esp_decode_attention_noalloc: batch*heads*(D+1) = %lld floats per split exceeds the fixed scratch of %lld floats",
                 per_split, kNoAllocScratchFloats);
        return ESP_ERR_TOO_LARGE;
    }
    const int max_len = max_len_in_batch > 0 ? max_len_in_batch : 1;
    const long long max_splits = kNoAllocScratchFloats / per_split;
    long long bs = (max_len + max_splits - 1) / max_splits;
    if (bs < 256) bs = 256;
    bs = (bs + 255) / 256 * 256;
    const int nblk = (int)((max_len + bs - 1) / bs);
    float* scratch = nullptr;
    int rc = noalloc_scratch(&scratch);
    if (rc) return rc;
    float* mid_o = scratch;
    float* mid_lse = scratch + (long long)nblk * batch * num_q_heads * head_dim;
    rc = esp_decode_stage1(mid_o, mid_lse, q, k, v, k_stride_t, k_stride_h, v_stride_t, v_stride_h, req_to_tokens,
                           req_to_tokens_stride, b_req_idx, b_seqlen, batch, num_q_heads, num_kv_heads, head_dim,
                           max_len, (int32_t)bs, dtype, sm_scale, pool_rows, stream);
    if (rc) return rc;
    return esp_decode_merge(o, out_lse, b_seqlen, mid_o, mid_lse, batch, num_q_heads, head_dim, nblk, (int32_t)bs,
                            o_dtype, stream);
}
