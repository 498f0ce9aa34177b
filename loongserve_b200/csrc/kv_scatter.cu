// Token-granular KV pool kernels: scatter, keep-range, scatter+register, index registration,
// decode-stage migration gather/scatter.  Pure byte copies and integer arithmetic (bit-exact).
//
// HBM-bound: every kernel moves whole [heads2, D] token rows (16 KiB for 32+32 heads x 128 x 2 B)
// with 16-byte loads/stores, one row per CTA-iteration, rows spread over a grid that is a multiple of
// the SM count.  Algorithmic bytes per token row: 2 x row bytes (read + write) + 4..8 B of index.
#include "esp_common.cuh"

namespace esp {

char* last_cuda_error_buf() {
    static thread_local char buf[256] = {0};
    return buf;
}

// Slot ids that fall outside the pool are never dereferenced: the row is skipped and the first such id of a run is
// recorded here as {ESP_ERR_BAD_SLOT, kernel id, position of the id in its index array, the id clamped to int32}.
__device__ int g_kv_status[4];

__device__ __forceinline__ bool slot_ok(int64_t slot, int64_t pool_rows, int kernel_id, int64_t pos) {
    if (pool_rows <= 0 || (slot >= 0 && slot < pool_rows)) return true;      // pool_rows <= 0: caller opted out
    if (threadIdx.x == 0 && atomicCAS(&g_kv_status[0], 0, ESP_ERR_BAD_SLOT) == 0) {
        g_kv_status[1] = kernel_id;
        g_kv_status[2] = (int)(pos > 2147483647LL ? 2147483647LL : pos);
        g_kv_status[3] = (int)(slot > 2147483647LL ? 2147483647LL : (slot < -2147483647LL ? -2147483647LL : slot));
    }
    return false;
}

template <bool IDX64>
__device__ __forceinline__ int64_t load_idx(const void* p, int64_t i) {
    if (IDX64) return reinterpret_cast<const int64_t*>(p)[i];
    return static_cast<int64_t>(reinterpret_cast<const int32_t*>(p)[i]);
}

// Copy one token row of `heads2` heads x `head_bytes` bytes with 16-byte accesses by a whole CTA.
// When both sides are dense (head stride == head bytes) the row is one contiguous span.
__device__ __forceinline__ void copy_row(const char* __restrict__ src, int64_t src_head_stride_b,
                                         char* __restrict__ dst, int64_t dst_head_stride_b,
                                         int heads2, int head_bytes) {
    const int vec_per_head = head_bytes >> 4;
    const int total = heads2 * vec_per_head;
    // four independent 16-byte loads in flight per thread before the first store
    for (int i0 = threadIdx.x; i0 < total; i0 += blockDim.x * 4) {
        uint4 val[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * blockDim.x;
            if (i < total) {
                const int h = i / vec_per_head;
                const int c = i - h * vec_per_head;
                val[u] = ld_nc_v4(src + h * src_head_stride_b + (int64_t)c * 16);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * blockDim.x;
            if (i < total) {
                const int h = i / vec_per_head;
                const int c = i - h * vec_per_head;
                *reinterpret_cast<uint4*>(dst + h * dst_head_stride_b + (int64_t)c * 16) = val[u];
            }
        }
    }
}

template <bool IDX64>
__global__ void __launch_bounds__(256) kv_scatter_kernel(
    const char* __restrict__ src, int64_t src_row_b, int64_t src_head_b, char* __restrict__ out,
    int64_t out_row_b, int64_t out_head_b, const void* __restrict__ dest, int64_t n, int heads2,
    int head_bytes, int64_t pool_rows) {
    for (int64_t i = blockIdx.x; i < n; i += gridDim.x) {
        const int64_t d = load_idx<IDX64>(dest, i);
        if (!slot_ok(d, pool_rows, 1, i)) continue;
        copy_row(src + i * src_row_b, src_head_b, out + d * out_row_b, out_head_b, heads2, head_bytes);
    }
}

__global__ void kv_keep_range_kernel(const int32_t* __restrict__ cb, const int32_t* __restrict__ ce,
                                     const int32_t* __restrict__ kvf, int P, int batch,
                                     int32_t* __restrict__ rb, int32_t* __restrict__ re,
                                     int32_t* __restrict__ nl) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= batch) return;
    // mathematical ceiling for either sign of the numerator
    auto cdiv = [P](int a) { return a >= 0 ? (a + P - 1) / P : -((-a) / P); };
    const int b = cdiv(cb[i] - kvf[i]);
    const int e = cdiv(ce[i] - kvf[i]);
    rb[i] = b; re[i] = e; nl[i] = e - b;
}

// grid: (row chunks, batch).  Each CTA walks rows chunk, chunk + gridDim.x, ... of one request.
template <bool IDX64>
__global__ void __launch_bounds__(256) kv_scatter_register_kernel(
    const int32_t* __restrict__ new_len, const int32_t* __restrict__ range_begin,
    const int32_t* __restrict__ range_end, const int64_t* __restrict__ new_len_cumsum,
    const char* __restrict__ kv, int64_t kv_row_b, int64_t kv_head_b,
    const int32_t* __restrict__ kv_b_start_loc, const int32_t* __restrict__ cur_kv_cache_index,
    const void* __restrict__ mem_index, char* __restrict__ pool, int64_t pool_row_b,
    int64_t pool_head_b, int32_t* __restrict__ req_to_token, int64_t rtt_stride,
    const int32_t* __restrict__ b_req_idx, int64_t num_used, int row_cap, int should_register,
    int heads2, int head_bytes, int64_t pool_rows) {
    const int b = blockIdx.y;
    int n_new = new_len[b];
    const int rb = range_begin[b], re = range_end[b];
    if (n_new <= 0 || rb < 0 || re < 0) return;
    if (n_new > row_cap) n_new = row_cap;
    const int64_t base = (b > 0 ? new_len_cumsum[b - 1] : 0) + num_used;
    const int64_t src0 = (int64_t)kv_b_start_loc[b] + rb;
    int32_t* rtt = nullptr;
    if (should_register) rtt = req_to_token + (int64_t)b_req_idx[b] * rtt_stride + cur_kv_cache_index[b];
    for (int n = blockIdx.x; n < n_new; n += gridDim.x) {
        const int64_t slot = load_idx<IDX64>(mem_index, base + n);
        if (!slot_ok(slot, pool_rows, 2, base + n)) continue;
        copy_row(kv + (src0 + n) * kv_row_b, kv_head_b, pool + slot * pool_row_b, pool_head_b, heads2,
                 head_bytes);
        if (should_register && threadIdx.x == 0) rtt[n] = (int32_t)slot;
    }
}

template <bool IDX64>
__global__ void kv_index_register_kernel(int32_t* __restrict__ req_to_token, int64_t rtt_stride,
                                         const int32_t* __restrict__ b_req_idx,
                                         const int32_t* __restrict__ b_seq_len,
                                         const void* __restrict__ memindex, int batch) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= batch) return;
    req_to_token[(int64_t)b_req_idx[i] * rtt_stride + (b_seq_len[i] - 1)] = (int32_t)load_idx<IDX64>(memindex, i);
}

// grid: (chunks, batch); every CTA recomputes the exclusive prefix of b_seq_len for its request with
// a block-wide reduction (batch is small), then copies its share of the slot ids.
template <bool IDX64>
__global__ void __launch_bounds__(256) kv_index_init_kernel(
    int32_t* __restrict__ req_to_token, int64_t rtt_stride, const int32_t* __restrict__ b_req_idx,
    const int32_t* __restrict__ b_seq_len, const void* __restrict__ alloc, int batch) {
    const int b = blockIdx.y;
    __shared__ long long s_part[8];
    long long acc = 0;
    for (int i = threadIdx.x; i < b; i += blockDim.x) acc += b_seq_len[i];
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    long long start = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) start += s_part[w];
    const int n = b_seq_len[b];
    int32_t* dst = req_to_token + (int64_t)b_req_idx[b] * rtt_stride;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        dst[i] = (int32_t)load_idx<IDX64>(alloc, start + i);
}

// Migration: grid (token chunks, batch, layers).  One CTA-iteration copies one token row of one layer.
__global__ void __launch_bounds__(256) mig_gather_kernel(
    char* __restrict__ send_buf, int64_t total_tokens, const int32_t* __restrict__ req_to_token,
    int64_t rtt_stride, int32_t* __restrict__ mem_state, const char* __restrict__ kv_cache,
    int64_t kv_layer_b, int64_t kv_row_b, const int32_t* __restrict__ request_ids,
    const int32_t* __restrict__ num_tokens, const int64_t* __restrict__ cumsum,
    const int32_t* __restrict__ b_seq_len, int row_bytes, int64_t pool_rows) {
    const int b = blockIdx.y, layer = blockIdx.z;
    const int n = num_tokens[b];
    const int L = b_seq_len[b];
    const int64_t off = b > 0 ? cumsum[b - 1] : 0;
    const int32_t* rtt = req_to_token + (int64_t)request_ids[b] * rtt_stride + (L - n);
    for (int i = blockIdx.x; i < n; i += gridDim.x) {
        const int64_t slot = rtt[i];
        if (!slot_ok(slot, pool_rows, 3, off + i)) continue;
        if (layer == 0 && threadIdx.x == 0) mem_state[slot] = 0;
        copy_row(kv_cache + layer * kv_layer_b + slot * kv_row_b, 0,
                 send_buf + ((int64_t)layer * total_tokens + off + i) * row_bytes, 0, 1, row_bytes);
    }
}

template <bool IDX64>
__global__ void __launch_bounds__(256) mig_scatter_kernel(
    const char* __restrict__ recv_buf, int64_t total_tokens, int32_t* __restrict__ req_to_token,
    int64_t rtt_stride, char* __restrict__ kv_cache, int64_t kv_layer_b, int64_t kv_row_b,
    const void* __restrict__ alloc_mem, const int32_t* __restrict__ request_ids,
    const int32_t* __restrict__ num_tokens, const int64_t* __restrict__ cumsum,
    const int32_t* __restrict__ b_seq_len, int row_bytes, int64_t pool_rows) {
    const int b = blockIdx.y, layer = blockIdx.z;
    const int n = num_tokens[b];
    const int L = b_seq_len[b];
    const int64_t off = b > 0 ? cumsum[b - 1] : 0;
    int32_t* rtt = req_to_token + (int64_t)request_ids[b] * rtt_stride + L;
    for (int i = blockIdx.x; i < n; i += gridDim.x) {
        const int64_t slot = load_idx<IDX64>(alloc_mem, off + i);
        if (!slot_ok(slot, pool_rows, 4, off + i)) continue;
        if (layer == 0 && threadIdx.x == 0) rtt[i] = (int32_t)slot;
        copy_row(recv_buf + ((int64_t)layer * total_tokens + off + i) * row_bytes, 0,
                 kv_cache + layer * kv_layer_b + slot * kv_row_b, 0, 1, row_bytes);
    }
}

static inline int row_grid(int64_t rows) {
    const int64_t cap = (int64_t)kNumSMs * 16;
    return (int)(rows < cap ? (rows > 0 ? rows : 1) : cap);
}

static inline int check_rows(int heads2, int head_dim, int elem_bytes, int64_t a, int64_t b, int64_t c,
                             int64_t d) {
    if (heads2 <= 0 || head_dim <= 0 || elem_bytes <= 0) return ESP_ERR_BAD_ARG;
    if (((int64_t)head_dim * elem_bytes) % 16) return ESP_ERR_ALIGNMENT;
    if ((a * elem_bytes) % 16 || (b * elem_bytes) % 16 || (c * elem_bytes) % 16 || (d * elem_bytes) % 16)
        return ESP_ERR_ALIGNMENT;
    return ESP_OK;
}

}  // namespace esp

using namespace esp;

extern "C" const char* esp_strerror(int code) {
    switch (code) {
        case ESP_OK: return "ok";
        case ESP_ERR_BAD_ARG: return "bad argument";
        case ESP_ERR_ALIGNMENT: return "pointer or stride not 16-byte aligned";
        case ESP_ERR_CUDA: return "CUDA call failed";
        case ESP_ERR_DEVICE_TIMEOUT: return "bounded device-side wait timed out";
        case ESP_ERR_UNSUPPORTED: return "unsupported configuration";
        case ESP_ERR_NCCL: return "NCCL call failed";
        case ESP_ERR_TOO_LARGE: return "size beyond the entry point's fixed capacity";
        case ESP_ERR_BAD_SLOT: return "slot id outside the pool (row skipped)";
        default: return "unknown error";
    }
}

extern "C" const char* esp_last_cuda_error(void) { return last_cuda_error_buf(); }
extern "C" int esp_abi_version(void) { return ESP_ABI_VERSION; }

extern "C" int esp_kv_scatter(const void* src, int64_t src_row_stride, int64_t src_head_stride,
                              void* out, int64_t out_row_stride, int64_t out_head_stride,
                              const void* dest, int32_t idx64, int64_t n, int32_t heads2,
                              int32_t head_dim, int32_t elem_bytes, int64_t pool_rows, void* stream) {
    if (n == 0) return ESP_OK;
    if (!src || !out || !dest || n < 0) return ESP_ERR_BAD_ARG;
    int rc = check_rows(heads2, head_dim, elem_bytes, src_row_stride, src_head_stride, out_row_stride,
                        out_head_stride);
    if (rc) return rc;
    if (!aligned16(src) || !aligned16(out)) return ESP_ERR_ALIGNMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int hb = head_dim * elem_bytes;
    const char* sp = (const char*)src; char* op = (char*)out;
    if (idx64)
        kv_scatter_kernel<true><<<row_grid(n), 256, 0, s>>>(sp, src_row_stride * elem_bytes,
            src_head_stride * elem_bytes, op, out_row_stride * elem_bytes, out_head_stride * elem_bytes,
            dest, n, heads2, hb, pool_rows);
    else
        kv_scatter_kernel<false><<<row_grid(n), 256, 0, s>>>(sp, src_row_stride * elem_bytes,
            src_head_stride * elem_bytes, op, out_row_stride * elem_bytes, out_head_stride * elem_bytes,
            dest, n, heads2, hb, pool_rows);
    ESP_LAUNCH_CHECK("kv_scatter_kernel");
    return ESP_OK;
}

extern "C" int esp_kv_keep_range(const int32_t* cache_begin, const int32_t* cache_end,
                                 const int32_t* kv_first, int32_t num_peers, int32_t batch,
                                 int32_t* range_begin, int32_t* range_end, int32_t* new_len,
                                 void* stream) {
    if (batch == 0) return ESP_OK;
    if (!cache_begin || !cache_end || !kv_first || !range_begin || !range_end || !new_len ||
        num_peers <= 0 || batch < 0)
        return ESP_ERR_BAD_ARG;
    kv_keep_range_kernel<<<(batch + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
        cache_begin, cache_end, kv_first, num_peers, batch, range_begin, range_end, new_len);
    ESP_LAUNCH_CHECK("kv_keep_range_kernel");
    return ESP_OK;
}

extern "C" int esp_kv_scatter_register(
    int32_t batch, const int32_t* new_len, const int32_t* range_begin, const int32_t* range_end,
    const int64_t* new_len_cumsum, const void* kv, int64_t kv_row_stride, int64_t kv_head_stride,
    const int32_t* kv_b_start_loc, const int32_t* cur_kv_cache_index, const void* mem_index,
    int32_t idx64, void* pool, int64_t pool_row_stride, int64_t pool_head_stride,
    int32_t* req_to_token, int64_t req_to_token_stride, const int32_t* b_req_idx,
    int64_t num_used_mem_index, int32_t max_len_in_batch, int32_t should_register, int32_t heads2,
    int32_t head_dim, int32_t elem_bytes, int64_t pool_rows, void* stream) {
    if (batch == 0 || max_len_in_batch <= 0) return ESP_OK;
    if (!new_len || !range_begin || !range_end || !new_len_cumsum || !kv || !kv_b_start_loc ||
        !mem_index || !pool || batch < 0)
        return ESP_ERR_BAD_ARG;
    if (should_register && (!req_to_token || !b_req_idx || !cur_kv_cache_index)) return ESP_ERR_BAD_ARG;
    int rc = check_rows(heads2, head_dim, elem_bytes, kv_row_stride, kv_head_stride, pool_row_stride,
                        pool_head_stride);
    if (rc) return rc;
    if (!aligned16(kv) || !aligned16(pool)) return ESP_ERR_ALIGNMENT;
    // The reference launches ceil(max_len/256) programs of 256 rows per request: rows beyond that
    // cap are not copied (copy_and_register_kv.py:146-148).
    const int row_cap = ((max_len_in_batch + 255) / 256) * 256;
    int gx = row_grid(max_len_in_batch) / (batch > 0 ? 1 : 1);
    int64_t per = ((int64_t)kNumSMs * 16 + batch - 1) / batch;
    if (gx > per) gx = (int)per;
    if (gx < 1) gx = 1;
    dim3 grid(gx, batch);
    cudaStream_t s = (cudaStream_t)stream;
    const int hb = head_dim * elem_bytes;
#define ESP_SR_ARGS new_len, range_begin, range_end, new_len_cumsum, (const char*)kv,                 \
        kv_row_stride * elem_bytes, kv_head_stride * elem_bytes, kv_b_start_loc, cur_kv_cache_index,   \
        mem_index, (char*)pool, pool_row_stride * elem_bytes, pool_head_stride * elem_bytes,           \
        req_to_token, req_to_token_stride, b_req_idx, num_used_mem_index, row_cap, should_register,    \
        heads2, hb, pool_rows
    if (idx64) kv_scatter_register_kernel<true><<<grid, 256, 0, s>>>(ESP_SR_ARGS);
    else kv_scatter_register_kernel<false><<<grid, 256, 0, s>>>(ESP_SR_ARGS);
#undef ESP_SR_ARGS
    ESP_LAUNCH_CHECK("kv_scatter_register_kernel");
    return ESP_OK;
}

extern "C" int esp_kv_index_register(int32_t* req_to_token, int64_t req_to_token_stride,
                                     const int32_t* b_req_idx, const int32_t* b_seq_len,
                                     const void* memindex, int32_t idx64, int32_t batch, void* stream) {
    if (batch == 0) return ESP_OK;
    if (!req_to_token || !b_req_idx || !b_seq_len || !memindex || batch < 0) return ESP_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (idx64) kv_index_register_kernel<true><<<(batch + 127) / 128, 128, 0, s>>>(
        req_to_token, req_to_token_stride, b_req_idx, b_seq_len, memindex, batch);
    else kv_index_register_kernel<false><<<(batch + 127) / 128, 128, 0, s>>>(
        req_to_token, req_to_token_stride, b_req_idx, b_seq_len, memindex, batch);
    ESP_LAUNCH_CHECK("kv_index_register_kernel");
    return ESP_OK;
}

extern "C" int esp_kv_index_init(int32_t* req_to_token, int64_t req_to_token_stride,
                                 const int32_t* b_req_idx, const int32_t* b_seq_len, const void* alloc,
                                 int32_t idx64, int32_t batch, int32_t max_len_in_batch, void* stream) {
    if (batch == 0 || max_len_in_batch <= 0) return ESP_OK;
    if (!req_to_token || !b_req_idx || !b_seq_len || !alloc || batch < 0) return ESP_ERR_BAD_ARG;
    if (batch > 65536) return ESP_ERR_TOO_LARGE;
    int gx = (max_len_in_batch + 255) / 256;
    if (gx > 64) gx = 64;
    dim3 grid(gx, batch);
    cudaStream_t s = (cudaStream_t)stream;
    if (idx64) kv_index_init_kernel<true><<<grid, 256, 0, s>>>(req_to_token, req_to_token_stride,
        b_req_idx, b_seq_len, alloc, batch);
    else kv_index_init_kernel<false><<<grid, 256, 0, s>>>(req_to_token, req_to_token_stride,
        b_req_idx, b_seq_len, alloc, batch);
    ESP_LAUNCH_CHECK("kv_index_init_kernel");
    return ESP_OK;
}

static int mig_grid(int32_t batch, int32_t max_num_tokens, int32_t num_layers, dim3* grid) {
    if (num_layers > 65535 || batch > 65535) return ESP_ERR_TOO_LARGE;
    int64_t per = ((int64_t)kNumSMs * 16) / ((int64_t)batch * num_layers) + 1;
    int gx = max_num_tokens < per ? max_num_tokens : (int)per;
    if (gx < 1) gx = 1;
    *grid = dim3(gx, batch, num_layers);
    return ESP_OK;
}

extern "C" int esp_mig_gather(void* send_buf, int64_t total_tokens, const int32_t* req_to_token,
                              int64_t req_to_token_stride, int32_t* mem_state, const void* kv_cache,
                              int64_t kv_layer_stride, int64_t kv_row_stride,
                              const int32_t* request_ids, const int32_t* num_tokens,
                              const int64_t* num_tokens_cumsum, const int32_t* b_seq_len,
                              int32_t batch, int32_t max_num_tokens, int32_t num_layers,
                              int32_t heads2, int32_t head_dim, int32_t elem_bytes, int64_t pool_rows, void* stream) {
    if (batch == 0 || total_tokens == 0 || max_num_tokens <= 0) return ESP_OK;
    if (!send_buf || !req_to_token || !mem_state || !kv_cache || !request_ids || !num_tokens ||
        !num_tokens_cumsum || !b_seq_len || batch < 0 || num_layers <= 0)
        return ESP_ERR_BAD_ARG;
    int rc = check_rows(heads2, head_dim, elem_bytes, kv_layer_stride, kv_row_stride, 0, 0);
    if (rc) return rc;
    if (!aligned16(send_buf) || !aligned16(kv_cache)) return ESP_ERR_ALIGNMENT;
    dim3 grid;
    rc = mig_grid(batch, max_num_tokens, num_layers, &grid);
    if (rc) return rc;
    mig_gather_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
        (char*)send_buf, total_tokens, req_to_token, req_to_token_stride, mem_state,
        (const char*)kv_cache, kv_layer_stride * elem_bytes, kv_row_stride * elem_bytes, request_ids,
        num_tokens, num_tokens_cumsum, b_seq_len, heads2 * head_dim * elem_bytes, pool_rows);
    ESP_LAUNCH_CHECK("mig_gather_kernel");
    return ESP_OK;
}

extern "C" int esp_mig_scatter(const void* recv_buf, int64_t total_tokens, int32_t* req_to_token,
                               int64_t req_to_token_stride, void* kv_cache, int64_t kv_layer_stride,
                               int64_t kv_row_stride, const void* alloc_mem, int32_t idx64,
                               const int32_t* request_ids, const int32_t* num_tokens,
                               const int64_t* num_tokens_cumsum, const int32_t* b_seq_len,
                               int32_t batch, int32_t max_num_tokens, int32_t num_layers,
                               int32_t heads2, int32_t head_dim, int32_t elem_bytes, int64_t pool_rows, void* stream) {
    if (batch == 0 || total_tokens == 0 || max_num_tokens <= 0) return ESP_OK;
    if (!recv_buf || !req_to_token || !kv_cache || !alloc_mem || !request_ids || !num_tokens ||
        !num_tokens_cumsum || !b_seq_len || batch < 0 || num_layers <= 0)
        return ESP_ERR_BAD_ARG;
    int rc = check_rows(heads2, head_dim, elem_bytes, kv_layer_stride, kv_row_stride, 0, 0);
    if (rc) return rc;
    if (!aligned16(recv_buf) || !aligned16(kv_cache)) return ESP_ERR_ALIGNMENT;
    dim3 grid;
    rc = mig_grid(batch, max_num_tokens, num_layers, &grid);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    const int rowb = heads2 * head_dim * elem_bytes;
    if (idx64) mig_scatter_kernel<true><<<grid, 256, 0, s>>>((const char*)recv_buf, total_tokens,
        req_to_token, req_to_token_stride, (char*)kv_cache, kv_layer_stride * elem_bytes,
        kv_row_stride * elem_bytes, alloc_mem, request_ids, num_tokens, num_tokens_cumsum, b_seq_len, rowb, pool_rows);
    else mig_scatter_kernel<false><<<grid, 256, 0, s>>>((const char*)recv_buf, total_tokens,
        req_to_token, req_to_token_stride, (char*)kv_cache, kv_layer_stride * elem_bytes,
        kv_row_stride * elem_bytes, alloc_mem, request_ids, num_tokens, num_tokens_cumsum, b_seq_len, rowb, pool_rows);
    ESP_LAUNCH_CHECK("mig_scatter_kernel");
    return ESP_OK;
}

extern "C" int esp_kv_device_status(int32_t out[4], int32_t clear) {
    if (!out) return ESP_ERR_BAD_ARG;
    ESP_CUDA_TRY(cudaDeviceSynchronize());
    ESP_CUDA_TRY(cudaMemcpyFromSymbol(out, g_kv_status, sizeof(int) * 4));
    if (clear) {
        int zero[4] = {0, 0, 0, 0};
        ESP_CUDA_TRY(cudaMemcpyToSymbol(g_kv_status, zero, sizeof(zero)));
    }
    return ESP_OK;
}

extern "C" int esp_memcpy_async(void* dst, const void* src, int64_t bytes, void* stream) {
    if (bytes == 0) return ESP_OK;
    if (!dst || !src || bytes < 0) return ESP_ERR_BAD_ARG;
    ESP_CUDA_TRY(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, (cudaStream_t)stream));
    return ESP_OK;
}

extern "C" int esp_memcpy_2d(void* dst, int64_t dpitch, const void* src, int64_t spitch, int64_t width, int64_t height,
                             int32_t kind, void* stream) {
    if (width == 0 || height == 0) return ESP_OK;
    if (!dst || !src || width < 0 || height < 0 || dpitch < width || spitch < width || kind < 0 || kind > 2) return ESP_ERR_BAD_ARG;
    const cudaMemcpyKind k = kind == 0 ? cudaMemcpyHostToDevice : kind == 1 ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
    ESP_CUDA_TRY(cudaMemcpy2DAsync(dst, (size_t)dpitch, src, (size_t)spitch, (size_t)width, (size_t)height, k, (cudaStream_t)stream));
    return ESP_OK;
}
