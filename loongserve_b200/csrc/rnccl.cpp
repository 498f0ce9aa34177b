// Raw NCCL point-to-point layer (C ABI).  One communicator, one private non-blocking stream, grouped
// byte sends/receives over NVLink, event fences against a caller-supplied stream.
#include <cuda_runtime.h>
#include <nccl.h>
#include <stdio.h>
#include <string.h>

#include "../../include/esp_attention.h"
#include "../../include/esp_rnccl.h"

struct esp_rnccl_comm {
    ncclComm_t comm;
    cudaStream_t stream;
    cudaEvent_t ev_in, ev_out;
    int world_size, rank, device;
};

static thread_local char g_err[256] = {0};

static int fail_nccl(ncclResult_t r, const char* what) {
    snprintf(g_err, sizeof(g_err), "%s: %s", what, ncclGetErrorString(r));
    return ESP_ERR_NCCL;
}
static int fail_cuda(cudaError_t e, const char* what) {
    snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
    return ESP_ERR_CUDA;
}
#define NCCL_TRY(x) do { ncclResult_t _r = (x); if (_r != ncclSuccess) return fail_nccl(_r, #x); } while (0)
#define CUDA_TRY(x) do { cudaError_t _e = (x); if (_e != cudaSuccess) return fail_cuda(_e, #x); } while (0)

extern "C" const char* esp_rnccl_last_error(void) { return g_err; }

extern "C" int esp_rnccl_unique_id(uint8_t out[ESP_RNCCL_UNIQUE_ID_BYTES]) {
    if (!out) return ESP_ERR_BAD_ARG;
    static_assert(sizeof(ncclUniqueId) == ESP_RNCCL_UNIQUE_ID_BYTES, "unexpected ncclUniqueId size");
    ncclUniqueId id;
    NCCL_TRY(ncclGetUniqueId(&id));
    memcpy(out, id.internal, ESP_RNCCL_UNIQUE_ID_BYTES);
    return ESP_OK;
}

extern "C" int esp_rnccl_create(const uint8_t id_bytes[ESP_RNCCL_UNIQUE_ID_BYTES], int32_t world_size,
                                int32_t rank, esp_rnccl_comm** out) {
    if (!id_bytes || !out || world_size <= 0 || rank < 0 || rank >= world_size) return ESP_ERR_BAD_ARG;
    ncclUniqueId id;
    memcpy(id.internal, id_bytes, ESP_RNCCL_UNIQUE_ID_BYTES);
    esp_rnccl_comm* c = new esp_rnccl_comm();
    c->world_size = world_size; c->rank = rank;
    cudaError_t e = cudaGetDevice(&c->device);
    if (e != cudaSuccess) { delete c; return fail_cuda(e, "cudaGetDevice"); }
    ncclResult_t r = ncclCommInitRank(&c->comm, world_size, id, rank);
    if (r != ncclSuccess) { delete c; return fail_nccl(r, "ncclCommInitRank"); }
    // Highest priority: the exchange kernels must get SM slots ahead of the queued blocks of a long attention
    // kernel that is already running, otherwise a small send waits for the whole kernel.
    int prio_least = 0, prio_greatest = 0;
    e = cudaDeviceGetStreamPriorityRange(&prio_least, &prio_greatest);
    if (e == cudaSuccess) e = cudaStreamCreateWithPriority(&c->stream, cudaStreamNonBlocking, prio_greatest);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_in, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_out, cudaEventDisableTiming);
    if (e != cudaSuccess) { ncclCommDestroy(c->comm); delete c; return fail_cuda(e, "stream/event creation"); }
    *out = c;
    return ESP_OK;
}

extern "C" int esp_rnccl_destroy(esp_rnccl_comm* c) {
    if (!c) return ESP_ERR_BAD_ARG;
    cudaStreamSynchronize(c->stream);
    ncclResult_t r = ncclCommDestroy(c->comm);
    cudaEventDestroy(c->ev_in);
    cudaEventDestroy(c->ev_out);
    cudaStreamDestroy(c->stream);
    delete c;
    if (r != ncclSuccess) return fail_nccl(r, "ncclCommDestroy");
    return ESP_OK;
}

extern "C" int esp_rnccl_group_start(esp_rnccl_comm* c) {
    if (!c) return ESP_ERR_BAD_ARG;
    NCCL_TRY(ncclGroupStart());
    return ESP_OK;
}

extern "C" int esp_rnccl_group_end(esp_rnccl_comm* c) {
    if (!c) return ESP_ERR_BAD_ARG;
    NCCL_TRY(ncclGroupEnd());
    return ESP_OK;
}

extern "C" int esp_rnccl_send(esp_rnccl_comm* c, const void* data, int64_t bytes, int32_t peer) {
    if (!c || bytes < 0 || peer < 0 || peer >= c->world_size) return ESP_ERR_BAD_ARG;
    if (bytes == 0) return ESP_OK;
    if (!data) return ESP_ERR_BAD_ARG;
    NCCL_TRY(ncclSend(data, (size_t)bytes, ncclChar, peer, c->comm, c->stream));
    return ESP_OK;
}

extern "C" int esp_rnccl_recv(esp_rnccl_comm* c, void* data, int64_t bytes, int32_t peer) {
    if (!c || bytes < 0 || peer < 0 || peer >= c->world_size) return ESP_ERR_BAD_ARG;
    if (bytes == 0) return ESP_OK;
    if (!data) return ESP_ERR_BAD_ARG;
    NCCL_TRY(ncclRecv(data, (size_t)bytes, ncclChar, peer, c->comm, c->stream));
    return ESP_OK;
}

extern "C" int esp_rnccl_fence_in(esp_rnccl_comm* c, void* stream) {
    if (!c) return ESP_ERR_BAD_ARG;
    CUDA_TRY(cudaEventRecord(c->ev_in, (cudaStream_t)stream));
    CUDA_TRY(cudaStreamWaitEvent(c->stream, c->ev_in, 0));
    return ESP_OK;
}

extern "C" int esp_rnccl_fence_out(esp_rnccl_comm* c, void* stream) {
    if (!c) return ESP_ERR_BAD_ARG;
    CUDA_TRY(cudaEventRecord(c->ev_out, c->stream));
    CUDA_TRY(cudaStreamWaitEvent((cudaStream_t)stream, c->ev_out, 0));
    return ESP_OK;
}

extern "C" void* esp_rnccl_stream(esp_rnccl_comm* c) { return c ? (void*)c->stream : nullptr; }
