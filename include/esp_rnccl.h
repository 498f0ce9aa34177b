/*
 * esp_rnccl.h -- C ABI of the raw NCCL point-to-point layer used by the ring prefill, the multi-master
 * decode exchange and decode-stage migration.  It replaces the reference's pybind11 module `rnccl`
 * (rnccl/src/main.cpp:61-292): one communicator per process with a private non-blocking stream,
 * grouped byte-typed ncclSend/ncclRecv on that stream, and event fences against a caller stream.
 *
 * Differences from the reference, on purpose: every call returns a status instead of exiting the
 * process (rnccl/src/main.cpp:9-27); the fences take the stream to fence against instead of assuming
 * the legacy default stream (:231-257), and reuse one event instead of creating one per call; the private stream has
 * the highest priority (the reference uses priority 0, :133) so that exchange kernels are not queued behind the
 * blocks of a running attention kernel.
 */
#ifndef ESP_RNCCL_H_
#define ESP_RNCCL_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ESP_RNCCL_UNIQUE_ID_BYTES 128

typedef struct esp_rnccl_comm esp_rnccl_comm;

/* get_nccl_unique_id (rnccl/src/main.cpp:61-65): fills 128 bytes. */
int esp_rnccl_unique_id(uint8_t out[ESP_RNCCL_UNIQUE_ID_BYTES]);
/* RNCCLComm(id, world_size, rank) (:68-144).  Uses the current CUDA device; blocking init. */
int esp_rnccl_create(const uint8_t id[ESP_RNCCL_UNIQUE_ID_BYTES], int32_t world_size, int32_t rank,
                     esp_rnccl_comm** out);
int esp_rnccl_destroy(esp_rnccl_comm* comm);
/* nccl_group_start / nccl_group_end (:178-189). */
int esp_rnccl_group_start(esp_rnccl_comm* comm);
int esp_rnccl_group_end(esp_rnccl_comm* comm);
/* nccl_send / nccl_recv (:192-228): `bytes` raw bytes on the communicator's private stream;
 * zero bytes is a no-op. */
int esp_rnccl_send(esp_rnccl_comm* comm, const void* data, int64_t bytes, int32_t peer);
int esp_rnccl_recv(esp_rnccl_comm* comm, void* data, int64_t bytes, int32_t peer);
/* wait_for_default_stream (:231-247): the private stream waits for work queued so far on `stream`. */
int esp_rnccl_fence_in(esp_rnccl_comm* comm, void* stream);
/* let_default_stream_wait (:250-257): `stream` waits for work queued so far on the private stream. */
int esp_rnccl_fence_out(esp_rnccl_comm* comm, void* stream);
/* The private stream (cudaStream_t), e.g. to record timing events on it. */
void* esp_rnccl_stream(esp_rnccl_comm* comm);
/* Text of the last NCCL/CUDA error on this thread. */
const char* esp_rnccl_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* ESP_RNCCL_H_ */
