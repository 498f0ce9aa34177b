/*
 * esp_attention.h -- C ABI of the B200 (sm_100a) elastic-sequence-parallel attention library.
 *
 * Every entry point takes raw device pointers, explicit sizes/strides (in ELEMENTS unless a name says
 * bytes) and a CUDA stream passed as void* (cudaStream_t).  No entry point allocates device memory
 * or synchronises the device unless its comment says so.  Return value: ESP_OK (0) or a negative
 * ESP_ERR_* code; esp_strerror() names it.  Kernels are launched asynchronously on `stream`.
 *
 * Each declaration cites the reference interface it replaces (path inside the reference project).
 */
#ifndef ESP_ATTENTION_H_
#define ESP_ATTENTION_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ESP_OK 0
#define ESP_ERR_BAD_ARG (-1)        /* null pointer, negative size, unsupported head_dim / dtype */
#define ESP_ERR_ALIGNMENT (-2)      /* pointer or stride not aligned as the kernel needs (16 bytes) */
#define ESP_ERR_CUDA (-3)           /* a CUDA runtime / driver call failed; see esp_last_cuda_error() */
#define ESP_ERR_DEVICE_TIMEOUT (-4) /* a bounded in-kernel wait gave up (reported by esp_device_status) */
#define ESP_ERR_UNSUPPORTED (-5)    /* valid request the library has no kernel for */
#define ESP_ERR_NCCL (-6)           /* an NCCL call failed */
#define ESP_ERR_TOO_LARGE (-7)      /* size beyond a fixed capacity stated by the entry point */
#define ESP_ERR_BAD_SLOT (-8)       /* a kernel met a slot id outside the pool and skipped that row (device status words) */

#define ESP_DTYPE_F16 0
#define ESP_DTYPE_BF16 1
#define ESP_DTYPE_F32 2

const char* esp_strerror(int code);
/* Text of the last CUDA error seen by this library on the calling thread ("" if none). */
const char* esp_last_cuda_error(void);
/* ABI version of this header (bumped on incompatible change).  Version 2: the peer-memory entry points take `value_base`.
 * Version 3: the kernels that dereference slot ids take the pool's row count; the self-test kernels left the library.
 * Version 4: esp_prefill_step_strided added (nothing removed or changed). */
#define ESP_ABI_VERSION 4
int esp_abi_version(void);

/* ------------------------------------------------------------------------------------------------
 * Ring prefill: one step of causal varlen attention with a running (o, m, l) state.
 * Replaces context_attention_fwd / _fwd_kernel,
 *   loongserve/models/llama/triton_kernel/ring_context_flashattention_nopad.py:191-284 (:13-188).
 *
 * q [q_tokens, Hq, D], k/v [kv_tokens, Hkv, D] (k and v may be the two halves of one
 * [kv_tokens, 2*Hkv, D] buffer: pass the two base pointers and the shared strides), o like q,
 * m/l fp32 [q_tokens, Hq] contiguous.  Last dimension contiguous everywhere; token and head strides
 * in elements, multiples of 8.  Six int32 [batch] vectors as in the reference.  Key n of request b is
 * visible to q row r iff  q_first[b] + r*s >= kv_first[b] + n*s  and  n < kv_len[b]
 * (s = logical_sp_peers_num).
 *
 * State convention (same as the reference): m = running maximum of score*scale*log2(e), l = matching
 * sum of 2^(.), o = NORMALISED output in `o_dtype` after every call.  Legal initial state:
 * m = -inf, l = 0, o = anything.  Rows that see no key in this call are left unchanged.
 * natural-log lse = ln2*m + ln(l).
 *
 * dtype: ESP_DTYPE_F16 or ESP_DTYPE_BF16 (q, k, v).  o_dtype: same as dtype, or ESP_DTYPE_F32 to
 * carry the output in fp32 between ring steps.  head_dim must be 128.  sm_scale <= 0 selects
 * head_dim^-0.5.  The host builds three TMA descriptors per call (no device work, no allocation).
 */
int esp_prefill_step(const void* q, int64_t q_stride_t, int64_t q_stride_h, int64_t q_tokens,
                     const void* k, const void* v, int64_t kv_stride_t, int64_t kv_stride_h,
                     int64_t kv_tokens,
                     void* o, int64_t o_stride_t, int64_t o_stride_h, float* m, float* l,
                     const int32_t* q_b_start_loc, const int32_t* q_b_seq_len,
                     const int32_t* q_first_token_global_idx, const int32_t* kv_b_start_loc,
                     const int32_t* kv_b_seq_len, const int32_t* kv_first_token_global_idx,
                     int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                     int32_t logical_sp_peers_num, int32_t max_q_b_seq_len, int32_t dtype,
                     int32_t o_dtype, float sm_scale, void* stream);

/* The same step with separate position strides for q rows and keys: key n of request b is visible to q row r iff
 *   q_first[b] + r*q_pos_stride >= kv_first[b] + n*kv_pos_stride  and  n < kv_len[b]
 * (q_pos_stride a positive multiple of kv_pos_stride; the firsts may be negative).  esp_prefill_step is this call with both
 * strides equal to logical_sp_peers_num.  With q_pos_stride = P-1 and kv_pos_stride = 1 one call attends the local q rows of
 * instance r of a striped ring of P to the KV rows of ALL other instances gathered into one buffer in position order
 * (row n*(P-1) + i holds token n of the i-th other instance): q_first = r - 1, kv_first = 0 -- what the reference's ring
 * loop does in P-1 steps (longserve_transformer_layer_infer.py:128-181). */
int esp_prefill_step_strided(const void* q, int64_t q_stride_t, int64_t q_stride_h, int64_t q_tokens,
                             const void* k, const void* v, int64_t kv_stride_t, int64_t kv_stride_h,
                             int64_t kv_tokens,
                             void* o, int64_t o_stride_t, int64_t o_stride_h, float* m, float* l,
                             const int32_t* q_b_start_loc, const int32_t* q_b_seq_len,
                             const int32_t* q_first_token_global_idx, const int32_t* kv_b_start_loc,
                             const int32_t* kv_b_seq_len, const int32_t* kv_first_token_global_idx,
                             int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                             int32_t q_pos_stride, int32_t kv_pos_stride, int32_t max_q_b_seq_len,
                             int32_t dtype, int32_t o_dtype, float sm_scale, void* stream);

/* Reset the running state before the first ring step: o = 0, m = -inf, l = 0
 * (longserve_transformer_layer_infer.py:123-126).  o may be NULL. */
int esp_prefill_state_init(void* o, int64_t o_bytes, float* m, float* l, int64_t rows_times_heads,
                           void* stream);

/* lse[i] = ln2*m[i] + ln(l[i])  (-inf where l == 0). */
int esp_prefill_lse(const float* m, const float* l, float* lse, int64_t n, void* stream);

/* Device-side status of the bounded waits inside the prefill kernel on the current device:
 * out[0] = 0 or ESP_ERR_DEVICE_TIMEOUT, out[1] = block index, out[2] = which wait, out[3] = detail.
 * Synchronises the device.  `clear` != 0 resets it. */
int esp_device_status(int32_t out[4], int32_t clear);

/* Limit, in SM cycles, of every bounded in-kernel wait of this library on the CURRENT device (the mbarrier waits of the
 * prefill kernel, the flag waits of the gated decode kernels and of esp_flag_wait).  Default 2e9 (about a second).
 * The reference has no counterpart: its kernels never wait on one another, and its NCCL calls wait without a limit. */
int esp_set_wait_limit_cycles(int64_t cycles);

/* ------------------------------------------------------------------------------------------------
 * Distributed flash-decoding.
 * esp_decode_stage1 replaces longserve_cuda_kernels.flash_decoding_stage1
 *   (longserve_cuda_kernels/src/entrypoints.cpp:103-164, flash_decoding_stage1.cu:25-215).
 * mid_o fp32 [num_blocks, batch, Hq, D], mid_lse fp32 [num_blocks, batch, Hq] (contiguous);
 * q [batch, Hq, D] contiguous; k, v [pool, Hkv, D] views (strides in elements, last dim contiguous);
 * req_to_tokens int32 [max_req, max_seq] (row stride max_seq); b_req_idx, b_seqlen int32 [batch].
 * Block j of request b covers tokens [j*seq_block_size, min((j+1)*seq_block_size, len_b)); blocks
 * past the length are not written.  Unlike the reference seq_block_size may be any positive value
 * (the reference caps it at 256); head_dim must be 128.
 * pool_rows: number of slot rows k and v have.  A slot id outside [0, pool_rows) -- the table's 2147483647 filler
 * included -- is not dereferenced: the token is left out, and esp_decode_device_status reports ESP_ERR_BAD_SLOT with
 * the id.  pool_rows <= 0 switches the check off (the reference has none: longserve_req_manager.py:19 is the filler).
 */
int esp_decode_stage1(float* mid_o, float* mid_lse, const void* q, const void* k, const void* v,
                      int64_t k_stride_t, int64_t k_stride_h, int64_t v_stride_t, int64_t v_stride_h,
                      const int32_t* req_to_tokens, int64_t req_to_tokens_stride,
                      const int32_t* b_req_idx, const int32_t* b_seqlen, int32_t batch,
                      int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                      int32_t max_len_in_batch, int32_t seq_block_size, int32_t dtype, float sm_scale,
                      int64_t pool_rows, void* stream);

/* esp_decode_merge replaces longserve_cuda_kernels.flash_decoding_stage2
 *   (entrypoints.cpp:166-221, flash_decoding_stage2.cu:15-150): lse-merge of
 * ceil(b_seqlen[b]/block_seq) partials per (request, head).  o_dtype F16/BF16/F32.
 * A request with zero partials gets o = 0, lse = -inf (the reference leaves both unwritten). */
int esp_decode_merge(void* o, float* out_lse, const int32_t* b_seqlen, const float* mid_o,
                     const float* mid_lse, int32_t batch, int32_t num_heads, int32_t head_dim,
                     int32_t num_blocks, int32_t block_seq, int32_t o_dtype, void* stream);

/* esp_decode_attention_noalloc has no counterpart in the reference.  It is stage 1 + merge in one
 * call for callers that may not allocate device memory on the serving path (a worker whose whole
 * memory budget went to the KV cache at start-up, or one replaying a fixed launch sequence): the
 * per-split partials live in a fixed 16 MiB array inside the library (held by every GPU that loads it,
 * until the process exits) instead of caller-provided mid_o / mid_lse.  The split size is chosen so the
 * partials fit; if batch * num_q_heads * (head_dim + 1) floats of a single split exceed the 4 Mi-float
 * capacity the call returns ESP_ERR_TOO_LARGE and launches nothing.  The call itself performs no
 * cudaMalloc / cudaFree.  Its first call on a device looks up the array's device address (once per
 * device, with that device current): make that first call before any stream capture.  Every call on a
 * device shares the array, so calls that overlap on the GPU race; calls on one stream are safe.  The array used is the
 * one of the device that is CURRENT when the call is made, so `stream` must belong to the current device.
 * Arguments as esp_decode_stage1 / esp_decode_merge; o_dtype F16/BF16/F32. */
int esp_decode_attention_noalloc(void* o, float* out_lse, const void* q, const void* k, const void* v,
                                 int64_t k_stride_t, int64_t k_stride_h, int64_t v_stride_t,
                                 int64_t v_stride_h, const int32_t* req_to_tokens,
                                 int64_t req_to_tokens_stride, const int32_t* b_req_idx,
                                 const int32_t* b_seqlen, int32_t batch, int32_t num_q_heads,
                                 int32_t num_kv_heads, int32_t head_dim, int32_t max_len_in_batch,
                                 int32_t dtype, int32_t o_dtype, float sm_scale, int64_t pool_rows, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Distributed decode over peer memory (NVLink loads/stores instead of NCCL messages).  The reference moves the
 * queries and the partial results with grouped ncclSend/ncclRecv (_selective_broadcast / _selective_gather /
 * _selective_scatter, longserve_transformer_layer_infer.py:468-504, used at :247-265 and :337-353); these
 * entry points do the same exchange inside the compute kernels: the master pushes q into every peer's
 * buffer and raises a flag there; a peer's stage 1 waits for that flag, its merge writes the fp32 (o, lse)
 * partial straight into the master's partial buffer, a one-word signal publishes it, and the master's merge
 * waits for the peers' flags.  Flags are int32 counters that only grow (one value per step).  Every wait is
 * bounded (about a second) and reports through esp_decode_device_status.
 * Every flag value is given as `value` plus an optional `value_base`: a device pointer (may be NULL = 0) to an
 * int32 the kernel adds when it runs.  A caller that records a whole step into a CUDA graph keeps the per-launch
 * values fixed (1, 2, ... within the step) and advances *value_base by the step's launch count between replays,
 * on every instance alike, so that replays keep using fresh values.
 */

/* A zero-filled device buffer that other processes on this node can map (CUDA IPC).  esp_peer_buffer_create
 * ALLOCATES (cudaMalloc) and returns the 64-byte handle to hand to the peers; esp_peer_buffer_open maps a peer's
 * buffer into this process.  Set-up time only. */
int esp_peer_buffer_create(int64_t bytes, void** dev_ptr, uint8_t handle_out[64]);
int esp_peer_buffer_open(const uint8_t handle[64], void** dev_ptr);
int esp_peer_buffer_close(void* dev_ptr);
int esp_peer_buffer_destroy(void* dev_ptr);

/* Copy `bytes` (multiple of 16) from src into each of the n_peers (<= 16) destination buffers (peer-mapped
 * pointers, host arrays of device pointers), then store flag_value (+ *value_base) to each peer's flag with release semantics. */
int esp_peer_push(const void* src, void* const* peer_dst, int32_t* const* peer_flags, int32_t n_peers,
                  int64_t bytes, int32_t flag_value, const int32_t* value_base, void* stream);
/* Publish everything this stream has written so far to the owner of remote_flag: *remote_flag = value (+ *value_base).
 * Nothing is published while the device's status word holds a timed-out wait: the kernels behind that wait returned
 * without writing their results, so the other side times out as well instead of consuming them. */
int esp_peer_signal(int32_t* remote_flag, int32_t value, const int32_t* value_base, void* stream);
/* A one-thread kernel that waits until *flag >= value (+ *value_base); work queued behind it on `stream` starts only
 * then.  The wait is bounded: it gives up after `patience` (1..1000) times the device's wait limit
 * (esp_set_wait_limit_cycles), and esp_decode_device_status then reports ESP_ERR_DEVICE_TIMEOUT with `wait_id` (>= 16,
 * the caller's label for this wait) and the awaited value.  Used by the copy-engine ring exchange; the reference's
 * ring waits inside ncclRecv, without a limit (longserve_transformer_layer_infer.py:162-178). */
int esp_flag_wait(const int32_t* flag, int32_t value, const int32_t* value_base, int32_t wait_id, int32_t patience,
                  void* stream);
/* cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault) on `stream`: a copy-engine transfer; dst or src may be a peer's
 * buffer mapped with esp_peer_buffer_open.  The reference moves KV blocks with ncclSend/ncclRecv
 * (rnccl/src/main.cpp:200-232), which copy with SM kernels. */
int esp_memcpy_async(void* dst, const void* src, int64_t bytes, void* stream);

/* esp_decode_stage1 whose blocks first wait until *wait_flag >= wait_value + *value_base (q then lives in a buffer the
 * master pushed into) and read q past the L1 cache. */
int esp_decode_stage1_gated(float* mid_o, float* mid_lse, const void* q, const void* k, const void* v,
                            int64_t k_stride_t, int64_t k_stride_h, int64_t v_stride_t,
                            int64_t v_stride_h, const int32_t* req_to_tokens,
                            int64_t req_to_tokens_stride, const int32_t* b_req_idx,
                            const int32_t* b_seqlen, int32_t batch, int32_t num_q_heads,
                            int32_t num_kv_heads, int32_t head_dim, int32_t max_len_in_batch,
                            int32_t seq_block_size, int32_t dtype, float sm_scale, int64_t pool_rows,
                            const int32_t* wait_flag, int32_t wait_value, const int32_t* value_base, void* stream);
/* esp_decode_merge whose blocks first wait until wait_flags[i] >= wait_value + *value_base for all i < n_wait. */
int esp_decode_merge_gated(void* o, float* out_lse, const int32_t* b_seqlen, const float* mid_o,
                           const float* mid_lse, int32_t batch, int32_t num_heads, int32_t head_dim,
                           int32_t num_blocks, int32_t block_seq, int32_t o_dtype,
                           const int32_t* wait_flags, int32_t n_wait, int32_t wait_value, const int32_t* value_base,
                           void* stream);
/* Status of the decode kernels and flag waits on the current device, like esp_device_status: out[0] = 0,
 * ESP_ERR_DEVICE_TIMEOUT (out[2] = which wait: 1 stage-1 gate, 2 merge gate, >= 16 esp_flag_wait ids; out[3] = awaited
 * value) or ESP_ERR_BAD_SLOT (out[3] = the slot id stage 1 refused).  After a timeout every later gated kernel on the
 * device returns at once until the status is cleared. */
int esp_decode_device_status(int32_t out[4], int32_t clear);

/* ------------------------------------------------------------------------------------------------
 * Token-indexed KV pool: scatter, registration, migration (all bit-exact copies / integer work).
 * Rows are [heads2, D] with D contiguous; `row_stride` = token stride, `head_stride` = head stride.
 * `elem_bytes` is 2 for fp16/bf16.  Index arrays may be int32 or int64 (`idx64` != 0).
 * `pool_rows` is the number of slot rows of the pool tensor a kernel indexes with slot ids: an id outside
 * [0, pool_rows) is never dereferenced, its row is skipped and esp_kv_device_status reports it
 * (pool_rows <= 0 switches the check off; the reference has no such check).
 */

/* out[0] = 0 or ESP_ERR_BAD_SLOT, out[1] = kernel (1 scatter, 2 scatter+register, 3 migration gather, 4 migration
 * scatter), out[2] = position of the id in its index array, out[3] = the id.  Synchronises the device. */
int esp_kv_device_status(int32_t out[4], int32_t clear);

/* out[dest[i]] = src[i], i < n.  Replaces destindex_copy_kv
 *   (loongserve/common/basemodel/triton_kernel/destindex_copy_kv.py:32-51). */
int esp_kv_scatter(const void* src, int64_t src_row_stride, int64_t src_head_stride, void* out,
                   int64_t out_row_stride, int64_t out_head_stride, const void* dest, int32_t idx64,
                   int64_t n, int32_t heads2, int32_t head_dim, int32_t elem_bytes, int64_t pool_rows, void* stream);

/* Keep-range of a passing striped block: begin = ceil((cache_begin - kv_first)/P), end likewise,
 * new_len = end - begin.  Replaces pre_copy_and_register_kv
 *   (loongserve/models/llama/triton_kernel/copy_and_register_kv.py:34-61). */
int esp_kv_keep_range(const int32_t* cache_begin, const int32_t* cache_end, const int32_t* kv_first,
                      int32_t num_peers, int32_t batch, int32_t* range_begin, int32_t* range_end,
                      int32_t* new_len, void* stream);

/* Copy the kept rows into pool slots mem_index[num_used + cumsum_prev[b] + n] and, when
 * `should_register` != 0, write the slot ids to req_to_token[b_req_idx[b], cur_kv_cache_index[b] + n].
 * Replaces destindex_copy_and_register_kv (copy_and_register_kv.py:123-169).
 * new_len_cumsum is the int64 inclusive cumsum of new_len. */
int esp_kv_scatter_register(int32_t batch, const int32_t* new_len, const int32_t* range_begin,
                            const int32_t* range_end, const int64_t* new_len_cumsum, const void* kv,
                            int64_t kv_row_stride, int64_t kv_head_stride,
                            const int32_t* kv_b_start_loc, const int32_t* cur_kv_cache_index,
                            const void* mem_index, int32_t idx64, void* pool, int64_t pool_row_stride,
                            int64_t pool_head_stride, int32_t* req_to_token,
                            int64_t req_to_token_stride, const int32_t* b_req_idx,
                            int64_t num_used_mem_index, int32_t max_len_in_batch,
                            int32_t should_register, int32_t heads2, int32_t head_dim,
                            int32_t elem_bytes, int64_t pool_rows, void* stream);

/* req_to_token[b_req_idx[i], b_seq_len[i]-1] = memindex[i].  Replaces copy_kv_index_to_req
 *   (loongserve/common/basemodel/triton_kernel/copy_kv_index_to_req.py:22-38). */
int esp_kv_index_register(int32_t* req_to_token, int64_t req_to_token_stride,
                          const int32_t* b_req_idx, const int32_t* b_seq_len, const void* memindex,
                          int32_t idx64, int32_t batch, void* stream);

/* Prefill registration without the host loop: req_to_token[b_req_idx[b], 0:len_b] =
 * alloc[start_b : start_b+len_b], start_b = exclusive cumsum of b_seq_len computed on the device.
 * Replaces init_req_to_token_indexes (loongserve/common/infer_utils.py:1-13).  batch <= 65536. */
int esp_kv_index_init(int32_t* req_to_token, int64_t req_to_token_stride, const int32_t* b_req_idx,
                      const int32_t* b_seq_len, const void* alloc, int32_t idx64, int32_t batch,
                      int32_t max_len_in_batch, void* stream);

/* Decode-stage migration, sender side: gather the last num_tokens[b] tokens of each request, all
 * layers, into send_buf [L, total, heads2, D] (contiguous) and zero mem_state of their slots.
 * Replaces decoding_stage_migration_sender_kernel
 *   (loongserve/models/llama/triton_kernel/decoding_stage_migration.py:71-95).
 * num_tokens_cumsum = int32/int64-agnostic: pass the int64 inclusive cumsum. kv_cache is
 * [L, slots, heads2, D] with `kv_layer_stride`, `kv_row_stride` in elements and contiguous rows. */
int esp_mig_gather(void* send_buf, int64_t total_tokens, const int32_t* req_to_token,
                   int64_t req_to_token_stride, int32_t* mem_state, const void* kv_cache,
                   int64_t kv_layer_stride, int64_t kv_row_stride, const int32_t* request_ids,
                   const int32_t* num_tokens, const int64_t* num_tokens_cumsum,
                   const int32_t* b_seq_len, int32_t batch, int32_t max_num_tokens,
                   int32_t num_layers, int32_t heads2, int32_t head_dim, int32_t elem_bytes,
                   int64_t pool_rows, void* stream);

/* Receiver side: scatter recv_buf into slots alloc_mem[cumsum_prev[b] + i] (all layers) and append
 * the slot ids at req_to_token[request_ids[b], b_seq_len[b] + i].  Replaces
 * decoding_stage_migration_receiver_kernel (decoding_stage_migration.py:160-184). */
int esp_mig_scatter(const void* recv_buf, int64_t total_tokens, int32_t* req_to_token,
                    int64_t req_to_token_stride, void* kv_cache, int64_t kv_layer_stride,
                    int64_t kv_row_stride, const void* alloc_mem, int32_t idx64,
                    const int32_t* request_ids, const int32_t* num_tokens,
                    const int64_t* num_tokens_cumsum, const int32_t* b_seq_len, int32_t batch,
                    int32_t max_num_tokens, int32_t num_layers, int32_t heads2, int32_t head_dim,
                    int32_t elem_bytes, int64_t pool_rows, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Host-side slot allocator with the allocation order of LongServeMemoryManager
 *   (loongserve/common/longserve_mem_manager.py:32-89): lowest free ids first, first free run for contiguous
 * requests, int32 reference counts -- kept entirely on the host (bitmap), so no device synchronisation.
 * esp_pool_alloc returns ESP_ERR_TOO_LARGE when fewer than n slots are free (the reference asserts);
 * esp_pool_alloc_contiguous stores -1 in *start when no run of n free slots exists (the reference returns None).
 */
typedef struct esp_pool esp_pool;
int esp_pool_create(int64_t size, esp_pool** out);
int esp_pool_destroy(esp_pool* pool);
int64_t esp_pool_can_use(const esp_pool* pool);
int esp_pool_alloc(esp_pool* pool, int64_t n, int64_t* out_ids);
int esp_pool_alloc_contiguous(esp_pool* pool, int64_t n, int64_t* start);
int esp_pool_add_refs(esp_pool* pool, const int64_t* ids, int64_t n);
int esp_pool_decrease_refs(esp_pool* pool, const int64_t* ids, int64_t n);
int esp_pool_free_all(esp_pool* pool);
int esp_pool_state(const esp_pool* pool, int32_t* out_refcounts);

/* Strided copy between pinned host memory and device memory (or device to device) on `stream`: `height` rows of
 * `width` bytes, row starts `spitch` / `dpitch` bytes apart.  kind: 0 host->device, 1 device->host, 2 device->device.
 * Used to move a chunk of heads of a [tokens, heads, D] host tensor without touching the other heads; the reference keeps
 * every tensor on the device and has no counterpart. */
int esp_memcpy_2d(void* dst, int64_t dpitch, const void* src, int64_t spitch, int64_t width, int64_t height,
                  int32_t kind, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Prefill scheduling search (host only, no device work).
 */

/* Fills the cost table [num_new_req+1, num_instances+1] (caller sets every cell to +inf) and the choice table
 * [num_new_req+1, num_instances+1, 2] (caller sets every cell to -1) of the batch / instance-run search.
 * Replaces longserve_c_scheduler.minimize_prefill_iteration_time (longserve_c_scheduler/src/main.cpp:12-87; call site
 * loongserve/longserve_server/router/manager.py:710-712) with the same argument order: inclusive prefix sums of
 * the request lengths (longest first), of their squares and of their reciprocals, of the free tokens per instance,
 * and predictor rows (A, B, C) indexed by ESP degree ([predictor_rows, 3], predictor_rows >= num_instances + 1).
 * All arrays C-contiguous.  Results are bit-identical to the reference's. */
int esp_sched_minimize_prefill_iteration_time(int64_t num_new_req, int64_t num_instances, double* min_iteration_times,
                                              int32_t* min_iteration_times_index, const int64_t* req_input_prefix_sum,
                                              const int64_t* req_input_square_prefix_sum,
                                              const double* inverted_req_input_prefix_sum,
                                              const int64_t* left_token_prefix_sum, const double* predictor_parameters,
                                              int64_t predictor_rows);

/* The whole planning step of `_schedule_new_req_list` (router/manager.py:687-760) in one call: prefix sums, the
 * search above, the choice of the instance count with the least cost, and the walk back through the choices.
 * req_tokens: lengths sorted longest first; left_tokens: free tokens of the instances in the caller's order.
 * Writes up to num_new_req batches, last batch first (the reference creates them in that order): batch k takes
 * batch_sizes[k] requests from the end of the not yet assigned requests and batch_instances[k] instances from the end
 * of the not yet assigned instances.  ESP_ERR_TOO_LARGE when the requests do not fit into the free tokens at all. */
int esp_sched_plan_prefill(int64_t num_new_req, const int64_t* req_tokens, int64_t num_instances, const int64_t* left_tokens,
                           const double* predictor_parameters, int64_t predictor_rows, int32_t* batch_sizes,
                           int32_t* batch_instances, int64_t* num_batches, double* total_cost, double* max_iteration_time);

/* ------------------------------------------------------------------------------------------------
 * Element-wise layer kernels around the attention path (needed only to run a whole Llama layer).
 */

/* out[t,:] = in[t,:] * rsqrt(mean(in[t,:]^2) + eps) * weight.  Replaces longserve_cuda_kernels.rms_norm
 *   (longserve_cuda_kernels/src/entrypoints.cpp:15-38, rms_norm.cu:10-60).  Contiguous [tokens, hidden],
 * hidden a multiple of 8; dtype F16/BF16; fp32 accumulation. */
int esp_rms_norm(void* out, const void* in, const void* weight, int64_t tokens, int32_t hidden,
                 float eps, int32_t dtype, void* stream);

/* In-place rotate-half RoPE on x [tokens, heads, head_dim] (strides in elements, last dim contiguous):
 * x1' = x1*cos - x2*sin, x2' = x1*sin + x2*cos with x1/x2 the first/second half of head_dim;
 * cos, sin [tokens, head_dim/2] contiguous in x's dtype.  Replaces one half of
 * longserve_cuda_kernels.rotary_emb (entrypoints.cpp:53-87, rotary_emb.cu:10-51), which rotates q and k
 * by two such calls.  Math in fp32, rounded once (the reference rounds after every half-precision op). */
int esp_rotary_emb(void* x, const void* cosv, const void* sinv, int64_t x_stride_t, int64_t x_stride_h,
                   int64_t tokens, int32_t heads, int32_t head_dim, int32_t dtype, void* stream);

/* io[:, :F] = silu(io[:, :F]) * io[:, F:2F] on a contiguous [tokens, 2F] buffer.  Replaces
 * longserve_cuda_kernels.silu_and_mul_inplace (entrypoints.cpp:40-51, silu_and_mul.cu:17-45). */
int esp_silu_and_mul_inplace(void* io, int64_t tokens, int32_t ffn_inter_dim, int32_t dtype,
                             void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ESP_ATTENTION_H_ */
