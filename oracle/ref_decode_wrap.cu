// TEST INFRASTRUCTURE.  extern "C" shims around the reference's own flash-decoding CUDA kernels
// (longserve_cuda_kernels/src/flash_decoding_stage1.cu, flash_decoding_stage2.cu), which oracle/Makefile
// compiles from the reference checkout where it lies.  Used only by the GPU parity tests to pin the
// decode path (fp16) against the reference implementation itself.  Nothing of the reference is copied.
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <cuda_fp16.h>

#include "flash_decoding_stage1.h"
#include "flash_decoding_stage2.h"
#include "rms_norm.h"
#include "rotary_emb.h"
#include "silu_and_mul.h"

extern "C" void ref_flash_decoding_stage1(float* mid_out, float* mid_lse, const void* q, const void* k, const void* v,
                                          int64_t k_stride_0, int64_t k_stride_1, int64_t v_stride_0, int64_t v_stride_1,
                                          float sm_scale, const int32_t* req_to_tokens, const int32_t* b_req_idx,
                                          const int32_t* b_seqlen, int64_t batch, int64_t num_q_heads, int64_t num_kv_heads,
                                          int64_t num_blocks, int64_t head_dim, int64_t max_seq_len, int64_t seq_block_size,
                                          int64_t max_len_in_batch) {
    LongServe::flash_decoding_stage1(mid_out, mid_lse, (const half*)q, (const half*)k, (const half*)v, k_stride_0, k_stride_1,
                                     v_stride_0, v_stride_1, sm_scale, req_to_tokens, b_req_idx, b_seqlen, batch, num_q_heads,
                                     num_kv_heads, num_blocks, head_dim, max_seq_len, seq_block_size, max_len_in_batch);
}

extern "C" void ref_flash_decoding_stage2_f32(float* o, float* out_lse, const int32_t* b_seqlen, const float* mid_o,
                                              const float* mid_lse, int64_t batch, int64_t num_heads, int64_t num_blocks,
                                              int64_t head_dim, int64_t block_seq) {
    LongServe::flash_decoding_stage2<float>(o, out_lse, b_seqlen, mid_o, mid_lse, batch, num_heads, num_blocks, head_dim, block_seq);
}

extern "C" void ref_flash_decoding_stage2_f16(void* o, float* out_lse, const int32_t* b_seqlen, const float* mid_o,
                                              const float* mid_lse, int64_t batch, int64_t num_heads, int64_t num_blocks,
                                              int64_t head_dim, int64_t block_seq) {
    LongServe::flash_decoding_stage2<half>((half*)o, out_lse, b_seqlen, mid_o, mid_lse, batch, num_heads, num_blocks, head_dim, block_seq);
}

// Element-wise layer kernels of the reference (fp16), for the same purpose.
extern "C" void ref_rms_norm(void* out, const void* in, const void* weight, int64_t tokens, int64_t hidden, float eps) {
    LongServe::rms_norm((half*)out, (const half*)in, (const half*)weight, tokens, hidden, eps);
}
extern "C" void ref_rotary_emb(void* x, const void* cosv, const void* sinv, int64_t s0, int64_t s1, int64_t s2, int64_t tokens,
                               int64_t heads, int64_t head_dim) {
    LongServe::rotary_emb((half*)x, (const half*)cosv, (const half*)sinv, s0, s1, s2, tokens, heads, head_dim);
}
extern "C" void ref_silu_and_mul_inplace(void* io, int64_t tokens, int64_t ffn_inter_dim) {
    LongServe::silu_and_mul_inplace((half*)io, tokens, ffn_inter_dim);
}
