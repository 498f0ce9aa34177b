// Ring-prefill attention step for sm_100a: causal varlen flash attention of the local q rows against
// one (local or remote) KV block, merged into the running (o, m, l) state.
//
// One CTA owns 256 consecutive q rows of one (request, head) as two 128-row tiles.  Warp roles:
//   warps 0-3  softmax of tile 0 (one thread per row), warps 4-7 softmax of tile 1,
//   warp 8     TMA producer (Q tiles once, then K_0, then the pairs {V_j, K_j+1} through two 64 KiB pair stages),
//   warp 9     tcgen05.mma issuer (one thread) and owner of the tensor-memory allocation; warps 10-11 only lend registers.
// Per kv tile and q tile:  S = Q K^T (tcgen05.mma, both operands K-major in 128B-swizzled smem, fp32
// accumulator in tensor memory) -> softmax threads read their row with tcgen05.ld, apply the mask only
// on diagonal/tail tiles, keep a running base-2 maximum with lazy rescaling of O, write P as packed
// 16-bit back into the S columns -> O += P V (tcgen05.mma, A from tensor memory, V MN-major in smem).
// The two q tiles ping-pong: while the tensor core runs tile 0's PV and next S, tile 1's softmax runs.
// Tensor-memory map (512 columns): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P aliases S.
//
// Two kernels share this design: prefill_step_kernel (one CTA as described) and prefill_pair_kernel (a cluster of two CTAs
// owns 512 rows; one thread issues cta_group::2 MMAs with M = 256 for both SMs, each CTA loading half of every K and V
// tile; used whenever a request has more than 256 local rows).
//
// Visibility.  Key n of a request is visible to q row r iff q_first + r * q_pos_stride >= kv_first + n * kv_pos_stride
// (and n < kv_len).  Within a ring step both strides are the ring size (striped placement) or 1; with q_pos_stride = P - 1
// and kv_pos_stride = 1 one call covers the rows of all other instances gathered in position order.
//
// What bounds it.  Per q tile the chain S -> softmax -> PV is serial; the softmax needs one MUFU exponential per score
// (16 per clock and SM: 1024 cycles per tile, as many as the tile's two MMAs need on the tensor pipe), and the one thread
// that issues the MMAs (about 50 cycles per tcgen05.mma against 64 cycles of pipe time) shares the issue slots of its SM
// sub-partition with two softmax warps.  Hence: one wait and one commit per kv tile for the K/V data (pairs), a
// register budget for the third warpgroup that keeps the issue loop out of local memory, no votes or warp barriers in
// the loop, and a softmax stripped to scale, exponential, sum and pack per score: exponentials are taken against the
// running maximum, and the row sum they produce anyway proves that no score outgrew the lazy-rescale threshold.
//
// Roofline: tensor-core bound; algorithmic FLOPs = 4 * D * (visible q,k pairs) per head.
// Every mbarrier wait is bounded; on expiry the kernel records a status word and drains.
#include <cuda.h>
#include <stdlib.h>

#include "esp_common.cuh"
#include "sm100_ptx.cuh"

namespace esp {

using namespace ptx;

constexpr int BM = 128;               // rows per q tile
constexpr int QT = 2;                 // q tiles per CTA
constexpr int BN = 128;               // keys per kv tile
constexpr int HD = 128;               // head dim
constexpr int NSTAGE = 4;             // K/V tile slots in shared memory
constexpr int TILE_BYTES = BN * HD * 2;
constexpr int HALF_BYTES = TILE_BYTES / 2;   // 64 head-dim columns x 128 rows (one swizzle-128B panel)
constexpr int NUM_THREADS = 384;      // 3 warpgroups: softmax tile 0, softmax tile 1, {producer, MMA issuer, 2 lenders}
constexpr int TMEM_COLS = 512;
constexpr float kRescaleThreshold = 8.0f;              // lazy O rescale: tolerate 2^8 growth
constexpr float kSpecSumLimit = 256.0f;                // 2^kRescaleThreshold
// setmaxnreg plan: the two softmax warpgroups raise their budget, the third warpgroup lowers it;
// 256 * kRegsSoftmax + 128 * kRegsOther must fit the 384 * 168 registers the CTA is launched with.  Measured at 262144
// tokens: (224, 56) 1049 TFLOP/s -- the issuing thread then spills inside its loop, which is the kernel's critical
// path --, (216, 72) 1090, (208, 88) 1091 with the same code otherwise.
constexpr int kRegsSoftmax = 216, kRegsOther = 72;
static_assert(256 * kRegsSoftmax + 128 * kRegsOther <= 384 * 168 && kRegsSoftmax % 8 == 0 && kRegsOther % 8 == 0, "setmaxnreg plan");
constexpr int kPReadyArrivals = 4;    // one arrival per softmax warp publishes a tile's P

// K/V tiles travel in pairs: after K_0 (which has barriers of its own), pair p = {V_p, K_p+1} is loaded under ONE
// "full" barrier and released by ONE "empty" commit, so the issuing thread pays one wait and one commit per kv tile
// instead of two of each.  Two pair stages; tile r of the sequence K_0 V_0 K_1 V_1 ... sits in slot r mod 4.
enum BarIdx { B_QFULL = 0, B_K0FULL = 2, B_K0EMPTY = 3, B_PFULL = 4, B_PEMPTY = 6, B_SFULL = 8,
              B_PREADY = 10, B_ODONE = 12, B_COUNT = 14 };

constexpr int SMEM_Q = 0;
constexpr int SMEM_KV = QT * TILE_BYTES;
constexpr int SMEM_BAR = SMEM_KV + NSTAGE * TILE_BYTES;
constexpr int SMEM_MISC = SMEM_BAR + B_COUNT * 8;
constexpr int SMEM_TOTAL = SMEM_MISC + 16;
constexpr int SMEM_DYN = SMEM_TOTAL + 1024;            // slack to align the base to 1024 B

__device__ int g_esp_status[4];
// Bound of every mbarrier wait in SM cycles (about a second by default); esp_set_wait_limit_cycles changes it.
__device__ long long g_wait_limit_cycles = 2000000000LL;


struct PrefillParams {
    void* o; float* m; float* l;
    int64_t o_stride_t, o_stride_h;
    const int32_t* q_start; const int32_t* q_len; const int32_t* q_first;
    const int32_t* kv_start; const int32_t* kv_len; const int32_t* kv_first;
    int num_q_heads, group, q_pos_stride, kv_pos_stride, num_qblocks;   // position strides of consecutive q rows / keys
    float scale_log2;
};

__device__ __noinline__ void report_timeout(int which, int detail) {
    if (atomicCAS(&g_esp_status[0], 0, ESP_ERR_DEVICE_TIMEOUT) == 0) {
        g_esp_status[1] = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
        g_esp_status[2] = which;
        g_esp_status[3] = detail;
    }
}

__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, volatile int* s_abort, int which, int detail) {
    const int r = mbar_wait_bounded(bar, parity, &g_wait_limit_cycles, s_abort);
    if (r == 2) {
        report_timeout(which, detail);
        *s_abort = 1;
    }
    return r == 0;
}

template <typename T> struct Fmt;
template <> struct Fmt<__half> { static constexpr uint32_t kAB = 0; };
template <> struct Fmt<__nv_bfloat16> { static constexpr uint32_t kAB = 1; };

template <typename OT> __device__ __forceinline__ void load_row32(const OT* p, float (&x)[32]);
template <> __device__ __forceinline__ void load_row32<float>(const float* p, float (&x)[32]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 v = *reinterpret_cast<const float4*>(p + 4 * i);
        x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
    }
}
template <typename OT> __device__ __forceinline__ void load_row32_16(const OT* p, float (&x)[32]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 v = *reinterpret_cast<const uint4*>(p + 8 * i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = Cvt<OT>::to_f2(w[k]);
            x[8 * i + 2 * k] = f.x; x[8 * i + 2 * k + 1] = f.y;
        }
    }
}
template <> __device__ __forceinline__ void load_row32<__half>(const __half* p, float (&x)[32]) { load_row32_16<__half>(p, x); }
template <> __device__ __forceinline__ void load_row32<__nv_bfloat16>(const __nv_bfloat16* p, float (&x)[32]) { load_row32_16<__nv_bfloat16>(p, x); }

template <typename OT> __device__ __forceinline__ void store_row32(OT* p, const float (&x)[32]);
template <> __device__ __forceinline__ void store_row32<float>(float* p, const float (&x)[32]) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
        *reinterpret_cast<float4*>(p + 4 * i) = make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]);
}
template <typename OT> __device__ __forceinline__ void store_row32_16(OT* p, const float (&x)[32]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint4 v;
        v.x = Cvt<OT>::pack(x[8 * i], x[8 * i + 1]); v.y = Cvt<OT>::pack(x[8 * i + 2], x[8 * i + 3]);
        v.z = Cvt<OT>::pack(x[8 * i + 4], x[8 * i + 5]); v.w = Cvt<OT>::pack(x[8 * i + 6], x[8 * i + 7]);
        *reinterpret_cast<uint4*>(p + 8 * i) = v;
    }
}
template <> __device__ __forceinline__ void store_row32<__half>(__half* p, const float (&x)[32]) { store_row32_16<__half>(p, x); }
template <> __device__ __forceinline__ void store_row32<__nv_bfloat16>(__nv_bfloat16* p, const float (&x)[32]) { store_row32_16<__nv_bfloat16>(p, x); }


// ---- softmax arithmetic helpers -------------------------------------------------------------------
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// max over one 32-column chunk, optionally masked (columns > limit are invisible); four independent
// chains keep the dependent latency off the critical path
__device__ __forceinline__ float chunk_max(uint32_t (&r)[32], int col0, int limit, bool masked) {
    if (masked) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (col0 + i > limit) r[i] = 0xff800000u;
    }
    float a[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        a[c] = fmax3(__uint_as_float(r[8 * c]), __uint_as_float(r[8 * c + 1]), __uint_as_float(r[8 * c + 2]));
        a[c] = fmax3(a[c], __uint_as_float(r[8 * c + 3]), __uint_as_float(r[8 * c + 4]));
        a[c] = fmax3(a[c], __uint_as_float(r[8 * c + 5]), __uint_as_float(r[8 * c + 6]));
        a[c] = fmaxf(a[c], __uint_as_float(r[8 * c + 7]));
    }
    return fmaxf(fmax3(a[0], a[1], a[2]), a[3]);
}

// p = 2^(s*scale - m) for one 32-column chunk; packs to 16-bit pairs and returns the chunk's row sum
// (two independent packed accumulators).
template <typename T, int OFF>
__device__ __forceinline__ float chunk_exp(const uint32_t (&r)[32], float scale, float neg_m, uint32_t (&pk)[32]) {
    const float2 sc2 = make_float2(scale, scale), nm2 = make_float2(neg_m, neg_m);
    float2 acc[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), sc2, nm2);
        float2 e;
        e.x = ex2(x.x); e.y = ex2(x.y);
        acc[(i / 2) & 1] = __fadd2_rn(acc[(i / 2) & 1], e);
        pk[OFF + i / 2] = Cvt<T>::pack(e.x, e.y);
    }
    const float2 t = __fadd2_rn(acc[0], acc[1]);
    return t.x + t.y;
}

// ------------------------------------------------------------------------------------------------
template <typename T, typename OT>
__global__ void __launch_bounds__(NUM_THREADS, 1) prefill_step_kernel(
    const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
    const __grid_constant__ CUtensorMap tm_v, const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar0 = smem_base + SMEM_BAR;
    auto bar = [bar0](int i) { return bar0 + 8u * i; };
    volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem_gen + SMEM_MISC);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem_gen + SMEM_MISC + 4);
    volatile int* s_skip = reinterpret_cast<volatile int*>(smem_gen + SMEM_MISC + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb = p.num_qblocks - 1 - (int)blockIdx.x;      // heaviest q block first
    const int head = blockIdx.y, b = blockIdx.z;
    const int kvh = head / p.group;

    const int q_len = p.q_len[b];
    const int m0 = qb * (QT * BM);
    if (m0 >= q_len) return;
    const int kv_len = p.kv_len[b];
    const int q_start = p.q_start[b], kv_start = p.kv_start[b];
    // key n visible to local row r  <=>  n <= vis_a * r + vis_c  and  n < kv_len
    const int dnum = p.q_first[b] - p.kv_first[b];
    const int vis_a = p.q_pos_stride / p.kv_pos_stride;      // keys that become visible per q row (1 within a ring step)
    const int vis_c = dnum >= 0 ? dnum / p.kv_pos_stride : -((-dnum + p.kv_pos_stride - 1) / p.kv_pos_stride);   // floor
    int n_tiles[QT];
#pragma unroll
    for (int t = 0; t < QT; ++t) {
        const int r0 = m0 + t * BM;
        int cnt = 0;
        if (r0 < q_len) {
            const int last_row = min(r0 + BM - 1, q_len - 1);
            const int range = max(0, min(vis_a * last_row + vis_c + 1, kv_len));
            cnt = (range + BN - 1) / BN;
        }
        n_tiles[t] = cnt;
    }
    const int nmax = max(n_tiles[0], n_tiles[1]);
    if (nmax == 0) return;      // nothing visible: state unchanged

    if (threadIdx.x == 0) {
        *s_abort = 0;
        *s_skip = (*reinterpret_cast<volatile int*>(&g_esp_status[0]) != 0);
        for (int i = 0; i < B_COUNT; ++i) mbar_init(bar(i), (i >= B_PREADY && i < B_PREADY + QT) ? kPReadyArrivals : 1);
        fence_barrier_init();
    }
    if (warp == 8 && lane == 0) {
        prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v);
    }
    __syncthreads();
    if (*s_skip) return;        // an earlier CTA reported a timeout: drain the grid quickly
    if (warp == 9) {
        tmem_alloc(smem_base + SMEM_MISC, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;

    // With 384 threads the third warpgroup (producer, MMA issuer, two idle warps) hands most of its
    // registers to the two softmax warpgroups; each role changes its budget at the top of its own branch.
    if (warp >= 8) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
      if (warp == 8) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
#pragma unroll
            for (int t = 0; t < QT; ++t) {
                if (n_tiles[t] > 0) {
                    const uint32_t dst = smem_base + SMEM_Q + t * TILE_BYTES;
                    mbar_expect_tx(bar(B_QFULL + t), TILE_BYTES);
                    tma_load_3d(dst, &tm_q, bar(B_QFULL + t), 0, head, q_start + m0 + t * BM);
                    tma_load_3d(dst + HALF_BYTES, &tm_q, bar(B_QFULL + t), 64, head, q_start + m0 + t * BM);
                }
            }
            auto load_tile = [&](const CUtensorMap* tm, int slot, int tile, uint32_t full_bar) {
                const uint32_t dst = smem_base + SMEM_KV + slot * TILE_BYTES;
                tma_load_3d(dst, tm, full_bar, 0, kvh, kv_start + tile * BN);
                tma_load_3d(dst + HALF_BYTES, tm, full_bar, 64, kvh, kv_start + tile * BN);
            };
            mbar_expect_tx(bar(B_K0FULL), TILE_BYTES);
            load_tile(&tm_k, 0, 0, bar(B_K0FULL));
            for (int pr = 0; pr < nmax; ++pr) {
                const int st = pr & 1;
                // slots of pair stage 1 are {3, 0}: its first fill waits for K_0 to be consumed; later fills for the pair
                // that used the stage before
                if (pr == 1 && !bounded_wait(bar(B_K0EMPTY), 0, s_abort, 1, pr)) break;
                if (pr >= 2 && !bounded_wait(bar(B_PEMPTY + st), ((pr >> 1) - 1) & 1, s_abort, 1, pr)) break;
                const bool with_k = pr + 1 < nmax;
                mbar_expect_tx(bar(B_PFULL + st), with_k ? 2 * TILE_BYTES : TILE_BYTES);
                load_tile(&tm_v, (2 * pr + 1) & 3, pr, bar(B_PFULL + st));
                if (with_k) load_tile(&tm_k, (2 * pr + 2) & 3, pr + 1, bar(B_PFULL + st));
            }
        }
      } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc_s = make_idesc(Fmt<T>::kAB, 0, BM, BN);
        constexpr uint32_t idesc_pv = make_idesc(Fmt<T>::kAB, 1, BM, HD);
        auto issue_s = [&](int t, int stage) {
            const uint32_t qa = smem_base + SMEM_Q + t * TILE_BYTES;
            const uint32_t kb = smem_base + SMEM_KV + stage * TILE_BYTES;
#pragma unroll
            for (int k = 0; k < HD / 16; ++k) {
                const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
                umma_ss(tmem_base + t * BN, desc_kmajor_sw128(qa + off), desc_kmajor_sw128(kb + off), idesc_s, k > 0);
            }
        };
        auto issue_pv = [&](int t, int stage, bool acc) {
            const uint32_t vb = smem_base + SMEM_KV + stage * TILE_BYTES;
#pragma unroll
            for (int k = 0; k < BN / 16; ++k) {
                umma_ts(tmem_base + QT * BN + t * HD, tmem_base + t * BN + k * 8,
                        desc_mnmajor_sw128(vb + k * 2048, HALF_BYTES), idesc_pv, (acc || k > 0) ? 1u : 0u);
            }
        };
        // One thread runs the whole issue loop: no votes, no warp barriers, nothing but waits, MMAs and commits in its
        // instruction stream (the loop of this thread is the kernel's critical path).
        if (lane == 0) {
            bool ok = true;
#pragma unroll
            for (int t = 0; t < QT; ++t)
                if (n_tiles[t] > 0) ok = ok && bounded_wait(bar(B_QFULL + t), 0, s_abort, 2, t);
            ok = ok && bounded_wait(bar(B_K0FULL), 0, s_abort, 3, 0);
            if (ok) {
                tc_fence_after();
#pragma unroll
                for (int t = 0; t < QT; ++t)
                    if (n_tiles[t] > 0) { issue_s(t, 0); umma_commit(bar(B_SFULL + t)); }
                umma_commit(bar(B_K0EMPTY));
            }
            for (int j = 0; j < nmax && ok; ++j) {
                const int st = j & 1, sv = (2 * j + 1) & 3, sk = (2 * j + 2) & 3;
                ok = bounded_wait(bar(B_PFULL + st), (j >> 1) & 1, s_abort, 4, j);      // V_j and K_j+1 have landed
                if (!ok) break;
                if ((j + 1) * BN > kv_len) {
                    // tail tile: rows past the request's last key may hold anything (even NaN); P is 0
                    // there, so make V finite by zeroing those rows in shared memory.
                    const int first_bad = kv_len - j * BN;
                    uint8_t* vs = smem_gen + SMEM_KV + sv * TILE_BYTES;
                    for (int i = first_bad * 8; i < BN * 8; ++i) {                 // 8 x 16 B per 128 B row
                        *reinterpret_cast<uint4*>(vs + i * 16) = make_uint4(0, 0, 0, 0);
                        *reinterpret_cast<uint4*>(vs + HALF_BYTES + i * 16) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async_smem();
                }
#pragma unroll
                for (int t = 0; t < QT; ++t) {
                    if (j < n_tiles[t]) {
                        ok = bounded_wait(bar(B_PREADY + t), j & 1, s_abort, 6 + t, j);
                        if (!ok) break;
                        tc_fence_after();
                        issue_pv(t, sv, j > 0);
                        if (j == n_tiles[t] - 1) umma_commit(bar(B_ODONE + t));
                    }
                    if (j + 1 < n_tiles[t]) {
                        issue_s(t, sk);
                        umma_commit(bar(B_SFULL + t));
                    }
                }
                if (!ok) break;
                umma_commit(bar(B_PEMPTY + st));
            }
        }
        __syncwarp();
      }
    } else {
        // ------------------------------------------------------------------ softmax + epilogue
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
        const int t = warp >> 2;                       // q tile of this warpgroup
        const int nt = n_tiles[t];
        if (nt > 0) {
            const int row_in_tile = (warp & 3) * 32 + lane;
            const int row = m0 + t * BM + row_in_tile;     // local row index inside the request
            const uint32_t lane_base = ((uint32_t)((warp & 3) * 32)) << 16;
            const uint32_t tS = tmem_base + lane_base + t * BN;
            const uint32_t tO = tmem_base + lane_base + QT * BN + t * HD;
            const float scale = p.scale_log2;
            float m_run = -INFINITY, l_run = 0.f;
            bool ok = true;
            for (int j = 0; j < nt; ++j) {
                ok = bounded_wait(bar(B_SFULL + t), j & 1, s_abort, 8 + t, j);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                uint32_t sr[4][32];
                tmem_ld32(tS, sr[0]);
                tmem_wait_ld();
                tmem_ld32(tS + 32, sr[1]);          // every later chunk streams in while the one before it is worked on
                const int n0 = j * BN;
                const int r0 = m0 + t * BM;
                const bool masked = (n0 + BN - 1 > vis_a * r0 + vis_c) || (n0 + BN > kv_len);
                const int limit = min(vis_a * row + vis_c, kv_len - 1) - n0;     // columns <= limit are visible
                // After the first tile the running maximum rarely grows by more than the lazy-rescale threshold, so the
                // exponentials of an unmasked tile are taken against the running maximum straight away, without looking
                // for the tile's own maximum (every instruction of this loop counts: the softmax warps' instruction
                // stream, with the issuing thread's, is what bounds the kernel).  P is stored only once every row of
                // the warp is known to have stayed within the threshold -- its row sum proves it; otherwise S (still
                // intact in tensor memory) is read again and the tile is done the slow way: maximum first, O rescaled,
                // then the exponentials.
                float lsum = 0.f;
                bool published = false;
                if (!masked && j > 0) {
                    const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
                    uint32_t pa[32], pb[32];
                    const float s0 = chunk_exp<T, 0>(sr[0], scale, neg_m, pa);
                    tmem_wait_ld();
                    tmem_ld32(tS + 64, sr[2]);
                    const float s1 = chunk_exp<T, 16>(sr[1], scale, neg_m, pa);
                    tmem_wait_ld();
                    tmem_ld32(tS + 96, sr[3]);
                    const float s2 = chunk_exp<T, 0>(sr[2], scale, neg_m, pb);
                    tmem_wait_ld();
                    const float s3 = chunk_exp<T, 16>(sr[3], scale, neg_m, pb);
                    lsum = (s0 + s1) + (s2 + s3);
                    // no exponential can exceed the row's sum of them: a sum within 2^threshold proves that the tile's maximum
                    // stayed within the threshold (a larger sum, an infinity or a NaN sends the tile down the exact path)
                    const bool outgrown = !(lsum <= kSpecSumLimit) || (m_run == -INFINITY);
                    if (!__any_sync(0xffffffffu, outgrown)) {
                        tmem_st32(tS, pa);
                        tmem_st32(tS + 32, pb);
                        published = true;
                    } else {
                        tmem_ld32(tS, sr[0]);
                        tmem_ld32(tS + 32, sr[1]);
                        tmem_wait_ld();
                        tmem_ld32(tS + 64, sr[2]);
                        tmem_ld32(tS + 96, sr[3]);
                    }
                }
                if (!published) {
                    if (masked || j == 0) {
                        tmem_wait_ld();
                        tmem_ld32(tS + 64, sr[2]);
                        tmem_ld32(tS + 96, sr[3]);
                    }
                    float mx = fmaxf(chunk_max(sr[0], 0, limit, masked), chunk_max(sr[1], 32, limit, masked));
                    tmem_wait_ld();
                    mx = fmax3(mx, chunk_max(sr[2], 64, limit, masked), chunk_max(sr[3], 96, limit, masked));
                    const float m_new = fmaxf(m_run, mx * scale);
                    // lazy rescale: keep the old reference maximum unless the row maximum grew by > 2^8
                    const bool need = (m_new > m_run + kRescaleThreshold) || (m_run == -INFINITY && m_new > -INFINITY);
                    float alpha = 1.f;
                    if (need) {
                        alpha = ex2(m_run - m_new);       // 0 when the row had no key before
                        l_run *= alpha;
                        m_run = m_new;
                    }
                    if (j > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            uint32_t orow[32];
                            tmem_ld32(tO + c * 32, orow);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
                            tmem_st32(tO + c * 32, orow);
                        }
                    }
                    const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
                    {
                        uint32_t pk[32];
                        const float s0 = chunk_exp<T, 0>(sr[0], scale, neg_m, pk);
                        const float s1 = chunk_exp<T, 16>(sr[1], scale, neg_m, pk);
                        tmem_st32(tS, pk);                 // P aliases the first 64 columns of S
                        lsum = s0 + s1;
                    }
                    {
                        uint32_t pk[32];
                        const float s2 = chunk_exp<T, 0>(sr[2], scale, neg_m, pk);
                        const float s3 = chunk_exp<T, 16>(sr[3], scale, neg_m, pk);
                        tmem_st32(tS + 32, pk);
                        lsum += s2 + s3;
                    }
                }
                l_run += lsum;
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_PREADY + t));
            }
            if (ok) {
                ok = bounded_wait(bar(B_ODONE + t), 0, s_abort, 10 + t, nt);
                ok = __all_sync(0xffffffffu, ok);
            }
            if (ok) {
                tc_fence_after();
                const bool live = (row < q_len) && (l_run > 0.f);
                const int64_t grow = (int64_t)q_start + row;
                float a_old = 0.f, a_new = 0.f, inv_l = 0.f;
                if (live) {
                    const int64_t si = grow * p.num_q_heads + head;
                    const float m_old = p.m[si], l_old = p.l[si];
                    const float m_new = fmaxf(m_run, m_old);
                    a_old = l_old * ex2(m_old - m_new);       // 0 for a fresh (-inf, 0) state
                    a_new = ex2(m_run - m_new);
                    const float l_new = a_old + l_run * a_new;
                    inv_l = 1.f / l_new;
                    p.m[si] = m_new;
                    p.l[si] = l_new;
                }
                OT* orow_g = reinterpret_cast<OT*>(p.o) + grow * p.o_stride_t + (int64_t)head * p.o_stride_h;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t acc[32];
                    tmem_ld32(tO + c * 32, acc);
                    tmem_wait_ld();
                    if (live) {
                        float x[32];
                        if (a_old != 0.f) {
                            load_row32<OT>(orow_g + c * 32, x);
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                x[i] = (x[i] * a_old + __uint_as_float(acc[i]) * a_new) * inv_l;
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) x[i] = __uint_as_float(acc[i]) * (a_new * inv_l);
                        }
                        store_row32<OT>(orow_g + c * 32, x);
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------
// The same step for CTA PAIRS (cluster of two, tcgen05 cta_group::2): a pair owns 512 consecutive q rows, CTA c of the pair the
// rows [256 c, 256 c + 256) as its two 128-row tiles.  Tile t of both CTAs forms one 256-row "slot": ONE thread of the even CTA
// issues M = 256 MMAs that run on both SMs, each CTA supplying its own Q rows / its own P (tensor memory) and HALF of the K tile
// (64 keys) or of the V tile (64 head dims) from its own shared memory.  So every MMA instruction does twice the work -- the
// issuing thread's instruction stream, the bound of the single-CTA kernel, is halved per FLOP -- and each SM reads half of B.
// Every CTA fetches its own halves with plain TMA loads (no multicast); loads of both CTAs are counted on barriers in the even
// CTA, where the issuing thread waits; tcgen05.commit arrives on the barriers of both CTAs.  K_0 has a buffer of its own, the
// pairs {V_j, K_j+1} go through four 32 KiB stages per CTA.
constexpr int NPS = 4;                                  // pair stages
constexpr int HALF_TILE = TILE_BYTES / 2;               // 16 KiB: 64 keys x 128 dims of K, or 128 keys x 64 dims of V
enum PairBar { PB_QFULL = 0, PB_K0FULL = 2, PB_PFULL = 3, PB_PEMPTY = 3 + NPS, PB_SFULL = 3 + 2 * NPS, PB_PREADY = 5 + 2 * NPS,
               PB_ODONE = 7 + 2 * NPS, PB_VREQ = 9 + 2 * NPS, PB_VCLEAN = 10 + 2 * NPS, PB_COUNT = 11 + 2 * NPS };
constexpr int PSMEM_Q = 0;
constexpr int PSMEM_K0 = QT * TILE_BYTES;
constexpr int PSMEM_PAIR = PSMEM_K0 + HALF_TILE;        // stage s: V half at +s*32 KiB, K half 16 KiB behind it
constexpr int PSMEM_BAR = PSMEM_PAIR + NPS * TILE_BYTES;
constexpr int PSMEM_MISC = PSMEM_BAR + PB_COUNT * 8;
constexpr int PSMEM_DYN = PSMEM_MISC + 16 + 1024;

template <typename T, typename OT>
__global__ void __launch_bounds__(NUM_THREADS, 1) prefill_pair_kernel(
    const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
    const __grid_constant__ CUtensorMap tm_v, const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar0 = smem_base + PSMEM_BAR;
    auto bar = [bar0](int i) { return bar0 + 8u * i; };                    // this CTA's barrier
    auto lbar = [bar0](int i) { return map_to_cta(bar0 + 8u * i, 0u); };   // the even CTA's barrier (cluster address)
    volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem_gen + PSMEM_MISC);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem_gen + PSMEM_MISC + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = cluster_ctarank();
    const int pb = p.num_qblocks - 1 - (int)(blockIdx.x >> 1);            // heaviest pair first (num_qblocks counts pairs here)
    const int head = blockIdx.y, b = blockIdx.z;
    const int kvh = head / p.group;

    const int q_len = p.q_len[b];
    const int m0p = pb * (2 * QT * BM);
    if (m0p >= q_len) return;                                              // the same decision in both CTAs of the pair
    const int m0 = m0p + (int)cta * (QT * BM);
    const int kv_len = p.kv_len[b];
    const int q_start = p.q_start[b], kv_start = p.kv_start[b];
    const int dnum = p.q_first[b] - p.kv_first[b];
    const int vis_a = p.q_pos_stride / p.kv_pos_stride;      // keys that become visible per q row (1 within a ring step)
    const int vis_c = dnum >= 0 ? dnum / p.kv_pos_stride : -((-dnum + p.kv_pos_stride - 1) / p.kv_pos_stride);   // floor
    // kv tiles a slot needs = what its later rows (the odd CTA's) need; the even CTA's rows see nothing in the extra tiles
    int nslot[QT];
#pragma unroll
    for (int t = 0; t < QT; ++t) {
        int cnt = 0;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int r0 = m0p + c * (QT * BM) + t * BM;
            if (r0 < q_len) {
                const int last_row = min(r0 + BM - 1, q_len - 1);
                const int range = max(0, min(vis_a * last_row + vis_c + 1, kv_len));
                cnt = max(cnt, (range + BN - 1) / BN);
            }
        }
        nslot[t] = cnt;
    }
    const int nmax = max(nslot[0], nslot[1]);
    if (nmax == 0) return;                                                 // pair-uniform as well

    if (threadIdx.x == 0) {
        // after a reported timeout later CTAs drain: every wait gives up at once, but both CTAs of a pair still walk
        // through the cluster barriers below together
        *s_abort = (*reinterpret_cast<volatile int*>(&g_esp_status[0]) != 0) ? 1 : 0;
        for (int i = 0; i < PB_COUNT; ++i) {
            const uint32_t cnt = (i >= PB_PREADY && i < PB_PREADY + QT) ? 2 * kPReadyArrivals : (i == PB_VCLEAN ? 2 : 1);
            mbar_init(bar(i), cnt);
        }
        fence_barrier_init();
    }
    if (warp == 8 && lane == 0) {
        prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v);
    }
    __syncthreads();
    if (warp == 9) {
        tmem_alloc_pair(smem_base + PSMEM_MISC, TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                 // the peer's barriers are initialised before anything is counted on them
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;

    if (warp >= 8) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
      if (warp == 8) {
        // ------------------------------------------------------------------ TMA producer (one per CTA, own halves)
        if (lane == 0 && !*s_abort) {       // when draining after a reported timeout nothing is loaded: the CTA leaves at once
#pragma unroll
            for (int t = 0; t < QT; ++t) {
                if (nslot[t] > 0) {
                    const uint32_t dst = smem_base + PSMEM_Q + t * TILE_BYTES;
                    if (cta == 0) mbar_expect_tx(bar(PB_QFULL + t), 2 * TILE_BYTES);
                    tma_load_3d_pair(dst, &tm_q, lbar(PB_QFULL + t), 0, head, q_start + m0 + t * BM);
                    tma_load_3d_pair(dst + HALF_BYTES, &tm_q, lbar(PB_QFULL + t), 64, head, q_start + m0 + t * BM);
                }
            }
            auto load_k_half = [&](uint32_t dst, int tile, uint32_t full_bar) {       // keys [64 cta, 64 cta + 64) of the tile
                tma_load_3d_pair(dst, &tm_k, full_bar, 0, kvh, kv_start + tile * BN + 64 * (int)cta);
                tma_load_3d_pair(dst + HALF_TILE / 2, &tm_k, full_bar, 64, kvh, kv_start + tile * BN + 64 * (int)cta);
            };
            if (cta == 0) mbar_expect_tx(bar(PB_K0FULL), 2 * HALF_TILE);
            load_k_half(smem_base + PSMEM_K0, 0, lbar(PB_K0FULL));
            for (int pr = 0; pr < nmax; ++pr) {
                const int st = pr % NPS;
                if (pr >= NPS && !bounded_wait(bar(PB_PEMPTY + st), ((pr / NPS) - 1) & 1, s_abort, 1, pr)) break;
                const bool with_k = pr + 1 < nmax;
                if (cta == 0) mbar_expect_tx(bar(PB_PFULL + st), with_k ? 4 * HALF_TILE : 2 * HALF_TILE);
                const uint32_t vdst = smem_base + PSMEM_PAIR + st * TILE_BYTES;
                tma_load_3d_pair(vdst, &tm_v, lbar(PB_PFULL + st), 64 * (int)cta, kvh, kv_start + pr * BN);   // dims [64 cta, +64)
                if (with_k) load_k_half(vdst + HALF_TILE, pr + 1, lbar(PB_PFULL + st));
            }
        }
      } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issuer (even CTA only)
        if (cta == 0 && lane == 0) {
            constexpr uint32_t idesc_s = make_idesc(Fmt<T>::kAB, 0, 2 * BM, BN);
            constexpr uint32_t idesc_pv = make_idesc(Fmt<T>::kAB, 1, 2 * BM, HD);
            auto issue_s = [&](int t, uint32_t kb) {          // kb: this CTA's K half, two 8 KiB panels of 64 rows
                const uint32_t qa = smem_base + PSMEM_Q + t * TILE_BYTES;
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    umma_pair_ss(tmem_base + t * BN, desc_kmajor_sw128(qa + (k >> 2) * HALF_BYTES + (k & 3) * 32),
                                 desc_kmajor_sw128(kb + (k >> 2) * (HALF_TILE / 2) + (k & 3) * 32), idesc_s, k > 0);
            };
            auto issue_pv = [&](int t, uint32_t vb, bool acc) {    // vb: this CTA's V half, one panel of 128 keys x 64 dims
#pragma unroll
                for (int k = 0; k < BN / 16; ++k)
                    umma_pair_ts(tmem_base + QT * BN + t * HD, tmem_base + t * BN + k * 8,
                                 desc_mnmajor_sw128(vb + k * 2048, HALF_TILE), idesc_pv, (acc || k > 0) ? 1u : 0u);
            };
            bool ok = bounded_wait(bar(PB_K0FULL), 0, s_abort, 3, 0);
#pragma unroll
            for (int t = 0; t < QT; ++t)
                if (nslot[t] > 0) ok = ok && bounded_wait(bar(PB_QFULL + t), 0, s_abort, 2, t);
            if (ok) {
                tc_fence_after();
#pragma unroll
                for (int t = 0; t < QT; ++t)
                    if (nslot[t] > 0) { issue_s(t, smem_base + PSMEM_K0); umma_pair_commit(bar(PB_SFULL + t)); }
            }
            for (int j = 0; j < nmax && ok; ++j) {
                const int st = j % NPS;
                const uint32_t vb = smem_base + PSMEM_PAIR + st * TILE_BYTES;
                ok = bounded_wait(bar(PB_PFULL + st), (j / NPS) & 1, s_abort, 4, j);          // V_j and K_j+1, both CTAs' halves
                if (!ok) break;
                if ((j + 1) * BN > kv_len) {
                    // the request's last, partly filled kv tile (at most one per pair): each CTA's sanitizer warp zeroes the
                    // rows of its V half behind the last key (P = 0 does not cancel a NaN), then this thread goes on
                    mbar_arrive(bar(PB_VREQ));
                    mbar_arrive_cluster(map_to_cta(bar(PB_VREQ), 1u));
                    ok = bounded_wait(bar(PB_VCLEAN), 0, s_abort, 5, j);
                    if (!ok) break;
                }
#pragma unroll
                for (int t = 0; t < QT; ++t) {
                    if (j < nslot[t]) {
                        ok = bounded_wait(bar(PB_PREADY + t), j & 1, s_abort, 6 + t, j);
                        if (!ok) break;
                        tc_fence_after();
                        issue_pv(t, vb, j > 0);
                        if (j == nslot[t] - 1) umma_pair_commit(bar(PB_ODONE + t));
                    }
                    if (j + 1 < nslot[t]) {
                        issue_s(t, vb + HALF_TILE);
                        umma_pair_commit(bar(PB_SFULL + t));
                    }
                }
                if (!ok) break;
                umma_pair_commit(bar(PB_PEMPTY + st));
            }
        }
        __syncwarp();
      } else if (warp == 10) {
        // ------------------------------------------------------------------ sanitizer of this CTA's V half (see the issuer)
        const int tail_j = kv_len / BN;
        if ((kv_len % BN) != 0 && tail_j < nmax) {
            bool go = bounded_wait(bar(PB_VREQ), 0, s_abort, 13, tail_j);
            go = __all_sync(0xffffffffu, go);
            if (go) {
                const int first_bad = kv_len - tail_j * BN;
                uint8_t* vs = smem_gen + PSMEM_PAIR + (tail_j % NPS) * TILE_BYTES;
                for (int i = first_bad * 8 + lane; i < BN * 8; i += 32)           // 8 x 16 B per 128 B row
                    *reinterpret_cast<uint4*>(vs + i * 16) = make_uint4(0, 0, 0, 0);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(lbar(PB_VCLEAN));
            }
        }
      }
    } else {
        // ------------------------------------------------------------------ softmax + epilogue (as in the single-CTA kernel)
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
        const int t = warp >> 2;                       // q tile of this warpgroup
        const int nt = nslot[t];              // both CTAs walk the slot's kv tiles together
        if (nt > 0) {
            const int row_in_tile = (warp & 3) * 32 + lane;
            const int row = m0 + t * BM + row_in_tile;     // local row index inside the request
            const uint32_t lane_base = ((uint32_t)((warp & 3) * 32)) << 16;
            const uint32_t tS = tmem_base + lane_base + t * BN;
            const uint32_t tO = tmem_base + lane_base + QT * BN + t * HD;
            const float scale = p.scale_log2;
            float m_run = -INFINITY, l_run = 0.f;
            bool ok = true;
            for (int j = 0; j < nt; ++j) {
                ok = bounded_wait(bar(PB_SFULL + t), j & 1, s_abort, 8 + t, j);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                uint32_t sr[4][32];
                tmem_ld32(tS, sr[0]);
                tmem_wait_ld();
                tmem_ld32(tS + 32, sr[1]);          // every later chunk streams in while the one before it is worked on
                const int n0 = j * BN;
                const int r0 = m0 + t * BM;
                const bool masked = (n0 + BN - 1 > vis_a * r0 + vis_c) || (n0 + BN > kv_len);
                const int limit = min(vis_a * row + vis_c, kv_len - 1) - n0;     // columns <= limit are visible
                // After the first tile the running maximum rarely grows by more than the lazy-rescale threshold, so the
                // exponentials of an unmasked tile are taken against the running maximum straight away, without looking
                // for the tile's own maximum (every instruction of this loop counts: the softmax warps' instruction
                // stream, with the issuing thread's, is what bounds the kernel).  P is stored only once every row of
                // the warp is known to have stayed within the threshold -- its row sum proves it; otherwise S (still
                // intact in tensor memory) is read again and the tile is done the slow way: maximum first, O rescaled,
                // then the exponentials.
                float lsum = 0.f;
                bool published = false;
                if (!masked && j > 0) {
                    const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
                    uint32_t pa[32], pb[32];
                    const float s0 = chunk_exp<T, 0>(sr[0], scale, neg_m, pa);
                    tmem_wait_ld();
                    tmem_ld32(tS + 64, sr[2]);
                    const float s1 = chunk_exp<T, 16>(sr[1], scale, neg_m, pa);
                    tmem_wait_ld();
                    tmem_ld32(tS + 96, sr[3]);
                    const float s2 = chunk_exp<T, 0>(sr[2], scale, neg_m, pb);
                    tmem_wait_ld();
                    const float s3 = chunk_exp<T, 16>(sr[3], scale, neg_m, pb);
                    lsum = (s0 + s1) + (s2 + s3);
                    // no exponential can exceed the row's sum of them: a sum within 2^threshold proves that the tile's maximum
                    // stayed within the threshold (a larger sum, an infinity or a NaN sends the tile down the exact path)
                    const bool outgrown = !(lsum <= kSpecSumLimit) || (m_run == -INFINITY);
                    if (!__any_sync(0xffffffffu, outgrown)) {
                        tmem_st32(tS, pa);
                        tmem_st32(tS + 32, pb);
                        published = true;
                    } else {
                        tmem_ld32(tS, sr[0]);
                        tmem_ld32(tS + 32, sr[1]);
                        tmem_wait_ld();
                        tmem_ld32(tS + 64, sr[2]);
                        tmem_ld32(tS + 96, sr[3]);
                    }
                }
                if (!published) {
                    if (masked || j == 0) {
                        tmem_wait_ld();
                        tmem_ld32(tS + 64, sr[2]);
                        tmem_ld32(tS + 96, sr[3]);
                    }
                    float mx = fmaxf(chunk_max(sr[0], 0, limit, masked), chunk_max(sr[1], 32, limit, masked));
                    tmem_wait_ld();
                    mx = fmax3(mx, chunk_max(sr[2], 64, limit, masked), chunk_max(sr[3], 96, limit, masked));
                    const float m_new = fmaxf(m_run, mx * scale);
                    // lazy rescale: keep the old reference maximum unless the row maximum grew by > 2^8
                    const bool need = (m_new > m_run + kRescaleThreshold) || (m_run == -INFINITY && m_new > -INFINITY);
                    float alpha = 1.f;
                    if (need) {
                        alpha = ex2(m_run - m_new);       // 0 when the row had no key before
                        l_run *= alpha;
                        m_run = m_new;
                    }
                    if (j > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            uint32_t orow[32];
                            tmem_ld32(tO + c * 32, orow);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
                            tmem_st32(tO + c * 32, orow);
                        }
                    }
                    const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
                    {
                        uint32_t pk[32];
                        const float s0 = chunk_exp<T, 0>(sr[0], scale, neg_m, pk);
                        const float s1 = chunk_exp<T, 16>(sr[1], scale, neg_m, pk);
                        tmem_st32(tS, pk);                 // P aliases the first 64 columns of S
                        lsum = s0 + s1;
                    }
                    {
                        uint32_t pk[32];
                        const float s2 = chunk_exp<T, 0>(sr[2], scale, neg_m, pk);
                        const float s3 = chunk_exp<T, 16>(sr[3], scale, neg_m, pk);
                        tmem_st32(tS + 32, pk);
                        lsum += s2 + s3;
                    }
                }
                l_run += lsum;
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(lbar(PB_PREADY + t));      // the issuing thread lives in the even CTA
            }
            if (ok) {
                ok = bounded_wait(bar(PB_ODONE + t), 0, s_abort, 10 + t, nt);
                ok = __all_sync(0xffffffffu, ok);
            }
            if (ok) {
                tc_fence_after();
                const bool live = (row < q_len) && (l_run > 0.f);
                const int64_t grow = (int64_t)q_start + row;
                float a_old = 0.f, a_new = 0.f, inv_l = 0.f;
                if (live) {
                    const int64_t si = grow * p.num_q_heads + head;
                    const float m_old = p.m[si], l_old = p.l[si];
                    const float m_new = fmaxf(m_run, m_old);
                    a_old = l_old * ex2(m_old - m_new);       // 0 for a fresh (-inf, 0) state
                    a_new = ex2(m_run - m_new);
                    const float l_new = a_old + l_run * a_new;
                    inv_l = 1.f / l_new;
                    p.m[si] = m_new;
                    p.l[si] = l_new;
                }
                OT* orow_g = reinterpret_cast<OT*>(p.o) + grow * p.o_stride_t + (int64_t)head * p.o_stride_h;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t acc[32];
                    tmem_ld32(tO + c * 32, acc);
                    tmem_wait_ld();
                    if (live) {
                        float x[32];
                        if (a_old != 0.f) {
                            load_row32<OT>(orow_g + c * 32, x);
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                x[i] = (x[i] * a_old + __uint_as_float(acc[i]) * a_new) * inv_l;
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) x[i] = __uint_as_float(acc[i]) * (a_new * inv_l);
                        }
                        store_row32<OT>(orow_g + c * 32, x);
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                 // neither CTA frees tensor memory or leaves while the peer's MMAs may still use it
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------
// Host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// [tokens, heads, 128] 16-bit tensor, box = 64 dims x 1 head x `box_tokens` tokens, 128-byte swizzle.
static int make_tile_map(CUtensorMap* tm, const void* base, int64_t tokens, int heads, int64_t stride_t,
                         int64_t stride_h, int dtype, int box_tokens = BN) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) { snprintf(last_cuda_error_buf(), 256, "cuTensorMapEncodeTiled entry point not found"); return ESP_ERR_CUDA; }
    cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)heads, (cuuint64_t)tokens};
    cuuint64_t strides[2] = {(cuuint64_t)stride_h * 2, (cuuint64_t)stride_t * 2};
    cuuint32_t box[3] = {64, 1, (cuuint32_t)box_tokens};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(tm, dtype == ESP_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                    3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(last_cuda_error_buf(), 256, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return ESP_ERR_CUDA;
    }
    return ESP_OK;
}

template <typename T, typename OT>
static int launch_prefill(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                          const PrefillParams& pp, dim3 grid, cudaStream_t s) {
    // set on every launch: the attribute is per device and a process may drive several
    ESP_CUDA_TRY(cudaFuncSetAttribute(prefill_step_kernel<T, OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DYN));
    {
        // the in-kernel register re-distribution (256 softmax threads x 224 + 128 other threads x 56) must fit the
        // registers the CTA is launched with, or setmaxnreg.inc would block
        cudaFuncAttributes fa;
        ESP_CUDA_TRY(cudaFuncGetAttributes(&fa, prefill_step_kernel<T, OT>));
        if (fa.numRegs * NUM_THREADS < 256 * kRegsSoftmax + 128 * kRegsOther) {
            snprintf(last_cuda_error_buf(), 256, "prefill kernel was built with %d registers per thread, too few for its setmaxnreg plan", fa.numRegs);
            return ESP_ERR_UNSUPPORTED;
        }
    }
    prefill_step_kernel<T, OT><<<grid, NUM_THREADS, SMEM_DYN, s>>>(tq, tk, tv, pp);
    ESP_LAUNCH_CHECK("prefill_step_kernel");
    return ESP_OK;
}

template <typename T, typename OT>
static int launch_prefill_pair(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                               const PrefillParams& pp, dim3 grid, cudaStream_t s) {
    ESP_CUDA_TRY(cudaFuncSetAttribute(prefill_pair_kernel<T, OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, PSMEM_DYN));
    cudaFuncAttributes fa;
    ESP_CUDA_TRY(cudaFuncGetAttributes(&fa, prefill_pair_kernel<T, OT>));
    if (fa.numRegs * NUM_THREADS < 256 * kRegsSoftmax + 128 * kRegsOther) {
        snprintf(last_cuda_error_buf(), 256, "prefill pair kernel was built with %d registers per thread, too few for its setmaxnreg plan", fa.numRegs);
        return ESP_ERR_UNSUPPORTED;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(NUM_THREADS); cfg.dynamicSmemBytes = PSMEM_DYN; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    ESP_CUDA_TRY(cudaLaunchKernelEx(&cfg, prefill_pair_kernel<T, OT>, tq, tk, tv, pp));
    return ESP_OK;
}

// Requests longer than one 256-row block run on CTA pairs; ESP_PREFILL_PAIRS=0 in the environment keeps the single-CTA kernel.
static bool use_pairs(int max_q_len) {
    static int env = -1;
    if (env < 0) { const char* e = getenv("ESP_PREFILL_PAIRS"); env = (e && e[0] == '0') ? 0 : 1; }
    return env == 1 && max_q_len > QT * BM;
}

__global__ void state_init_kernel(float* m, float* l, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        m[i] = -INFINITY; l[i] = 0.f;
    }
}
__global__ void lse_kernel(const float* m, const float* l, float* lse, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        lse[i] = l[i] > 0.f ? m[i] * 0.6931471805599453f + logf(l[i]) : -INFINITY;
}

int set_prefill_wait_limit(long long cycles) {
    ESP_CUDA_TRY(cudaMemcpyToSymbol(g_wait_limit_cycles, &cycles, sizeof(cycles)));
    return ESP_OK;
}

}  // namespace esp

using namespace esp;

extern "C" int esp_prefill_step(const void* q, int64_t q_stride_t, int64_t q_stride_h, int64_t q_tokens,
                                const void* k, const void* v, int64_t kv_stride_t, int64_t kv_stride_h,
                                int64_t kv_tokens, void* o, int64_t o_stride_t, int64_t o_stride_h,
                                float* m, float* l, const int32_t* q_b_start_loc,
                                const int32_t* q_b_seq_len, const int32_t* q_first_token_global_idx,
                                const int32_t* kv_b_start_loc, const int32_t* kv_b_seq_len,
                                const int32_t* kv_first_token_global_idx, int32_t batch,
                                int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                                int32_t logical_sp_peers_num, int32_t max_q_b_seq_len, int32_t dtype,
                                int32_t o_dtype, float sm_scale, void* stream) {
    return esp_prefill_step_strided(q, q_stride_t, q_stride_h, q_tokens, k, v, kv_stride_t, kv_stride_h, kv_tokens, o, o_stride_t,
                                    o_stride_h, m, l, q_b_start_loc, q_b_seq_len, q_first_token_global_idx, kv_b_start_loc,
                                    kv_b_seq_len, kv_first_token_global_idx, batch, num_q_heads, num_kv_heads, head_dim,
                                    logical_sp_peers_num, logical_sp_peers_num, max_q_b_seq_len, dtype, o_dtype, sm_scale, stream);
}

extern "C" int esp_prefill_step_strided(const void* q, int64_t q_stride_t, int64_t q_stride_h, int64_t q_tokens,
                                        const void* k, const void* v, int64_t kv_stride_t, int64_t kv_stride_h,
                                        int64_t kv_tokens, void* o, int64_t o_stride_t, int64_t o_stride_h,
                                        float* m, float* l, const int32_t* q_b_start_loc,
                                        const int32_t* q_b_seq_len, const int32_t* q_first_token_global_idx,
                                        const int32_t* kv_b_start_loc, const int32_t* kv_b_seq_len,
                                        const int32_t* kv_first_token_global_idx, int32_t batch,
                                        int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                                        int32_t q_pos_stride, int32_t kv_pos_stride, int32_t max_q_b_seq_len,
                                        int32_t dtype, int32_t o_dtype, float sm_scale, void* stream) {
    if (batch == 0 || max_q_b_seq_len <= 0 || q_tokens == 0 || kv_tokens == 0) return ESP_OK;
    if (!q || !k || !v || !o || !m || !l || !q_b_start_loc || !q_b_seq_len || !q_first_token_global_idx ||
        !kv_b_start_loc || !kv_b_seq_len || !kv_first_token_global_idx || batch < 0 || num_q_heads <= 0 ||
        num_kv_heads <= 0 || num_q_heads % num_kv_heads || q_pos_stride <= 0 || kv_pos_stride <= 0 ||
        q_pos_stride % kv_pos_stride || q_tokens < 0 || kv_tokens < 0)
        return ESP_ERR_BAD_ARG;
    if (dtype != ESP_DTYPE_F16 && dtype != ESP_DTYPE_BF16) return ESP_ERR_BAD_ARG;
    if (o_dtype != dtype && o_dtype != ESP_DTYPE_F32) return ESP_ERR_BAD_ARG;
    if (head_dim != HD) return ESP_ERR_UNSUPPORTED;
    if (batch > 65535 || num_q_heads > 65535) return ESP_ERR_TOO_LARGE;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || (q_stride_t % 8) ||
        (q_stride_h % 8) || (kv_stride_t % 8) || (kv_stride_h % 8) || (o_stride_t % 8) || (o_stride_h % 8))
        return ESP_ERR_ALIGNMENT;
    CUtensorMap tq, tk, tv;
    int rc;
    const bool pairs = use_pairs(max_q_b_seq_len);
    if ((rc = make_tile_map(&tq, q, q_tokens, num_q_heads, q_stride_t, q_stride_h, dtype))) return rc;
    if ((rc = make_tile_map(&tk, k, kv_tokens, num_kv_heads, kv_stride_t, kv_stride_h, dtype, pairs ? BN / 2 : BN))) return rc;
    if ((rc = make_tile_map(&tv, v, kv_tokens, num_kv_heads, kv_stride_t, kv_stride_h, dtype))) return rc;
    PrefillParams pp;
    pp.o = o; pp.m = m; pp.l = l; pp.o_stride_t = o_stride_t; pp.o_stride_h = o_stride_h;
    pp.q_start = q_b_start_loc; pp.q_len = q_b_seq_len; pp.q_first = q_first_token_global_idx;
    pp.kv_start = kv_b_start_loc; pp.kv_len = kv_b_seq_len; pp.kv_first = kv_first_token_global_idx;
    pp.num_q_heads = num_q_heads; pp.group = num_q_heads / num_kv_heads;
    pp.q_pos_stride = q_pos_stride; pp.kv_pos_stride = kv_pos_stride;
    pp.num_qblocks = (max_q_b_seq_len + QT * BM - 1) / (QT * BM);
    pp.scale_log2 = (sm_scale > 0.f ? sm_scale : 1.0f / sqrtf((float)head_dim)) * 1.4426950408889634f;
    dim3 grid(pp.num_qblocks, num_q_heads, batch);
    cudaStream_t s = (cudaStream_t)stream;
    if (pairs) {
        pp.num_qblocks = (max_q_b_seq_len + 2 * QT * BM - 1) / (2 * QT * BM);       // pairs of 256-row blocks
        grid.x = 2 * pp.num_qblocks;
        if (dtype == ESP_DTYPE_F16)
            return o_dtype == ESP_DTYPE_F32 ? launch_prefill_pair<__half, float>(tq, tk, tv, pp, grid, s)
                                            : launch_prefill_pair<__half, __half>(tq, tk, tv, pp, grid, s);
        return o_dtype == ESP_DTYPE_F32 ? launch_prefill_pair<__nv_bfloat16, float>(tq, tk, tv, pp, grid, s)
                                        : launch_prefill_pair<__nv_bfloat16, __nv_bfloat16>(tq, tk, tv, pp, grid, s);
    }
    if (dtype == ESP_DTYPE_F16)
        return o_dtype == ESP_DTYPE_F32 ? launch_prefill<__half, float>(tq, tk, tv, pp, grid, s)
                                        : launch_prefill<__half, __half>(tq, tk, tv, pp, grid, s);
    return o_dtype == ESP_DTYPE_F32 ? launch_prefill<__nv_bfloat16, float>(tq, tk, tv, pp, grid, s)
                                    : launch_prefill<__nv_bfloat16, __nv_bfloat16>(tq, tk, tv, pp, grid, s);
}

extern "C" int esp_prefill_state_init(void* o, int64_t o_bytes, float* m, float* l,
                                      int64_t rows_times_heads, void* stream) {
    if (!m || !l || rows_times_heads < 0 || o_bytes < 0) return ESP_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (o && o_bytes) ESP_CUDA_TRY(cudaMemsetAsync(o, 0, (size_t)o_bytes, s));
    if (rows_times_heads) {
        state_init_kernel<<<kNumSMs * 4, 256, 0, s>>>(m, l, rows_times_heads);
        ESP_LAUNCH_CHECK("state_init_kernel");
    }
    return ESP_OK;
}

extern "C" int esp_prefill_lse(const float* m, const float* l, float* lse, int64_t n, void* stream) {
    if (n == 0) return ESP_OK;
    if (!m || !l || !lse || n < 0) return ESP_ERR_BAD_ARG;
    lse_kernel<<<kNumSMs * 4, 256, 0, (cudaStream_t)stream>>>(m, l, lse, n);
    ESP_LAUNCH_CHECK("lse_kernel");
    return ESP_OK;
}


extern "C" int esp_device_status(int32_t out[4], int32_t clear) {
    if (!out) return ESP_ERR_BAD_ARG;
    ESP_CUDA_TRY(cudaDeviceSynchronize());
    ESP_CUDA_TRY(cudaMemcpyFromSymbol(out, g_esp_status, sizeof(int) * 4));
    if (clear) {
        int zero[4] = {0, 0, 0, 0};
        ESP_CUDA_TRY(cudaMemcpyToSymbol(g_esp_status, zero, sizeof(zero)));
    }
    return ESP_OK;
}
