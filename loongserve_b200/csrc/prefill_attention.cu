// Ring-prefill attention step for sm_100a: causal varlen flash attention of the local q rows against
// one (local or remote) KV block, merged into the running (o, m, l) state.
//
// One CTA owns 256 consecutive q rows of one (request, head) as two 128-row tiles.  Warp roles:
//   warps 0-3  softmax of tile 0 (one thread per row), warps 4-7 softmax of tile 1,
//   warp 8     TMA producer (Q tiles once, then K_0 V_0 K_1 V_1 ... through a ring of 32 KiB stages),
//   warp 9     tcgen05.mma issuer and owner of the tensor-memory allocation; warps 10-11 only lend registers.
// Per kv tile and q tile:  S = Q K^T (tcgen05.mma, both operands K-major in 128B-swizzled smem, fp32
// accumulator in tensor memory) -> softmax threads read their row with tcgen05.ld, apply the mask only
// on diagonal/tail tiles, keep a running base-2 maximum with lazy rescaling of O, write P as packed
// 16-bit back into the S columns -> O += P V (tcgen05.mma, A from tensor memory, V MN-major in smem).
// The two q tiles ping-pong: while the tensor core runs tile 0's PV and next S, tile 1's softmax runs.
// Tensor-memory map (512 columns): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P aliases S.
//
// Roofline: tensor-core bound; algorithmic FLOPs = 4 * D * (visible q,k pairs) per head.
// Every mbarrier wait is bounded; on expiry the kernel records a status word and drains.
#include <cuda.h>

#include "esp_common.cuh"
#include "sm100_ptx.cuh"

namespace esp {

using namespace ptx;

constexpr int BM = 128;               // rows per q tile
constexpr int QT = 2;                 // q tiles per CTA
constexpr int BN = 128;               // keys per kv tile
constexpr int HD = 128;               // head dim
constexpr int NSTAGE = 4;             // K/V ring stages
constexpr int TILE_BYTES = BN * HD * 2;
constexpr int HALF_BYTES = TILE_BYTES / 2;   // 64 head-dim columns x 128 rows (one swizzle-128B panel)
#ifndef ESP_PREFILL_THREADS
#define ESP_PREFILL_THREADS 384       // 3 warpgroups: softmax tile 0, softmax tile 1, {producer, MMA, 2 idle warps}
#endif
#ifndef ESP_POLY_EXP_PER_32
#define ESP_POLY_EXP_PER_32 0         // of every 32 exponentials, this many run on the FMA pipe instead of MUFU
#endif
constexpr int NUM_THREADS = ESP_PREFILL_THREADS;
constexpr bool kUseSetMaxNReg = (NUM_THREADS == 384);
constexpr int kPolyPer32 = ESP_POLY_EXP_PER_32;
static_assert(kPolyPer32 == 0 || kPolyPer32 == 2 || kPolyPer32 == 4 || kPolyPer32 == 8 || kPolyPer32 == 16 || kPolyPer32 == 32,
              "ESP_POLY_EXP_PER_32 must be 0 or a power of two up to 32");
constexpr int TMEM_COLS = 512;
constexpr float kRescaleThreshold = 8.0f;              // lazy O rescale: tolerate 2^8 growth
#ifndef ESP_SPEC_MAX
#define ESP_SPEC_MAX 0
#endif
constexpr bool kSpeculateMax = ESP_SPEC_MAX != 0;
#ifndef ESP_CHEAP_DESC
#define ESP_CHEAP_DESC 0
#endif
#ifndef ESP_WARP_ARRIVE
#define ESP_WARP_ARRIVE 0
#endif
constexpr int kPReadyArrivals = ESP_WARP_ARRIVE ? 4 : 128;   // arrivals that publish one tile's P

enum BarIdx { B_QFULL = 0, B_KVFULL = 2, B_KVEMPTY = 2 + NSTAGE, B_SFULL = 2 + 2 * NSTAGE,
              B_PREADY = 4 + 2 * NSTAGE, B_ODONE = 6 + 2 * NSTAGE, B_COUNT = 8 + 2 * NSTAGE };

constexpr int SMEM_Q = 0;
constexpr int SMEM_KV = QT * TILE_BYTES;
constexpr int SMEM_BAR = SMEM_KV + NSTAGE * TILE_BYTES;
constexpr int SMEM_MISC = SMEM_BAR + B_COUNT * 8;
constexpr int SMEM_TOTAL = SMEM_MISC + 16;
constexpr int SMEM_DYN = SMEM_TOTAL + 1024;            // slack to align the base to 1024 B

__device__ int g_esp_status[4];
// Bound of every mbarrier wait in SM cycles (about a second by default); esp_set_wait_limit_cycles changes it.
__device__ long long g_wait_limit_cycles = 2000000000LL;

#ifdef ESP_PREFILL_TRACE
// Tuning aid, compiled only into experiment builds: per-phase SM clock stamps of one CTA.
// g_trace[role][iteration][stamp]; role 0/1 = softmax tile 0/1 (lane 0 of its first warp), 2 = MMA issuer.
__device__ long long g_trace[3][64][8];
#define ESP_TRACE(role, j, k) do { if (trace_on && (j) < 64) g_trace[role][j][k] = clock64(); } while (0)
#else
#define ESP_TRACE(role, j, k) do { } while (0)
#endif

struct PrefillParams {
    void* o; float* m; float* l;
    int64_t o_stride_t, o_stride_h;
    const int32_t* q_start; const int32_t* q_len; const int32_t* q_first;
    const int32_t* kv_start; const int32_t* kv_len; const int32_t* kv_first;
    int num_q_heads, group, stride_s, num_qblocks;
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
// 2^x on the FMA/ALU pipes for x <= ~8 (Cody-Waite split + degree-3 minimax polynomial on [0,1),
// relative error < 1e-4, below the 16-bit rounding of P).  x is clamped at -126; -inf gives ~0 (2^-126 * p).
__device__ __forceinline__ float exp2_poly(float x) {
    x = fmaxf(x, -126.f);
    float xf;
    asm("add.rm.ftz.f32 %0, %1, %2;" : "=f"(xf) : "f"(x), "f"(12582912.f));   // 1.5 * 2^23: floor(x) lands in the mantissa
    const float fl = xf - 12582912.f;
    const float f = x - fl;                                                     // in [0, 1)
    float pz = fmaf(f, 0.077119089663028717f, 0.227564394474029541f);
    pz = fmaf(pz, f, 0.695146143436431885f);
    pz = fmaf(pz, f, 1.0f);
    return __uint_as_float(__float_as_uint(pz) + (__float_as_uint(xf) << 23));
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

// Packed version of exp2_poly for two values (f32x2 FMA-pipe instructions).
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
    x.x = fmaxf(x.x, -126.f); x.y = fmaxf(x.y, -126.f);
    const float2 magic = make_float2(12582912.f, 12582912.f);
    const float2 xf = __fadd2_rd(x, magic);                              // floor(x) in the mantissa
    const float2 fl = __fadd2_rn(xf, make_float2(-12582912.f, -12582912.f));
    const float2 f = __ffma2_rn(fl, make_float2(-1.f, -1.f), x);         // x - floor(x) in [0, 1)
    float2 pz = __ffma2_rn(f, make_float2(0.077119089663028717f, 0.077119089663028717f),
                           make_float2(0.227564394474029541f, 0.227564394474029541f));
    pz = __ffma2_rn(pz, f, make_float2(0.695146143436431885f, 0.695146143436431885f));
    pz = __ffma2_rn(pz, f, make_float2(1.f, 1.f));
    return make_float2(__uint_as_float(__float_as_uint(pz.x) + (__float_as_uint(xf.x) << 23)),
                       __uint_as_float(__float_as_uint(pz.y) + (__float_as_uint(xf.y) << 23)));
}

#ifndef ESP_EXP_VARIANT
#define ESP_EXP_VARIANT 0
#endif
// p = 2^(s*scale - m) for one 32-column chunk; packs to 16-bit pairs and returns the chunk's row sum
// (two independent packed accumulators)
template <typename T, int OFF, bool kTrackMax = false>
__device__ __forceinline__ float chunk_exp(const uint32_t (&r)[32], float scale, float neg_m, uint32_t (&pk)[32],
                                           float* mx4 = nullptr) {
    const float2 sc2 = make_float2(scale, scale), nm2 = make_float2(neg_m, neg_m);
    float2 acc[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
    constexpr int kStride = kPolyPer32 > 0 ? 32 / kPolyPer32 : 1;   // every kStride-th pair goes to the FMA pipe
#if ESP_EXP_VARIANT == 1
    // staged: all scale/subtract first, then all exponentials, then sums and packing
    float2 x[16], e[16];
#pragma unroll
    for (int i = 0; i < 16; ++i)
        x[i] = __ffma2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), sc2, nm2);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        if (kPolyPer32 > 0 && (i % kStride) == kStride - 1) e[i] = exp2_poly2(x[i]);
        else { e[i].x = ex2(x[i].x); e[i].y = ex2(x[i].y); }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        acc[i & 1] = __fadd2_rn(acc[i & 1], e[i]);
        pk[OFF + i] = Cvt<T>::pack(e[i].x, e[i].y);
    }
#else
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), sc2, nm2);
        float2 e;
        if (kPolyPer32 > 0 && ((i / 2) % kStride) == kStride - 1) {
            e = exp2_poly2(x);
        } else {
            e.x = ex2(x.x); e.y = ex2(x.y);
        }
        acc[(i / 2) & 1] = __fadd2_rn(acc[(i / 2) & 1], e);
        pk[OFF + i / 2] = Cvt<T>::pack(e.x, e.y);
        if (kTrackMax) mx4[(i / 2) & 3] = fmax3(mx4[(i / 2) & 3], __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
    }
#endif
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
#ifdef ESP_PREFILL_TRACE
    const bool trace_on = (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && (warp == 0 || warp == 4 || warp == 9));
#endif
    const int qb = p.num_qblocks - 1 - (int)blockIdx.x;      // heaviest q block first
    const int head = blockIdx.y, b = blockIdx.z;
    const int kvh = head / p.group;

    const int q_len = p.q_len[b];
    const int m0 = qb * (QT * BM);
    if (m0 >= q_len) return;
    const int kv_len = p.kv_len[b];
    const int q_start = p.q_start[b], kv_start = p.kv_start[b];
    // key n visible to local row r  <=>  n <= r - delta  and  n < kv_len
    const int dnum = p.kv_first[b] - p.q_first[b];
    const int delta = dnum >= 0 ? (dnum + p.stride_s - 1) / p.stride_s : -((-dnum) / p.stride_s);
    int n_tiles[QT];
#pragma unroll
    for (int t = 0; t < QT; ++t) {
        const int r0 = m0 + t * BM;
        int cnt = 0;
        if (r0 < q_len) {
            const int last_row = min(r0 + BM - 1, q_len - 1);
            const int range = max(0, min(last_row - delta + 1, kv_len));
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
      if (kUseSetMaxNReg) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
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
            for (int r = 0; r < 2 * nmax; ++r) {
                const int stage = r % NSTAGE, use = r / NSTAGE;
                if (use > 0 && !bounded_wait(bar(B_KVEMPTY + stage), (use - 1) & 1, s_abort, 1, r)) break;
                const int j = r >> 1;
                const CUtensorMap* tm = (r & 1) ? &tm_v : &tm_k;
                const uint32_t dst = smem_base + SMEM_KV + stage * TILE_BYTES;
                mbar_expect_tx(bar(B_KVFULL + stage), TILE_BYTES);
                tma_load_3d(dst, tm, bar(B_KVFULL + stage), 0, kvh, kv_start + j * BN);
                tma_load_3d(dst + HALF_BYTES, tm, bar(B_KVFULL + stage), 64, kvh, kv_start + j * BN);
            }
        }
      } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc_s = make_idesc(Fmt<T>::kAB, 0, BM, BN);
        constexpr uint32_t idesc_pv = make_idesc(Fmt<T>::kAB, 1, BM, HD);
#if ESP_CHEAP_DESC
        // The issuing thread shares its scheduler with two softmax warps, so every instruction between two MMAs costs
        // tensor-pipe time: descriptors are formed once per operand tile and stepped with one 64-bit add per MMA
        // (the address field cannot carry out of its 14 bits: shared memory ends below 256 KiB).
        const uint64_t dq0 = desc_kmajor_sw128(smem_base + SMEM_Q);
        const uint64_t dk0 = desc_kmajor_sw128(smem_base + SMEM_KV);
        const uint64_t dv0 = desc_mnmajor_sw128(smem_base + SMEM_KV, HALF_BYTES);
        auto issue_s = [&](int t, int stage) {
            const uint64_t qa = dq0 + (uint64_t)(t * (TILE_BYTES >> 4));
            const uint64_t kb = dk0 + (uint64_t)(stage * (TILE_BYTES >> 4));
            const uint32_t d = tmem_base + t * BN;
#pragma unroll
            for (int k = 0; k < HD / 16; ++k) {
                const uint64_t off = (uint64_t)(((k >> 2) * HALF_BYTES + (k & 3) * 32) >> 4);
                umma_ss(d, qa + off, kb + off, idesc_s, k > 0);
            }
        };
        auto issue_pv = [&](int t, int stage, bool acc) {
            const uint64_t vb = dv0 + (uint64_t)(stage * (TILE_BYTES >> 4));
            const uint32_t d = tmem_base + QT * BN + t * HD, a = tmem_base + t * BN;
#pragma unroll
            for (int k = 0; k < BN / 16; ++k)
                umma_ts(d, a + k * 8, vb + (uint64_t)(k * (2048 >> 4)), idesc_pv, (acc || k > 0) ? 1u : 0u);
        };
#else
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
#endif
        bool ok = true;
#pragma unroll
        for (int t = 0; t < QT; ++t)
            if (n_tiles[t] > 0) ok = ok && bounded_wait(bar(B_QFULL + t), 0, s_abort, 2, t);
        ok = ok && bounded_wait(bar(B_KVFULL + 0), 0, s_abort, 3, 0);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after();
            if (lane == 0) {
#pragma unroll
                for (int t = 0; t < QT; ++t)
                    if (n_tiles[t] > 0) { issue_s(t, 0); umma_commit(bar(B_SFULL + t)); }
                umma_commit(bar(B_KVEMPTY + 0));
            }
            for (int j = 0; j < nmax && ok; ++j) {
                const int rv = 2 * j + 1, sv = rv % NSTAGE;
                ok = bounded_wait(bar(B_KVFULL + sv), (rv / NSTAGE) & 1, s_abort, 4, j);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if ((j + 1) * BN > kv_len) {
                    // tail tile: rows past the request's last key may hold anything (even NaN); P is 0
                    // there, so make V finite by zeroing those rows in shared memory.
                    const int first_bad = kv_len - j * BN;
                    uint8_t* vs = smem_gen + SMEM_KV + sv * TILE_BYTES;
                    for (int i = first_bad * 8 + lane; i < BN * 8; i += 32) {      // 8 x 16 B per 128 B row
                        *reinterpret_cast<uint4*>(vs + i * 16) = make_uint4(0, 0, 0, 0);
                        *reinterpret_cast<uint4*>(vs + HALF_BYTES + i * 16) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                }
                const bool have_next = j + 1 < nmax;
                const int rk = 2 * j + 2, sk = rk % NSTAGE;
                if (have_next) {
                    ok = bounded_wait(bar(B_KVFULL + sk), (rk / NSTAGE) & 1, s_abort, 5, j);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
#pragma unroll
                for (int t = 0; t < QT; ++t) {
                    if (j < n_tiles[t]) {
                        ESP_TRACE(2, j, t * 4 + 0);
                        ok = bounded_wait(bar(B_PREADY + t), j & 1, s_abort, 6 + t, j);
                        ESP_TRACE(2, j, t * 4 + 1);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        tc_fence_after();
                        if (lane == 0) {
                            issue_pv(t, sv, j > 0);
                            ESP_TRACE(2, j, t * 4 + 2);
                            if (j == n_tiles[t] - 1) umma_commit(bar(B_ODONE + t));
                        }
                    }
                    if (j + 1 < n_tiles[t] && lane == 0) {
                        issue_s(t, sk);
                        umma_commit(bar(B_SFULL + t));
                        ESP_TRACE(2, j, t * 4 + 3);
                    }
                }
                if (!ok) break;
                if (lane == 0) {
                    umma_commit(bar(B_KVEMPTY + sv));
                    if (have_next) umma_commit(bar(B_KVEMPTY + sk));
                }
                __syncwarp();
            }
        }
      }
    } else {
        // ------------------------------------------------------------------ softmax + epilogue
        if (kUseSetMaxNReg) asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
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
                ESP_TRACE(t, j, 0);
                ok = bounded_wait(bar(B_SFULL + t), j & 1, s_abort, 8 + t, j);
                ESP_TRACE(t, j, 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                uint32_t sr[4][32];
                tmem_ld32(tS, sr[0]);
                tmem_ld32(tS + 32, sr[1]);
                tmem_wait_ld();
                ESP_TRACE(t, j, 2);
                tmem_ld32(tS + 64, sr[2]);          // second half streams in while the first is reduced
                tmem_ld32(tS + 96, sr[3]);
                const int n0 = j * BN;
                const int r0 = m0 + t * BM;
                const bool masked = (n0 + BN - 1 > r0 - delta) || (n0 + BN > kv_len);
                const int limit = min(row - delta, kv_len - 1) - n0;     // columns <= limit are visible
                // After the first tile the running maximum rarely grows by more than the lazy-rescale threshold, so the
                // exponentials of an unmasked tile are taken against the running maximum straight away while the
                // tile's own maximum is found alongside on the ALU pipe.  P is stored only once every row of the warp
                // is known to have stayed within the threshold; otherwise S (still intact in tensor memory) is read
                // again and the tile is done the slow way: maximum first, O rescaled, then the exponentials.
                float lsum = 0.f;
                bool published = false;
                if (kSpeculateMax && !masked && j > 0) {
                    ESP_TRACE(t, j, 3);
                    const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
                    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                    uint32_t pa[32], pb[32];
                    const float s0 = chunk_exp<T, 0, true>(sr[0], scale, neg_m, pa, mx4);
                    const float s1 = chunk_exp<T, 16, true>(sr[1], scale, neg_m, pa, mx4);
                    tmem_wait_ld();
                    const float s2 = chunk_exp<T, 0, true>(sr[2], scale, neg_m, pb, mx4);
                    const float s3 = chunk_exp<T, 16, true>(sr[3], scale, neg_m, pb, mx4);
                    const float m_tile = fmaxf(fmax3(mx4[0], mx4[1], mx4[2]), mx4[3]) * scale;
                    const bool outgrown = (m_tile > m_run + kRescaleThreshold) || (m_run == -INFINITY);
                    if (!__any_sync(0xffffffffu, outgrown)) {
                        tmem_st32(tS, pa);
                        tmem_st32(tS + 32, pb);
                        lsum = (s0 + s1) + (s2 + s3);
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
                    float mx = fmaxf(chunk_max(sr[0], 0, limit, masked), chunk_max(sr[1], 32, limit, masked));
                    tmem_wait_ld();
                    mx = fmax3(mx, chunk_max(sr[2], 64, limit, masked), chunk_max(sr[3], 96, limit, masked));
                    ESP_TRACE(t, j, 3);
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
                ESP_TRACE(t, j, 4);
                l_run += lsum;
                tmem_wait_st();
                tc_fence_before();
#if ESP_WARP_ARRIVE
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_PREADY + t));
#else
                mbar_arrive(bar(B_PREADY + t));
#endif
                ESP_TRACE(t, j, 5);
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

// [tokens, heads, 128] 16-bit tensor, box = 64 dims x 1 head x 128 tokens, 128-byte swizzle.
static int make_tile_map(CUtensorMap* tm, const void* base, int64_t tokens, int heads, int64_t stride_t,
                         int64_t stride_h, int dtype) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) { snprintf(last_cuda_error_buf(), 256, "cuTensorMapEncodeTiled entry point not found"); return ESP_ERR_CUDA; }
    cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)heads, (cuuint64_t)tokens};
    cuuint64_t strides[2] = {(cuuint64_t)stride_h * 2, (cuuint64_t)stride_t * 2};
    cuuint32_t box[3] = {64, 1, (cuuint32_t)BN};
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
    if (kUseSetMaxNReg) {
        // the in-kernel register re-distribution (256 softmax threads x 224 + 128 other threads x 56) must fit the
        // registers the CTA is launched with, or setmaxnreg.inc would block
        cudaFuncAttributes fa;
        ESP_CUDA_TRY(cudaFuncGetAttributes(&fa, prefill_step_kernel<T, OT>));
        if (fa.numRegs * NUM_THREADS < 256 * 224 + 128 * 56) {
            snprintf(last_cuda_error_buf(), 256, "prefill kernel was built with %d registers per thread, too few for its setmaxnreg plan", fa.numRegs);
            return ESP_ERR_UNSUPPORTED;
        }
    }
    prefill_step_kernel<T, OT><<<grid, NUM_THREADS, SMEM_DYN, s>>>(tq, tk, tv, pp);
    ESP_LAUNCH_CHECK("prefill_step_kernel");
    return ESP_OK;
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
    if (batch == 0 || max_q_b_seq_len <= 0 || q_tokens == 0 || kv_tokens == 0) return ESP_OK;
    if (!q || !k || !v || !o || !m || !l || !q_b_start_loc || !q_b_seq_len || !q_first_token_global_idx ||
        !kv_b_start_loc || !kv_b_seq_len || !kv_first_token_global_idx || batch < 0 || num_q_heads <= 0 ||
        num_kv_heads <= 0 || num_q_heads % num_kv_heads || logical_sp_peers_num <= 0 || q_tokens < 0 ||
        kv_tokens < 0)
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
    if ((rc = make_tile_map(&tq, q, q_tokens, num_q_heads, q_stride_t, q_stride_h, dtype))) return rc;
    if ((rc = make_tile_map(&tk, k, kv_tokens, num_kv_heads, kv_stride_t, kv_stride_h, dtype))) return rc;
    if ((rc = make_tile_map(&tv, v, kv_tokens, num_kv_heads, kv_stride_t, kv_stride_h, dtype))) return rc;
    PrefillParams pp;
    pp.o = o; pp.m = m; pp.l = l; pp.o_stride_t = o_stride_t; pp.o_stride_h = o_stride_h;
    pp.q_start = q_b_start_loc; pp.q_len = q_b_seq_len; pp.q_first = q_first_token_global_idx;
    pp.kv_start = kv_b_start_loc; pp.kv_len = kv_b_seq_len; pp.kv_first = kv_first_token_global_idx;
    pp.num_q_heads = num_q_heads; pp.group = num_q_heads / num_kv_heads; pp.stride_s = logical_sp_peers_num;
    pp.num_qblocks = (max_q_b_seq_len + QT * BM - 1) / (QT * BM);
    pp.scale_log2 = (sm_scale > 0.f ? sm_scale : 1.0f / sqrtf((float)head_dim)) * 1.4426950408889634f;
    dim3 grid(pp.num_qblocks, num_q_heads, batch);
    cudaStream_t s = (cudaStream_t)stream;
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

#ifdef ESP_PREFILL_TRACE
extern "C" int esp_debug_read_trace(long long* out) {
    ESP_CUDA_TRY(cudaDeviceSynchronize());
    ESP_CUDA_TRY(cudaMemcpyFromSymbol(out, g_trace, sizeof(long long) * 3 * 64 * 8));
    return ESP_OK;
}
#endif

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
