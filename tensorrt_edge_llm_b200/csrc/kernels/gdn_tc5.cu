// Gated DeltaNet prefill as a chunked scan on 5th-generation tensor cores.
//
// Per token (value head h, key / value dims 128, state H [K, V] fp32):
//   q̂ = q/‖q‖/√K, k̂ = k/‖k‖,  g = exp(−exp(A_log) · softplus(a + dt_bias)),  β = σ(b)
//   H ← g H;   Δ = β (v − Hᵀ k̂);   H ← H + k̂ ⊗ Δ;   o = Hᵀ q̂
// Over a chunk of 64 tokens with γ_t = Π_{i≤t} g_i the recurrence closes into matrix form (H0 = state at chunk entry):
//   (I + A) Δ = β ∘ (V − diag(γ) K̂ H0),   A[t,s] = β_t (γ_t/γ_s) (k̂_t·k̂_s)  for s < t      (unit lower-triangular system)
//   O = diag(γ) Q̂ H0 + W Δ,               W[t,s] = (γ_t/γ_s) (q̂_t·k̂_s)      for s ≤ t
//   H ← γ_L H0 + K̂ᵀ diag(γ_L/γ_s) Δ
// Five of the six products — K̂K̂ᵀ, Q̂K̂ᵀ, K̂H0, Q̂H0 (issued together), WΔ and the state update — run on tcgen05 with fp32
// accumulation in TMEM; the triangular system is solved by forward substitution, one value column per thread with the
// column's 64 unknowns in registers (2016 multiply-adds per thread and chunk, coefficients broadcast from shared memory).
// One CTA owns a (sequence, value head) pair and walks its chunks in order: the fp32 state never leaves TMEM, a 16-bit
// copy in shared memory feeds the next chunk's K̂H0 / Q̂H0 products.
//
// The 64 token rows are loaded twice (rows 0-63 and 64-127 of the 128-row MMA operand), so all four lane quadrants of
// TMEM hold valid rows and all 128 compute threads take part in every read-out: thread r serves token r % 64 and the
// column half r / 64.  Rows past the end of a ragged sequence get g = 1, β = 0: no state change, nothing stored.
// TMEM (512 columns): K̂K̂ᵀ [0,64) · Q̂K̂ᵀ [64,128) · K̂H0, later WΔ [128,256) · Q̂H0 [256,384) · H [384,512).
// Compiled shape: key and value dims 128.  Every wait is bounded.
//
// Reference counterpart: the CuTe-DSL kernels kernelSrcs/gdn_cutedsl/gdn_prefill_blackwell.py (+ varlen), registered in
// kernelSrcs/build_cutedsl.py:251-261; semantics follow unittests/cpp/kernels/gdnKernels/gdnCuteDslTests.cu:157-238.
#include <type_traits>

#include "host_utils.h"
#include "tc5_common.cuh"

namespace telb {

constexpr int kGdnL = 64;
constexpr int kGdnThreads = 192;

struct GdnParams {
    const void* a;             // [T, hv]
    const void* b;             // [T, hv]
    const float* A_log;        // [hv]
    const float* dt_bias;      // [hv]
    float* state;              // [rows, hv, 128, 128] fp32
    void* out;                 // [T, hv, 128]
    const int* q_start;
    const int* q_len;
    const int* past_len;
    const int* slot_ids;
    int hk, hv;
    int* status;
};

__device__ __forceinline__ float gdn_softplus(float x) { return x > 20.f ? x : log1pf(__expf(x)); }
__device__ __forceinline__ void tmem_st_x32_g(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
          "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
          "r"(r[30]), "r"(r[31]) : "memory");
}

// byte offset of 16-byte chunk `c` of row `row` in a [rows x 128 B] tile with the 128-byte swizzle
__device__ __forceinline__ uint32_t sw128(int row, int c) { return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((c ^ (row & 7)) << 4)); }

template <typename T>
__global__ void __launch_bounds__(kGdnThreads, 1)
gdn_chunk_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                 const __grid_constant__ CUtensorMap tma_v, GdnParams p) {
    constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;                        // 2 key halves x [128 rows x 128 B] (rows 64-127 repeat rows 0-63); reused for R
    uint8_t* sK = sQ + 32768;                  // same shape
    uint8_t* sV = sK + 32768;                  // 2 value halves x [64 rows x 128 B]
    uint8_t* sH = sV + 16384;                  // state copy: 2 value halves x [128 key rows x 128 B]
    uint8_t* sW = sH + 32768;                  // W: [128 rows x 128 B] (64 chunk columns)
    uint8_t* sD = sW + 16384;                  // Δ: 2 value halves x [64 rows x 128 B]
    uint8_t* sDs = sD + 16384;                 // Δ · γ_L/γ_s, same shape
    float* sCoef = reinterpret_cast<float*>(sDs + 16384);     // A [64][64] fp32
    float* sCum = sCoef + kGdnL * kGdnL;                      // log2 γ_t [64]
    float* sBeta = sCum + kGdnL;                              // β_t [64]
    float* sTmp = sBeta + kGdnL;                              // [8]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sTmp + 8);
    uint64_t* full_bar = bars;        // the chunk's q, k, v have landed
    uint64_t* qk_ready = bars + 1;    // q̂, k̂ normalised in place (128 arrivals)
    uint64_t* h_ready = bars + 2;     // 16-bit state copy written (128 arrivals)
    uint64_t* g_bar = bars + 3;       // the four entry products are in TMEM
    uint64_t* d_ready = bars + 4;     // W, Δ, scaled Δ in shared memory, H decayed (128 arrivals)
    uint64_t* o_bar = bars + 5;       // W Δ is in TMEM
    uint64_t* s_bar = bars + 6;       // the state update has completed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* sR = reinterpret_cast<float*>(sQ);                 // R [64][128] fp32, 16-byte chunks XOR-swizzled by the row

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int seq = blockIdx.x / p.hv, h = blockIdx.x - seq * p.hv;
    const int kh = h / (p.hv / p.hk);

    if (threadIdx.x == 0) {
        mbar_init(full_bar, 1);
        mbar_init(qk_ready, 128);
        mbar_init(h_ready, 128);
        mbar_init(g_bar, 1);
        mbar_init(d_ready, 128);
        mbar_init(o_bar, 1);
        mbar_init(s_bar, 1);
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tensormap(&tma_q);
        prefetch_tensormap(&tma_k);
        prefetch_tensormap(&tma_v);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    pdl_prologue();
    const uint32_t tmem_base = *tmem_slot;
    const int ql = p.q_len[seq];
    const int t_first = p.q_start[seq];
    const int nchunks = (ql + kGdnL - 1) / kGdnL;
    constexpr uint32_t kColKK = 0, kColQK = 64, kColKH = 128, kColQH = 256, kColH = 384;

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            for (int c = 0; c < nchunks; ++c) {
                if (c > 0 && !mbar_wait(s_bar, (uint32_t)(c - 1) & 1u, abort_flag, p.status, kStatusProducerTimeout)) break;
                const int t0 = t_first + c * kGdnL;
                mbar_expect_tx(full_bar, 32768 + 32768 + 16384);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
#pragma unroll
                    for (int copy = 0; copy < 2; ++copy) {
                        tma_load_2d(sQ + half * 16384 + copy * 8192, &tma_q, full_bar, kh * 128 + half * 64, t0);
                        tma_load_2d(sK + half * 16384 + copy * 8192, &tma_k, full_bar, kh * 128 + half * 64, t0);
                    }
                    tma_load_2d(sV + half * 8192, &tma_v, full_bar, h * 128 + half * 64, t0);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t id_kk = idesc_f16(128, 64, kBf16);                    // K-major x K-major
            const uint32_t id_xh = idesc_f16(128, 128, kBf16, false, true);      // K-major A x MN-major B
            const uint32_t id_st = idesc_f16(128, 128, kBf16, true, true);       // MN-major A (K̂ᵀ) x MN-major B
            for (int c = 0; c < nchunks; ++c) {
                const uint32_t par = (uint32_t)c & 1u;
                if (!mbar_wait(qk_ready, par, abort_flag, p.status, kStatusMmaTimeout)) break;
                if (!mbar_wait(h_ready, par, abort_flag, p.status, kStatusMmaTimeout)) break;
                tc_fence_after_sync();
                const uint64_t dQ = smem_desc_sw128(sQ), dK = smem_desc_sw128(sK);
                const uint64_t dH = smem_desc_sw128_mn(sH, 16384, 1024);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint64_t off = (uint64_t)((k >> 2) * 16384 >> 4) + 2 * (k & 3);
                    umma_f16(tmem_base + kColKK, dK + off, dK + off, id_kk, k > 0 ? 1u : 0u);
                    umma_f16(tmem_base + kColQK, dQ + off, dK + off, id_kk, k > 0 ? 1u : 0u);
                    umma_f16(tmem_base + kColKH, dK + off, dH + (uint64_t)(k * 2048 >> 4), id_xh, k > 0 ? 1u : 0u);
                    umma_f16(tmem_base + kColQH, dQ + off, dH + (uint64_t)(k * 2048 >> 4), id_xh, k > 0 ? 1u : 0u);
                }
                umma_commit(g_bar);
                if (!mbar_wait(d_ready, par, abort_flag, p.status, kStatusMmaTimeout)) break;
                tc_fence_after_sync();
                const uint64_t dW = smem_desc_sw128(sW);
                const uint64_t dD = smem_desc_sw128_mn(sD, 8192, 1024), dDs = smem_desc_sw128_mn(sDs, 8192, 1024);
                const uint64_t dKt = smem_desc_sw128_mn(sK, 16384, 1024);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_f16(tmem_base + kColKH, dW + 2 * k, dD + (uint64_t)(k * 2048 >> 4), id_xh, k > 0 ? 1u : 0u);
                umma_commit(o_bar);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_f16(tmem_base + kColH, dKt + (uint64_t)(k * 2048 >> 4), dDs + (uint64_t)(k * 2048 >> 4), id_st, 1u);
                umma_commit(s_bar);
            }
        }
    } else {
        // ---------------- compute threads ----------------
        const int quad = warp & 3;
        const int r = quad * 32 + lane;            // physical row / TMEM lane / key index / value column
        const int tt = r & 63;                     // token of the chunk served in the read-outs
        const int ch = r >> 6;                     // column half served in the read-outs
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
        const float neg_exp_a = -__expf(p.A_log[h]) * 1.4426950408889634f, db = p.dt_bias[h];
        const T* ap = reinterpret_cast<const T*>(p.a);
        const T* bp = reinterpret_cast<const T*>(p.b);
        T* op = reinterpret_cast<T*>(p.out);
        float* st = p.state + ((size_t)p.slot_ids[seq] * p.hv + h) * (size_t)(128 * 128);
        bool ok = nchunks > 0;
        if (ok) {
            // initial state: fp32 master copy in TMEM (row = key index r), 16-bit copy in shared memory
            const bool fresh = p.past_len[seq] <= 0;
#pragma unroll 1
            for (int c32 = 0; c32 < 4; ++c32) {
                uint32_t v[32];
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    float4 f = fresh ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(st + (size_t)r * 128 + c32 * 32 + i);
                    v[i] = __float_as_uint(f.x); v[i + 1] = __float_as_uint(f.y); v[i + 2] = __float_as_uint(f.z); v[i + 3] = __float_as_uint(f.w);
                }
                tmem_st_x32_g(lane_addr + kColH + c32 * 32, v);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 u;
                    u.x = Cvt<T>::pack2(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
                    u.y = Cvt<T>::pack2(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
                    u.z = Cvt<T>::pack2(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
                    u.w = Cvt<T>::pack2(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
                    const int vc = c32 * 32 + q * 8;                   // first value column of this 16-byte chunk
                    *reinterpret_cast<uint4*>(sH + (vc >> 6) * 16384 + sw128(r, (vc & 63) >> 3)) = u;
                }
            }
            tmem_st_wait();
            tc_fence_before_sync();
            fence_proxy_async_smem();
            mbar_arrive(h_ready);
        }
        for (int c = 0; c < nchunks && ok; ++c) {
            const uint32_t par = (uint32_t)c & 1u;
            const int len = min(kGdnL, ql - c * kGdnL);
            const size_t tbase = (size_t)t_first + (size_t)c * kGdnL;
            // ---- gates: log2 γ (inclusive cumulative sum over the chunk), β ----
            named_barrier_sync(1, 128);                      // readers of sCum / sBeta of the previous chunk are done
            if (r < kGdnL) {
                float lg = 0.f, beta = 0.f;
                if (r < len) {
                    lg = neg_exp_a * gdn_softplus(Cvt<T>::to_f(ap[(tbase + r) * p.hv + h]) + db);
                    beta = 1.f / (1.f + __expf(-Cvt<T>::to_f(bp[(tbase + r) * p.hv + h])));
                }
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float n = __shfl_up_sync(0xffffffffu, lg, o);
                    if (lane >= o) lg += n;
                }
                if (r == 31) sTmp[0] = lg;
                sBeta[r] = beta;
                sCum[r] = lg;                                 // second warp adds the first warp's total below
            }
            named_barrier_sync(1, 128);
            if (r >= 32 && r < kGdnL) sCum[r] += sTmp[0];
            named_barrier_sync(1, 128);
            const float c_t = sCum[tt], beta_t = sBeta[tt], c_last = sCum[kGdnL - 1];
            // ---- q̂, k̂: every thread normalises its own physical row (both key halves) in place ----
            if (!mbar_wait(full_bar, par, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
            {
                float sq = 0.f, sk = 0.f;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
#pragma unroll
                    for (int cc = 0; cc < 8; ++cc) {
                        const uint4 uq = *reinterpret_cast<const uint4*>(sQ + half * 16384 + sw128(r, cc));
                        const uint4 uk = *reinterpret_cast<const uint4*>(sK + half * 16384 + sw128(r, cc));
                        const T* eq = reinterpret_cast<const T*>(&uq);
                        const T* ek = reinterpret_cast<const T*>(&uk);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float fq = Cvt<T>::to_f(eq[i]), fk = Cvt<T>::to_f(ek[i]);
                            sq += fq * fq;
                            sk += fk * fk;
                        }
                    }
                }
                const float nq = rsqrtf(sq + 1e-6f) * 0.08838834764831845f, nk = rsqrtf(sk + 1e-6f);      // 1/sqrt(128)
#pragma unroll
                for (int half = 0; half < 2; ++half) {
#pragma unroll
                    for (int cc = 0; cc < 8; ++cc) {
                        uint4* pq = reinterpret_cast<uint4*>(sQ + half * 16384 + sw128(r, cc));
                        uint4* pk = reinterpret_cast<uint4*>(sK + half * 16384 + sw128(r, cc));
                        uint4 uq = *pq, uk = *pk;
                        const T* eq = reinterpret_cast<const T*>(&uq);
                        const T* ek = reinterpret_cast<const T*>(&uk);
                        uint4 oq, ok4;
                        oq.x = Cvt<T>::pack2(Cvt<T>::to_f(eq[0]) * nq, Cvt<T>::to_f(eq[1]) * nq);
                        oq.y = Cvt<T>::pack2(Cvt<T>::to_f(eq[2]) * nq, Cvt<T>::to_f(eq[3]) * nq);
                        oq.z = Cvt<T>::pack2(Cvt<T>::to_f(eq[4]) * nq, Cvt<T>::to_f(eq[5]) * nq);
                        oq.w = Cvt<T>::pack2(Cvt<T>::to_f(eq[6]) * nq, Cvt<T>::to_f(eq[7]) * nq);
                        ok4.x = Cvt<T>::pack2(Cvt<T>::to_f(ek[0]) * nk, Cvt<T>::to_f(ek[1]) * nk);
                        ok4.y = Cvt<T>::pack2(Cvt<T>::to_f(ek[2]) * nk, Cvt<T>::to_f(ek[3]) * nk);
                        ok4.z = Cvt<T>::pack2(Cvt<T>::to_f(ek[4]) * nk, Cvt<T>::to_f(ek[5]) * nk);
                        ok4.w = Cvt<T>::pack2(Cvt<T>::to_f(ek[6]) * nk, Cvt<T>::to_f(ek[7]) * nk);
                        *pq = oq;
                        *pk = ok4;
                    }
                }
            }
            fence_proxy_async_smem();
            mbar_arrive(qk_ready);
            // ---- read-out of the entry products: A coefficients, W, R; decay of H ----
            if (!mbar_wait(g_bar, par, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
            tc_fence_after_sync();
            {
                uint32_t kk[32], qk[32];
                tmem_ld_x32(lane_addr + kColKK + ch * 32, kk);
                tmem_ld_x32(lane_addr + kColQK + ch * 32, qk);
                tmem_ld_wait();
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    float w[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int j = q4 * 8 + i, s = ch * 32 + j;
                        const float dec = exp2f(c_t - sCum[s]);
                        sCoef[tt * kGdnL + s] = s < tt ? beta_t * dec * __uint_as_float(kk[j]) : 0.f;
                        w[i] = s <= tt ? dec * __uint_as_float(qk[j]) : 0.f;
                    }
                    uint4 u;
                    u.x = Cvt<T>::pack2(w[0], w[1]);
                    u.y = Cvt<T>::pack2(w[2], w[3]);
                    u.z = Cvt<T>::pack2(w[4], w[5]);
                    u.w = Cvt<T>::pack2(w[6], w[7]);
                    const int chunk16 = ch * 4 + q4;
                    *reinterpret_cast<uint4*>(sW + sw128(tt, chunk16)) = u;            // both copies of the row: the MMA's
                    *reinterpret_cast<uint4*>(sW + sw128(tt + 64, chunk16)) = u;       // M side has 128 rows
                }
            }
            {
                const float gam = exp2f(c_t);
#pragma unroll 1
                for (int c32 = 0; c32 < 2; ++c32) {
                    uint32_t khv[32];
                    tmem_ld_x32(lane_addr + kColKH + ch * 64 + c32 * 32, khv);
                    tmem_ld_wait();
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const uint4 uv = *reinterpret_cast<const uint4*>(sV + ch * 8192 + sw128(tt, c32 * 4 + q4));
                        const T* ev = reinterpret_cast<const T*>(&uv);
                        float rr[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) rr[i] = beta_t * (Cvt<T>::to_f(ev[i]) - gam * __uint_as_float(khv[q4 * 8 + i]));
                        const int v4 = (ch * 64 + c32 * 32 + q4 * 8) >> 2;             // index of the first 16-byte chunk
                        *reinterpret_cast<float4*>(sR + tt * 128 + (((v4) ^ (tt & 31)) << 2)) = make_float4(rr[0], rr[1], rr[2], rr[3]);
                        *reinterpret_cast<float4*>(sR + tt * 128 + (((v4 + 1) ^ (tt & 31)) << 2)) = make_float4(rr[4], rr[5], rr[6], rr[7]);
                    }
                }
            }
            {
                const float gl = exp2f(c_last);
#pragma unroll 1
                for (int c32 = 0; c32 < 4; ++c32) {
                    uint32_t hv32[32];
                    tmem_ld_x32(lane_addr + kColH + c32 * 32, hv32);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) hv32[i] = __float_as_uint(__uint_as_float(hv32[i]) * gl);
                    tmem_st_x32_g(lane_addr + kColH + c32 * 32, hv32);
                }
                tmem_st_wait();
            }
            tc_fence_before_sync();
            named_barrier_sync(1, 128);                      // coefficients and R complete before any column is solved
            // ---- forward substitution: thread r solves value column r ----
            {
                float dlt[kGdnL];
                const int v4 = r >> 2, vi = r & 3;
#pragma unroll
                for (int t = 0; t < kGdnL; ++t) {
                    // four partial sums: the chain of dependent multiply-adds per unknown is a quarter as long (the four
                    // compute warps sit on four different schedulers, so nothing else hides that latency)
                    float acc0 = sR[t * 128 + ((v4 ^ (t & 31)) << 2) + vi], acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
#pragma unroll
                    for (int s4 = 0; s4 < (t + 3) / 4; ++s4) {
                        const float4 cf = *reinterpret_cast<const float4*>(sCoef + t * kGdnL + s4 * 4);
                        if (s4 * 4 + 0 < t) acc0 -= cf.x * dlt[s4 * 4 + 0];
                        if (s4 * 4 + 1 < t) acc1 -= cf.y * dlt[s4 * 4 + 1];
                        if (s4 * 4 + 2 < t) acc2 -= cf.z * dlt[s4 * 4 + 2];
                        if (s4 * 4 + 3 < t) acc3 -= cf.w * dlt[s4 * 4 + 3];
                    }
                    dlt[t] = (acc0 + acc1) + (acc2 + acc3);
                }
                // Δ and Δ · γ_L/γ_s as 16-bit MN-major operands: row = chunk token, value columns contiguous
                const uint32_t col_off = (uint32_t)((r >> 6) * 8192);
#pragma unroll
                for (int t = 0; t < kGdnL; ++t) {
                    const uint32_t o2 = col_off + sw128(t, (r & 63) >> 3) + (r & 7) * 2;
                    *reinterpret_cast<T*>(sD + o2) = Cvt<T>::from_f(dlt[t]);
                    *reinterpret_cast<T*>(sDs + o2) = Cvt<T>::from_f(dlt[t] * exp2f(c_last - sCum[t]));
                }
            }
            fence_proxy_async_smem();
            mbar_arrive(d_ready);
            // ---- outputs ----
            if (!mbar_wait(o_bar, par, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
            tc_fence_after_sync();
            {
                const float gam = exp2f(c_t);
                const bool valid = tt < len;
#pragma unroll 1
                for (int c32 = 0; c32 < 2; ++c32) {
                    uint32_t qh[32], wd[32];
                    tmem_ld_x32(lane_addr + kColQH + ch * 64 + c32 * 32, qh);
                    tmem_ld_x32(lane_addr + kColKH + ch * 64 + c32 * 32, wd);
                    tmem_ld_wait();
                    if (valid) {
                        T* dst = op + ((tbase + tt) * p.hv + h) * 128 + ch * 64 + c32 * 32;
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            float o[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) o[i] = gam * __uint_as_float(qh[q4 * 8 + i]) + __uint_as_float(wd[q4 * 8 + i]);
                            uint4 u;
                            u.x = Cvt<T>::pack2(o[0], o[1]);
                            u.y = Cvt<T>::pack2(o[2], o[3]);
                            u.z = Cvt<T>::pack2(o[4], o[5]);
                            u.w = Cvt<T>::pack2(o[6], o[7]);
                            reinterpret_cast<uint4*>(dst)[q4] = u;
                        }
                    }
                }
            }
            // ---- new state: 16-bit copy for the next chunk, fp32 to the pool after the last chunk ----
            if (!mbar_wait(s_bar, par, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
            tc_fence_after_sync();
            const bool last = c == nchunks - 1;
#pragma unroll 1
            for (int c32 = 0; c32 < 4; ++c32) {
                uint32_t v[32];
                tmem_ld_x32(lane_addr + kColH + c32 * 32, v);
                tmem_ld_wait();
                if (last) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4*>(st + (size_t)r * 128 + c32 * 32 + i) =
                            make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]), __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                } else {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint4 u;
                        u.x = Cvt<T>::pack2(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
                        u.y = Cvt<T>::pack2(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
                        u.z = Cvt<T>::pack2(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
                        u.w = Cvt<T>::pack2(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
                        const int vc = c32 * 32 + q * 8;
                        *reinterpret_cast<uint4*>(sH + (vc >> 6) * 16384 + sw128(r, (vc & 63) >> 3)) = u;
                    }
                }
            }
            if (!last) {
                tc_fence_before_sync();
                fence_proxy_async_smem();
                mbar_arrive(h_ready);
            }
        }
    }

    if (*abort_flag) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace telb

using namespace telb;

// Gated DeltaNet chunked prefill (see the top of the file).  q, k [T, hk, 128], v [T, hv, 128], a, b [T, hv] 16-bit,
// A_log / dt_bias [hv] fp32, state [rows, hv, 128, 128] fp32 (read when past_len > 0, always written), out [T, hv, 128].
// One CTA per (sequence, value head).
extern "C" int telb_gdn_chunk_prefill(const void* q, const void* k, const void* v, const void* a, const void* b, const float* A_log,
                                      const float* dt_bias, float* state, void* out, const int* q_start, const int* q_len,
                                      const int* past_len, const int* slot_ids, int num_seqs, int total_tokens, int hk, int hv, int kdim,
                                      int vdim, int is_bf16, int* status, cudaStream_t stream) {
    if (num_seqs <= 0 || total_tokens <= 0) return 0;
    if (kdim != 128 || vdim != 128) return fail("telb_gdn_chunk_prefill: key / value head dims of 128 are the compiled shape");
    if (hk <= 0 || hv % hk) return fail("telb_gdn_chunk_prefill: value heads must be a multiple of key heads");
    const CUtensorMapDataType dtp = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap tq, tk, tv;
    if (make_tmap_2d(&tq, dtp, 2, q, total_tokens, (uint64_t)hk * 128, (uint64_t)hk * 256, kGdnL, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    if (make_tmap_2d(&tk, dtp, 2, k, total_tokens, (uint64_t)hk * 128, (uint64_t)hk * 256, kGdnL, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    if (make_tmap_2d(&tv, dtp, 2, v, total_tokens, (uint64_t)hv * 128, (uint64_t)hv * 256, kGdnL, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    GdnParams p{};
    p.a = a;
    p.b = b;
    p.A_log = A_log;
    p.dt_bias = dt_bias;
    p.state = state;
    p.out = out;
    p.q_start = q_start;
    p.q_len = q_len;
    p.past_len = past_len;
    p.slot_ids = slot_ids;
    p.hk = hk;
    p.hv = hv;
    p.status = status;
    constexpr int smem = 32768 * 2 + 16384 + 32768 + 16384 * 3 + (kGdnL * kGdnL + 2 * kGdnL + 8) * 4 + 128 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gdn_chunk_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gdn_chunk_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail("cudaFuncSetAttribute(gdn_chunk)", e);
        configured = true;
    }
    const dim3 grid(num_seqs * hv), block(kGdnThreads);
    if (is_bf16) TELB_LAUNCH("gdn_chunk_kernel", (gdn_chunk_kernel<__nv_bfloat16>), grid, block, smem, stream, tq, tk, tv, p);
    else TELB_LAUNCH("gdn_chunk_kernel", (gdn_chunk_kernel<__half>), grid, block, smem, stream, tq, tk, tv, p);
    TELB_CHECK_LAUNCH("gdn_chunk_kernel");
    return 0;
}
