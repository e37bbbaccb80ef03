// Mamba2 selective-state prefill as a chunked scan on 5th-generation tensor cores.
//
//   h_t = exp(A dt_t) h_{t-1} + (dt_t x_t) ⊗ B_t,     y_t = C_t · h_t + D x_t   (× silu(z_t))
//
// A sequence is cut into chunks of 128 tokens.  With a_l = Σ_{i≤l} A dt_i (inclusive, within the chunk) the chunk's
// outputs and its end state are four small matrix products (the "state-space duality" form):
//   G      = C Bᵀ                                    [128 x 128]   scores between token l and token s of the chunk
//   P[l,s] = G[l,s] · exp(a_l − a_s) · dt_s  (s ≤ l)               decay-masked, lower triangular
//   Y      = P X  +  diag(exp(a_l)) · (C S_prev)     [128 x 64]    inside-chunk part + carried state
//   S      = exp(a_end) S_prev + Bᵀ · diag(exp(a_end − a_l) dt_l) X   [128 x 64]  (state index n on rows)
// One CTA owns a (sequence, head) pair and walks its chunks in order, so the state never leaves the SM: the fp32
// master copy lives in TMEM and is updated by an accumulating MMA, a 16-bit copy in shared memory feeds the next
// chunk's C·S product.  All four products run on tcgen05 with fp32 accumulation in TMEM; the 128 compute threads
// (one per chunk row / TMEM lane) do the cumulative sum, the decay mask, the epilogue and the state rescale.
//
// Shared memory (96 KB, two CTAs per SM so that one CTA's tensor-core phases fill the other's scalar phases):
//   X [128 x 64] · B [128 x 128] · C [128 x 128] (later overwritten by P) · S_prev [128 x 64], all 16-bit, 128-byte
//   swizzled rows as TMA writes them.  TMEM (256 columns): G / then Y_intra at [0,128), S at [128,192), C·S at [192,256).
// Rows past the end of a ragged sequence get dt = 0: they add nothing to the state or to other rows and are not stored.
// Compiled shape: head_dim 64, state 128 (the Nemotron-H / Mamba2 configuration).  Every wait is bounded.
//
// Reference counterpart: the CuTe-DSL kernel kernelSrcs/ssd_cutedsl/ssd_prefill_blackwell.py (registered in
// kernelSrcs/build_cutedsl.py:367-411); semantics follow unittests/cpp/kernels/mamba/ssdCuteDslTests.cpp:178.
#include <type_traits>

#include "host_utils.h"
#include "tc5_common.cuh"

namespace telb {

constexpr int kSsdL = 128;        // chunk length
constexpr int kSsdP = 64;         // head dim
constexpr int kSsdN = 128;        // state size
constexpr int kSsdThreads = 192;

struct SsdParams {
    const void* dt;            // [T, nh]
    const float* A;            // [nh] (negative)
    const float* D;            // [nh]
    const float* dt_bias;      // [nh]
    const void* z;             // [T, nh, 64] or null
    float* state;              // [rows, nh, 64, 128] fp32
    void* y;                   // [T, nh, 64]
    const int* q_start;
    const int* q_len;
    const int* past_len;
    const int* slot_ids;
    int nheads, ngroups, dt_softplus;
    float dt_limit;
    int* status;
};

__device__ __forceinline__ float ssd_softplus(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

template <typename T>
__global__ void __launch_bounds__(kSsdThreads, 2)
ssd_chunk_scan_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_b,
                      const __grid_constant__ CUtensorMap tma_c, SsdParams p) {
    constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sX = smem;                       // 16 KB
    uint8_t* sB = sX + 16384;                 // 2 x 16 KB (state columns 0-63 | 64-127)
    uint8_t* sC = sB + 32768;                 // 2 x 16 KB; reused for P (chunk columns 0-63 | 64-127)
    uint8_t* sS = sC + 32768;                 // 16 KB
    float* sA = reinterpret_cast<float*>(sS + 16384);        // a_l * log2(e)   [128]
    float* sDt = sA + kSsdL;                                  // dt_l            [128]
    float* sWarp = sDt + kSsdL;                               // per-warp totals [4]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sWarp + 8);
    uint64_t* full_bar = bars;        // inputs of the chunk have landed (TMA)
    uint64_t* g_bar = bars + 1;       // G and C·S_prev are in TMEM
    uint64_t* p_full = bars + 2;      // P is in shared memory (128 arrivals)
    uint64_t* y_bar = bars + 3;       // P·X is in TMEM
    uint64_t* xs_full = bars + 4;     // X is rescaled, S is decayed (128 arrivals)
    uint64_t* s_bar = bars + 5;       // the state update has completed
    uint64_t* s_ready = bars + 6;     // the 16-bit state copy is in shared memory (128 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int seq = blockIdx.x / p.nheads, h = blockIdx.x - seq * p.nheads;
    const int g = h / (p.nheads / p.ngroups);

    if (threadIdx.x == 0) {
        mbar_init(full_bar, 1);
        mbar_init(g_bar, 1);
        mbar_init(p_full, 128);
        mbar_init(y_bar, 1);
        mbar_init(xs_full, 128);
        mbar_init(s_bar, 1);
        mbar_init(s_ready, 128);
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tensormap(&tma_x);
        prefetch_tensormap(&tma_b);
        prefetch_tensormap(&tma_c);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 256);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    pdl_prologue();
    const uint32_t tmem_base = *tmem_slot;
    const int ql = p.q_len[seq];
    const int t_first = p.q_start[seq];
    const int nchunks = (ql + kSsdL - 1) / kSsdL;
    constexpr uint32_t kColG = 0, kColS = 128, kColYI = 192;

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            for (int c = 0; c < nchunks; ++c) {
                // X, B are read by the state update of the previous chunk, C / P by its P·X product
                if (c > 0 && !mbar_wait(s_bar, (uint32_t)(c - 1) & 1u, abort_flag, p.status, kStatusProducerTimeout)) break;
                const int t0 = t_first + c * kSsdL;
                mbar_expect_tx(full_bar, 16384 + 32768 + 32768);
                tma_load_2d(sX, &tma_x, full_bar, h * kSsdP, t0);
                tma_load_2d(sB, &tma_b, full_bar, g * kSsdN, t0);
                tma_load_2d(sB + 16384, &tma_b, full_bar, g * kSsdN + 64, t0);
                tma_load_2d(sC, &tma_c, full_bar, g * kSsdN, t0);
                tma_load_2d(sC + 16384, &tma_c, full_bar, g * kSsdN + 64, t0);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc_g = idesc_f16(128, 128, kBf16);                 // C (K-major) x B (K-major)
            const uint32_t idesc_y = idesc_f16(128, 64, kBf16, false, true);     // K-major A x MN-major B
            const uint32_t idesc_s = idesc_f16(128, 64, kBf16, true, true);      // MN-major A (Bᵀ) x MN-major B
            for (int c = 0; c < nchunks; ++c) {
                const uint32_t par = (uint32_t)c & 1u;
                if (!mbar_wait(full_bar, par, abort_flag, p.status, kStatusMmaTimeout)) break;
                if (!mbar_wait(s_ready, par, abort_flag, p.status, kStatusMmaTimeout)) break;     // completion c: state copy of chunk c-1
                tc_fence_after_sync();
                const uint64_t dC = smem_desc_sw128(sC), dB = smem_desc_sw128(sB);
                const uint64_t dS = smem_desc_sw128_mn(sS, 0, 1024), dX = smem_desc_sw128_mn(sX, 0, 1024);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint64_t off = (uint64_t)((k >> 2) * 16384 >> 4) + 2 * (k & 3);
                    umma_f16(tmem_base + kColG, dC + off, dB + off, idesc_g, k > 0 ? 1u : 0u);
                }
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint64_t off = (uint64_t)((k >> 2) * 16384 >> 4) + 2 * (k & 3);
                    umma_f16(tmem_base + kColYI, dC + off, dS + (uint64_t)(k * 2048 >> 4), idesc_y, k > 0 ? 1u : 0u);
                }
                umma_commit(g_bar);
                if (!mbar_wait(p_full, par, abort_flag, p.status, kStatusMmaTimeout)) break;
                tc_fence_after_sync();
                const uint64_t dP = smem_desc_sw128(sC);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint64_t off = (uint64_t)((k >> 2) * 16384 >> 4) + 2 * (k & 3);
                    umma_f16(tmem_base + kColG, dP + off, dX + (uint64_t)(k * 2048 >> 4), idesc_y, k > 0 ? 1u : 0u);
                }
                umma_commit(y_bar);
                if (!mbar_wait(xs_full, par, abort_flag, p.status, kStatusMmaTimeout)) break;
                tc_fence_after_sync();
                const uint64_t dBt = smem_desc_sw128_mn(sB, 16384, 1024);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    umma_f16(tmem_base + kColS, dBt + (uint64_t)(k * 2048 >> 4), dX + (uint64_t)(k * 2048 >> 4), idesc_s, 1u);
                umma_commit(s_bar);
            }
        }
    } else {
        // ---------------- compute threads: row r of the chunk (and state row r) ----------------
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
        const float a_head = p.A[h], d_head = p.D[h], db = p.dt_bias[h];
        const T* dtp = reinterpret_cast<const T*>(p.dt);
        const T* zp = reinterpret_cast<const T*>(p.z);
        T* yp = reinterpret_cast<T*>(p.y);
        float* st = p.state + ((size_t)p.slot_ids[seq] * p.nheads + h) * (size_t)(kSsdP * kSsdN);
        uint8_t* srow = sS + (r >> 3) * 1024 + (r & 7) * 128;
        uint8_t* xrow = sX + (r >> 3) * 1024 + (r & 7) * 128;
        bool ok = nchunks > 0;
        // initial state: TMEM master copy (fp32) and the 16-bit copy the first C·S product reads
        if (ok) {
            const bool fresh = p.past_len[seq] <= 0;
#pragma unroll 1
            for (int c8 = 0; c8 < 8; ++c8) {
                uint32_t v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = fresh ? 0u : __float_as_uint(st[(size_t)(c8 * 8 + i) * kSsdN + r]);
                tmem_st_x8(lane_addr + kColS + c8 * 8, v);
                uint4 u;
                u.x = Cvt<T>::pack2(__uint_as_float(v[0]), __uint_as_float(v[1]));
                u.y = Cvt<T>::pack2(__uint_as_float(v[2]), __uint_as_float(v[3]));
                u.z = Cvt<T>::pack2(__uint_as_float(v[4]), __uint_as_float(v[5]));
                u.w = Cvt<T>::pack2(__uint_as_float(v[6]), __uint_as_float(v[7]));
                *reinterpret_cast<uint4*>(srow + ((c8 ^ (r & 7)) << 4)) = u;
            }
            tmem_st_wait();
            tc_fence_before_sync();
            fence_proxy_async_smem();
            mbar_arrive(s_ready);
        }
        for (int c = 0; c < nchunks && ok; ++c) {
            const uint32_t par = (uint32_t)c & 1u;
            const int len = min(kSsdL, ql - c * kSsdL);
            const size_t t = (size_t)t_first + (size_t)c * kSsdL + r;
            const bool valid = r < len;
            // ---- dt, cumulative decay exponent (base-2) ----
            float d = 0.f;
            if (valid) {
                d = Cvt<T>::to_f(dtp[t * p.nheads + h]) + db;
                if (p.dt_softplus) d = ssd_softplus(d);
                if (p.dt_limit > 0.f) d = fminf(d, p.dt_limit);
            }
            float a = a_head * d * 1.4426950408889634f;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float n = __shfl_up_sync(0xffffffffu, a, o);
                if (lane >= o) a += n;
            }
            named_barrier_sync(1, 128);                    // the previous chunk's readers of sA / sDt / sWarp are done
            if (lane == 31) sWarp[quad] = a;
            named_barrier_sync(1, 128);
            for (int w = 0; w < quad; ++w) a += sWarp[w];
            sA[r] = a;
            sDt[r] = d;
            named_barrier_sync(1, 128);
            const float a_end = sA[kSsdL - 1];
            // ---- P = G ∘ decay mask, written over C ----
            if (!mbar_wait(g_bar, par, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
            tc_fence_after_sync();
#pragma unroll 1
            for (int cc = 0; cc < 4; ++cc) {                // 32 chunk columns at a time
                uint32_t gr[32];
                tmem_ld_x32(lane_addr + kColG + cc * 32, gr);
                tmem_ld_wait();
                uint8_t* prow = sC + (cc >> 1) * 16384 + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float e[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int s = cc * 32 + q * 8 + i;
                        e[i] = s <= r ? __uint_as_float(gr[q * 8 + i]) * exp2f(a - sA[s]) * sDt[s] : 0.f;
                    }
                    uint4 u;
                    u.x = Cvt<T>::pack2(e[0], e[1]);
                    u.y = Cvt<T>::pack2(e[2], e[3]);
                    u.z = Cvt<T>::pack2(e[4], e[5]);
                    u.w = Cvt<T>::pack2(e[6], e[7]);
                    const int chunk16 = (cc & 1) * 4 + q;
                    *reinterpret_cast<uint4*>(prow + ((chunk16 ^ (r & 7)) << 4)) = u;
                }
            }
            tc_fence_before_sync();
            fence_proxy_async_smem();
            mbar_arrive(p_full);
            // ---- y = P X + exp(a) (C S_prev) + D x, gated, stored; then X ← X · exp(a_end − a) dt ----
            if (!mbar_wait(y_bar, par, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
            tc_fence_after_sync();
            const float ea = exp2f(a);
            const float wgt = exp2f(a_end - a) * d;
#pragma unroll 1
            for (int c8 = 0; c8 < 8; ++c8) {
                uint32_t ya[8], yi[8];
                tmem_ld_x8(lane_addr + kColG + c8 * 8, ya);
                tmem_ld_x8(lane_addr + kColYI + c8 * 8, yi);
                tmem_ld_wait();
                uint4* xp = reinterpret_cast<uint4*>(xrow + ((c8 ^ (r & 7)) << 4));
                uint4 xu = *xp;
                const T* xe = reinterpret_cast<const T*>(&xu);
                float xv[8], o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    xv[i] = Cvt<T>::to_f(xe[i]);
                    o[i] = __uint_as_float(ya[i]) + ea * __uint_as_float(yi[i]) + d_head * xv[i];
                }
                if (valid) {
                    if (zp) {
                        const uint4 zu = *reinterpret_cast<const uint4*>(zp + (t * p.nheads + h) * kSsdP + c8 * 8);
                        const T* ze = reinterpret_cast<const T*>(&zu);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float zf = Cvt<T>::to_f(ze[i]);
                            o[i] *= zf / (1.f + __expf(-zf));
                        }
                    }
                    uint4 u;
                    u.x = Cvt<T>::pack2(o[0], o[1]);
                    u.y = Cvt<T>::pack2(o[2], o[3]);
                    u.z = Cvt<T>::pack2(o[4], o[5]);
                    u.w = Cvt<T>::pack2(o[6], o[7]);
                    *reinterpret_cast<uint4*>(yp + (t * p.nheads + h) * kSsdP + c8 * 8) = u;
                }
                uint4 xs;
                xs.x = Cvt<T>::pack2(xv[0] * wgt, xv[1] * wgt);
                xs.y = Cvt<T>::pack2(xv[2] * wgt, xv[3] * wgt);
                xs.z = Cvt<T>::pack2(xv[4] * wgt, xv[5] * wgt);
                xs.w = Cvt<T>::pack2(xv[6] * wgt, xv[7] * wgt);
                *xp = xs;
            }
            // ---- S ← exp(a_end) S (row r of the state), before the accumulating state update ----
            {
                const float dec = exp2f(a_end);
#pragma unroll 1
                for (int c16 = 0; c16 < 4; ++c16) {
                    uint32_t v[16];
                    tmem_ld_x16(lane_addr + kColS + c16 * 16, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * dec);
                    tmem_st_x16(lane_addr + kColS + c16 * 16, v);
                }
                tmem_st_wait();
            }
            tc_fence_before_sync();
            fence_proxy_async_smem();
            mbar_arrive(xs_full);
            // ---- new state: 16-bit copy for the next chunk, fp32 to the pool after the last chunk ----
            if (!mbar_wait(s_bar, par, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
            tc_fence_after_sync();
            const bool last = c == nchunks - 1;
#pragma unroll 1
            for (int c8 = 0; c8 < 8; ++c8) {
                uint32_t v[8];
                tmem_ld_x8(lane_addr + kColS + c8 * 8, v);
                tmem_ld_wait();
                if (last) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) st[(size_t)(c8 * 8 + i) * kSsdN + r] = __uint_as_float(v[i]);
                } else {
                    uint4 u;
                    u.x = Cvt<T>::pack2(__uint_as_float(v[0]), __uint_as_float(v[1]));
                    u.y = Cvt<T>::pack2(__uint_as_float(v[2]), __uint_as_float(v[3]));
                    u.z = Cvt<T>::pack2(__uint_as_float(v[4]), __uint_as_float(v[5]));
                    u.w = Cvt<T>::pack2(__uint_as_float(v[6]), __uint_as_float(v[7]));
                    *reinterpret_cast<uint4*>(srow + ((c8 ^ (r & 7)) << 4)) = u;
                }
            }
            if (!last) {
                tc_fence_before_sync();
                fence_proxy_async_smem();
                mbar_arrive(s_ready);
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
        tmem_dealloc(tmem_base, 256);
    }
}

}  // namespace telb

using namespace telb;

// Mamba2 chunked prefill scan (see the top of the file).  x [T, nh, 64], dt [T, nh], B / C [T, ngroups, 128] 16-bit,
// A / D / dt_bias [nh] fp32, z [T, nh, 64] or null, state [rows, nh, 64, 128] fp32 (read when past_len > 0, always
// written), y [T, nh, 64].  One CTA per (sequence, head).
extern "C" int telb_ssd_chunk_scan(const void* x, const void* dt, const float* A, const void* B, const void* C, const float* D,
                                   const float* dt_bias, const void* z, float* state, void* y, const int* q_start, const int* q_len,
                                   const int* past_len, const int* slot_ids, int num_seqs, int total_tokens, int nheads, int head_dim,
                                   int d_state, int ngroups, int dt_softplus, float dt_limit, int is_bf16, int* status,
                                   cudaStream_t stream) {
    if (num_seqs <= 0 || total_tokens <= 0) return 0;
    if (head_dim != kSsdP || d_state != kSsdN) return fail("telb_ssd_chunk_scan: head_dim 64 and d_state 128 are the compiled shape");
    if (ngroups <= 0 || nheads % ngroups) return fail("telb_ssd_chunk_scan: heads must divide evenly into groups");
    const CUtensorMapDataType dtp = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap tx, tb, tc;
    if (make_tmap_2d(&tx, dtp, 2, x, total_tokens, (uint64_t)nheads * kSsdP, (uint64_t)nheads * kSsdP * 2, kSsdL, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    if (make_tmap_2d(&tb, dtp, 2, B, total_tokens, (uint64_t)ngroups * kSsdN, (uint64_t)ngroups * kSsdN * 2, kSsdL, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    if (make_tmap_2d(&tc, dtp, 2, C, total_tokens, (uint64_t)ngroups * kSsdN, (uint64_t)ngroups * kSsdN * 2, kSsdL, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    SsdParams p{};
    p.dt = dt;
    p.A = A;
    p.D = D;
    p.dt_bias = dt_bias;
    p.z = z;
    p.state = state;
    p.y = y;
    p.q_start = q_start;
    p.q_len = q_len;
    p.past_len = past_len;
    p.slot_ids = slot_ids;
    p.nheads = nheads;
    p.ngroups = ngroups;
    p.dt_softplus = dt_softplus;
    p.dt_limit = dt_limit;
    p.status = status;
    constexpr int smem = 16384 + 32768 + 32768 + 16384 + (2 * kSsdL + 8) * 4 + 128 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(ssd_chunk_scan_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(ssd_chunk_scan_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail("cudaFuncSetAttribute(ssd_chunk_scan)", e);
        configured = true;
    }
    const dim3 grid(num_seqs * nheads), block(kSsdThreads);
    if (is_bf16) TELB_LAUNCH("ssd_chunk_scan_kernel", (ssd_chunk_scan_kernel<__nv_bfloat16>), grid, block, smem, stream, tx, tb, tc, p);
    else TELB_LAUNCH("ssd_chunk_scan_kernel", (ssd_chunk_scan_kernel<__half>), grid, block, smem, stream, tx, tb, tc, p);
    TELB_CHECK_LAUNCH("ssd_chunk_scan_kernel");
    return 0;
}
