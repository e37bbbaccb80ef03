// Paged GQA attention on tcgen05: one kernel family for prefill chunks, decode rows and
// speculative tree verification.
//
// A CTA owns (sequence, KV head, 128-row query tile, KV split).  The 128 MMA rows stack the G
// query heads that share the KV head on top of 128/G consecutive query tokens (row = token*G + g),
// so a decode step (1 token) and a 60-token verification tree use the same tile shape as a
// prefill chunk and every K/V page is fetched once per KV head, not once per query head.
//   S = Q Kᵀ   tcgen05.mma, Q and K tiles in 128B-swizzled shared memory (TMA), S in TMEM (2 buffers)
//   softmax    4 warps, one row per thread, online max/sum with lazy rescaling of O (only when the
//              running max grows by more than 2^8), probabilities written to shared memory as bf16
//   O += P V   tcgen05.mma with V as an MN-major operand straight from the paged pool
// KV pages are 64 tokens (or 128, consumed as two 64-token tiles); the cache layer layout is
// [pages, 2, Hkv, P, D] so a (page, K|V, head) tile is one contiguous box for TMA.
// With `splits > 1` (decode at small batch) each split writes a normalised fp32 partial and its
// log-sum-exp to a workspace and `attn_combine_kernel` merges them.
//
// Roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer / TMEM owner, warps 2-5 softmax.
// All waits are bounded (tc5_common.cuh).
//
// Reference counterparts: CuTe-DSL FMHA (kernelSrcs/fmha_cutedsl_blackwell/fmha.py), CTM decode
// (kernelSrcs/fmha_decode_ctm/fmha_decode.py) and XQA (kernelSrcs/xqa/mha.cu); semantics follow
// unittests/support/references.h:29-37 (bottom-right aligned causal mask, GQA, sliding window).
#include <type_traits>

#include "host_utils.h"
#include "nvfp4_common.cuh"
#include "tc5_common.cuh"

namespace telb {

struct AttnParams {
    void* out;                 // [T, Hq, D] 16-bit
    float* ws_o;               // [splits, T, Hq, D] fp32 (splits > 1)
    float* ws_lse;             // [splits, T, Hq]    log2-domain log-sum-exp
    const int* q_start;        // [N+1]
    const int* q_len;          // [N]
    const int* past_len;       // [N]
    const int* page_table;     // [N, max_pages]
    const int* tree_mask;      // [T, mask_words] or null
    int mask_words;
    int max_pages, page_size;
    int hq, hkv, group;        // group = hq / hkv
    int tq;                    // query tokens per tile = 128 / group
    int splits;
    int total_tokens;
    int window;                // sliding window, 0 = none, -1 = no causal mask (every row sees every cached and new token)
    float scale_log2;          // softmax scale * log2(e)
    const float* sinks;        // [Hq] fp32 per-head sink logits (natural-log units) joining every row's softmax denominator, or null
    // Skip-softmax (BLASST tile vote): skip_thr[seq] = log2(lambda) of the sequence (lambda = S / length, -inf = dense), or null.
    // A KV tile whose largest score lies more than that below the running maximum for every query row of a warp is not
    // exponentiated (its P rows are zeros); when all four warps vote so, the tile's P·V products are not issued either.
    const float* skip_thr;
    int* skip_stats;           // optional [2]: tiles processed, tiles whose P·V was skipped (diagnostics / tests), or null
    int out_bf16;
    int* status;
};

constexpr int kAttnThreads = 192;
constexpr int kKvTile = 64;
constexpr float kRescaleThreshold = 8.0f;   // log2 units

__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// KVS: depth of the K and V tile rings; MINB: CTAs resident per SM.  Two resident CTAs with single-stage rings let
// one CTA's MMAs run under the other's softmax; one CTA with deep rings prefetches further ahead.
template <int D, typename T, int KVS, int MINB>
__global__ void __launch_bounds__(kAttnThreads, MINB)
attn_tc5_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_kv, AttnParams p) {
    constexpr int kDChunks = D / 64;
    constexpr int kQBytes = 128 * D * 2;
    constexpr int kKvBytes = kKvTile * D * 2;            // one K or V tile
    constexpr int kPBytes = 128 * kKvTile * 2;
    constexpr int kTmemCols = D <= 128 ? 256 : 512;      // S0 | S1 | O (D columns)
    constexpr uint32_t kOCol = 128;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* s_q = smem;
    uint8_t* s_k = s_q + kQBytes;
    uint8_t* s_v = s_k + KVS * kKvBytes;
    uint8_t* s_p = s_v + KVS * kKvBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_p + 2 * kPBytes);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;
    uint64_t* k_empty = k_full + KVS;
    uint64_t* v_full = k_empty + KVS;
    uint64_t* v_empty = v_full + KVS;
    uint64_t* s_full = v_empty + KVS;
    uint64_t* s_free = s_full + 2;
    uint64_t* p_full = s_free + 2;
    uint64_t* p_free = p_full + 2;
    uint64_t* o_bar = p_free + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_bar + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* s_keep = tmem_slot + 4;           // [2 P buffers][4 warps]: the warp computed probabilities for the tile

    pdl_prologue();          // step metadata and Q/KV are produced by earlier kernels
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int qt = blockIdx.x;
    const int kvh = blockIdx.y;
    const int seq = blockIdx.z / p.splits;
    const int split = blockIdx.z - seq * p.splits;

    const int qlen = p.q_len[seq];
    const int past = p.past_len[seq];
    const int qrow0 = p.q_start[seq];
    const int tok0 = qt * p.tq;                          // first query token of this tile (within the sequence)
    if (tok0 >= qlen) return;                            // uniform per CTA, before any barrier / TMEM use

    // KV tile range of this CTA
    int kv_end = past + ((p.tree_mask || p.window < 0) ? qlen : min(qlen, tok0 + p.tq));
    int tile_lo = 0;
    if (p.window > 0) tile_lo = max(0, past + tok0 - p.window + 1) / kKvTile;
    const int tile_hi_all = (kv_end + kKvTile - 1) / kKvTile;
    const int per = (tile_hi_all - tile_lo + p.splits - 1) / p.splits;
    const int j0 = tile_lo + split * per;
    const int j1 = min(tile_hi_all, j0 + per);
    const int ntiles = max(0, j1 - j0);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < KVS; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&s_full[s], 1);
            mbar_init(&s_free[s], 128);
            mbar_init(&p_full[s], 128);
            mbar_init(&p_free[s], 1);
        }
        mbar_init(o_bar, 1);
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tensormap(&tma_q);
        prefetch_tensormap(&tma_kv);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------ producer ------------------------------
        if (lane == 0 && ntiles > 0) {
            mbar_expect_tx(q_full, kQBytes);
#pragma unroll
            for (int c = 0; c < kDChunks; ++c)
                tma_load_3d(s_q + c * (128 * 128), &tma_q, q_full, c * 64, kvh * p.group, qrow0 + tok0);
            const int tiles_per_page = p.page_size / kKvTile;
            for (int j = 0; j < ntiles; ++j) {
                const int stage = j % KVS;
                const uint32_t ph = ((j / KVS) & 1) ^ 1;
                const int tile = j0 + j;
                int page = p.page_table[(size_t)seq * p.max_pages + tile / tiles_per_page];
                if (page < 0) page = 0;              // unreserved page: read page 0, the mask hides it
                const int row_k = ((page * 2 + 0) * p.hkv + kvh) * p.page_size + (tile % tiles_per_page) * kKvTile;
                const int row_v = row_k + p.hkv * p.page_size;
                if (!mbar_wait(&k_empty[stage], ph, abort_flag, p.status, kStatusProducerTimeout)) break;
                mbar_expect_tx(&k_full[stage], kKvBytes);
#pragma unroll
                for (int c = 0; c < kDChunks; ++c)
                    tma_load_2d(s_k + stage * kKvBytes + c * (kKvTile * 128), &tma_kv, &k_full[stage], c * 64, row_k);
                if (!mbar_wait(&v_empty[stage], ph, abort_flag, p.status, kStatusProducerTimeout)) break;
                mbar_expect_tx(&v_full[stage], kKvBytes);
#pragma unroll
                for (int c = 0; c < kDChunks; ++c)
                    tma_load_2d(s_v + stage * kKvBytes + c * (kKvTile * 128), &tma_kv, &v_full[stage], c * 64, row_v);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0 && ntiles > 0) {
            constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
            const uint32_t idesc_s = idesc_f16(128, kKvTile, kBf16);
            const uint32_t idesc_o = idesc_f16(128, D, kBf16, false, true);
            auto issue_s = [&](int j) {
                const int stage = j % KVS;
                const uint64_t dq = smem_desc_sw128(s_q);
                const uint64_t dk = smem_desc_sw128(s_k + stage * kKvBytes);
                const uint32_t d_tmem = tmem_base + (j & 1) * kKvTile;
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const int c = k >> 2, kk = k & 3;
                    umma_f16(d_tmem, dq + (uint64_t)(c * (128 * 128) >> 4) + 2 * kk,
                             dk + (uint64_t)(c * (kKvTile * 128) >> 4) + 2 * kk, idesc_s, k > 0 ? 1u : 0u);
                }
                umma_commit(&k_empty[stage]);
                umma_commit(&s_full[j & 1]);
            };
            bool o_started = false;                      // the first P·V issued overwrites the accumulator
            bool ok = mbar_wait(q_full, 0, abort_flag, p.status, kStatusMmaTimeout);
            ok = ok && mbar_wait(&k_full[0], 0, abort_flag, p.status, kStatusMmaTimeout);
            if (ok) {
                tc_fence_after_sync();
                issue_s(0);
            }
            for (int j = 0; j < ntiles && ok; ++j) {
                if (j + 1 < ntiles) {
                    const int jn = j + 1;
                    ok = mbar_wait(&k_full[jn % KVS], (jn / KVS) & 1, abort_flag, p.status, kStatusMmaTimeout) &&
                         mbar_wait(&s_free[jn & 1], ((jn >> 1) & 1) ^ 1, abort_flag, p.status, kStatusMmaTimeout);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_s(jn);
                }
                const int stage = j % KVS;
                ok = mbar_wait(&p_full[j & 1], (j >> 1) & 1, abort_flag, p.status, kStatusMmaTimeout) &&
                     mbar_wait(&v_full[stage], (j / KVS) & 1, abort_flag, p.status, kStatusMmaTimeout);
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t dp = smem_desc_sw128(s_p + (j & 1) * kPBytes);
                const uint64_t dv = smem_desc_sw128_mn(s_v + stage * kKvBytes, kKvTile * 128, 1024);
                const volatile uint32_t* kf = s_keep + (j & 1) * 4;
                const bool keep = !p.skip_thr || (kf[0] | kf[1] | kf[2] | kf[3]) != 0;
                if (keep) {
#pragma unroll
                    for (int k = 0; k < kKvTile / 16; ++k)
                        umma_f16(tmem_base + kOCol, dp + 2 * k, dv + (uint64_t)(k * 2048 >> 4), idesc_o, (o_started || k > 0) ? 1u : 0u);
                    o_started = true;
                }
                if (p.skip_stats && (threadIdx.x & 31) == 0) {
                    atomicAdd(&p.skip_stats[0], 1);
                    if (!keep) atomicAdd(&p.skip_stats[1], 1);
                }
                umma_commit(&v_empty[stage]);
                umma_commit(&p_free[j & 1]);
                umma_commit(o_bar);
            }
        }
    } else {
        // ------------------------------ softmax / epilogue ------------------------------
        const int quad = warp & 3;
        const int r = quad * 32 + lane;                 // MMA row == TMEM lane
        const int ti = r / p.group;                     // token within the tile
        const int g = r - ti * p.group;
        const int qi = tok0 + ti;                       // token within the sequence
        const bool row_valid = qi < qlen;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
        const int* mask_row = p.tree_mask ? p.tree_mask + (size_t)(qrow0 + min(qi, qlen - 1)) * p.mask_words : nullptr;
        const int causal_limit = past + qi;             // last visible cache slot
        float m_used = -INFINITY, l_sum = 0.f;
        const float skip_thr = p.skip_thr ? p.skip_thr[seq] : -INFINITY;
        bool ok = true;
        for (int j = 0; j < ntiles && ok; ++j) {
            const int b = j & 1;
            if (!mbar_wait(&s_full[b], (j >> 1) & 1, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
            tc_fence_after_sync();
            float s[kKvTile];
            {
                uint32_t r0[32], r1[32];
                tmem_ld_x32(lane_addr + b * kKvTile, r0);
                tmem_ld_x32(lane_addr + b * kKvTile + 32, r1);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    s[i] = __uint_as_float(r0[i]);
                    s[32 + i] = __uint_as_float(r1[i]);
                }
            }
            tc_fence_before_sync();
            mbar_arrive(&s_free[b]);
            const int c0 = (j0 + j) * kKvTile;
            float mx = -INFINITY;
            // Tiles that lie wholly below the causal diagonal of this query tile need no mask at all (most tiles of a
            // long prompt): scale and take the maximum only.
            const bool unmasked_tile = !mask_row && p.window == 0 && (c0 + kKvTile - 1 <= past + tok0);
            if (row_valid && unmasked_tile) {
#pragma unroll
                for (int i = 0; i < kKvTile; ++i) {
                    s[i] *= p.scale_log2;
                    mx = fmaxf(mx, s[i]);
                }
            } else if (row_valid) {
#pragma unroll
                for (int i = 0; i < kKvTile; ++i) {
                    const int c = c0 + i;
                    bool vis;
                    if (mask_row) {
                        const int nc = c - past;
                        vis = c < past || (nc < qlen && ((mask_row[nc >> 5] >> (nc & 31)) & 1));
                    } else if (p.window < 0) {
                        vis = c < past + qlen;                      // bidirectional (vision / audio encoders)
                    } else {
                        vis = c <= causal_limit;
                    }
                    if (p.window > 0) vis = vis && (c > causal_limit - p.window);
                    s[i] = vis ? s[i] * p.scale_log2 : -INFINITY;
                    mx = fmaxf(mx, s[i]);
                }
            }
            const float m_new = fmaxf(m_used, mx);
            // tile vote of this warp: a row keeps the tile when its best score is within the threshold of the running
            // maximum (a tile that raises the maximum always is); rows of a warp that all vote "skip" write zero probabilities
            const bool warp_keep = __any_sync(0xffffffffu, row_valid && (mx - m_new >= skip_thr));
            const bool need = warp_keep && row_valid && (m_new > m_used + kRescaleThreshold);
            // P buffer b is free once P·V of tile j-2 has completed; this wait is taken at every use of the buffer, so
            // its parity is exact (a barrier polled only now and then could be two phases ahead and alias).
            if (!mbar_wait(&p_free[b], ((j >> 1) & 1) ^ 1, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
            if (j == 0) {
                if (row_valid) m_used = m_new;
            } else if (__any_sync(0xffffffffu, need)) {
                // O must be quiescent: P·V of tile j-1 is the next completion of the other buffer's barrier
                if (!mbar_wait(&p_free[b ^ 1], ((j - 1) >> 1) & 1, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
                tc_fence_after_sync();
                const float f = need ? exp2f(m_used - m_new) : 1.f;
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld_x32(lane_addr + kOCol + c * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = f == 0.f ? 0u : __float_as_uint(__uint_as_float(o[i]) * f);   // 0: nothing accumulated yet
                    tmem_st_x32(lane_addr + kOCol + c * 32, o);
                }
                tmem_st_wait();
                tc_fence_before_sync();
                if (need) {
                    l_sum *= f;
                    m_used = m_new;
                }
            }
            uint8_t* prow = s_p + b * kPBytes + (r >> 3) * 1024 + (r & 7) * 128;
            if (lane == 0) s_keep[b * 4 + quad] = warp_keep ? 1u : 0u;      // published by the arrive on p_full below
            if (row_valid && warp_keep) {
                const float mref = m_used == -INFINITY ? 0.f : m_used;
                float acc = 0.f;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    float e[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        e[i] = exp2f(s[c * 8 + i] - mref);
                        acc += e[i];
                    }
                    uint4 u;
                    u.x = Cvt<T>::pack2(e[0], e[1]);
                    u.y = Cvt<T>::pack2(e[2], e[3]);
                    u.z = Cvt<T>::pack2(e[4], e[5]);
                    u.w = Cvt<T>::pack2(e[6], e[7]);
                    *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = u;
                }
                l_sum += acc;
            } else {
#pragma unroll
                for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(prow + (c << 4)) = make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async_smem();
            mbar_arrive(&p_full[b]);
        }
        // ---- epilogue ----
        // commits complete in issue order: the last tile's completion covers every earlier P·V
        if (ok && ntiles > 0)
            ok = mbar_wait(&p_free[(ntiles - 1) & 1], ((ntiles - 1) >> 1) & 1, abort_flag, p.status, kStatusEpilogueTimeout);
        if (ok) {
            tc_fence_after_sync();
            const size_t tok = (size_t)qrow0 + qi;
            const int head = kvh * p.group + g;
            float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
            float lse = l_sum > 0.f ? m_used + log2f(l_sum) : -INFINITY;
            if (p.sinks != nullptr && split == 0 && row_valid) {
                // the sink is one more logit with no value row: it only grows the denominator (first split only)
                const float z = p.sinks[head] * 1.44269504f;
                if (l_sum > 0.f) {
                    const float m2 = fmaxf(m_used, z);
                    const float os = exp2f(m_used - m2);
                    const float l2 = l_sum * os + exp2f(z - m2);
                    inv = os / l2;
                    lse = m2 + log2f(l2);
                } else {
                    lse = z;
                }
            }
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                float v[32];
                if (ntiles > 0) {
                    uint32_t o[32];
                    tmem_ld_x32(lane_addr + kOCol + c * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = inv > 0.f ? __uint_as_float(o[i]) * inv : 0.f;
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0.f;
                }
                if (!row_valid) continue;
                if (p.splits == 1) {
                    T* dst = reinterpret_cast<T*>(p.out) + (tok * p.hq + head) * D + c * 32;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint4 u;
                        u.x = Cvt<T>::pack2(v[q * 8 + 0], v[q * 8 + 1]);
                        u.y = Cvt<T>::pack2(v[q * 8 + 2], v[q * 8 + 3]);
                        u.z = Cvt<T>::pack2(v[q * 8 + 4], v[q * 8 + 5]);
                        u.w = Cvt<T>::pack2(v[q * 8 + 6], v[q * 8 + 7]);
                        reinterpret_cast<uint4*>(dst)[q] = u;
                    }
                } else {
                    float* dst = p.ws_o + (((size_t)split * p.total_tokens + tok) * p.hq + head) * D + c * 32;
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        reinterpret_cast<float4*>(dst)[q] = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
                }
            }
            if (row_valid && p.splits > 1)
                p.ws_lse[((size_t)split * p.total_tokens + tok) * p.hq + head] = lse;
            tc_fence_before_sync();
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
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// Merge split partials: out = Σ_s 2^(lse_s - max) O_s / Σ_s 2^(lse_s - max).
// One CTA of D threads per (token, head); splits (<= 32) are weighted by lanes of warp 0 first so
// the D-wide accumulation issues all of its loads independently.
template <int D, typename T>
__global__ void attn_combine_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_lse, T* __restrict__ out,
                                    int total_rows /* T*Hq */, int splits) {
    pdl_prologue();
    __shared__ float w[32];
    const int row = blockIdx.x;
    const int d = threadIdx.x;
    if (threadIdx.x < 32) {
        const float l = threadIdx.x < splits ? ws_lse[(size_t)threadIdx.x * total_rows + row] : -INFINITY;
        float mx = l;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float e = (l == -INFINITY) ? 0.f : exp2f(l - mx);
        float den = e;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        w[threadIdx.x] = den > 0.f ? e / den : 0.f;
    }
    __syncthreads();
    float acc = 0.f;
#pragma unroll 8
    for (int s = 0; s < splits; ++s) acc += w[s] * __ldcg(&ws_o[((size_t)s * total_rows + row) * D + d]);
    out[(size_t)row * D + d] = Cvt<T>::from_f(acc);
}

// The same merge with the result written as NVFP4 (input of the output projection): thread d of row (token, head) holds
// output dim d, so a 16-element block is 16 consecutive lanes.
template <int D, typename T>
__global__ void attn_combine_quant_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_lse, uint8_t* __restrict__ oq,
                                          uint8_t* __restrict__ osf, const float* __restrict__ ogs, int total_rows /* T*Hq */, int hq,
                                          int splits, int k64) {
    pdl_prologue();
    __shared__ float w[32];
    const int row = blockIdx.x;
    const int d = threadIdx.x;
    if (threadIdx.x < 32) {
        const float l = threadIdx.x < splits ? ws_lse[(size_t)threadIdx.x * total_rows + row] : -INFINITY;
        float mx = l;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float e = (l == -INFINITY) ? 0.f : exp2f(l - mx);
        float den = e;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        w[threadIdx.x] = den > 0.f ? e / den : 0.f;
    }
    __syncthreads();
    float acc = 0.f;
#pragma unroll 8
    for (int s = 0; s < splits; ++s) acc += w[s] * __ldcg(&ws_o[((size_t)s * total_rows + row) * D + d]);
    const float gs = *ogs;
    uint8_t s8;
    const uint32_t w4 = nvfp4_quantize_lane16(Cvt<T>::to_f(Cvt<T>::from_f(acc)), gs, 1.f / gs, s8);
    const int tok = row / hq, head = row - tok * hq;
    const int col = head * D + d;
    if ((d & 7) == 0) *reinterpret_cast<uint32_t*>(oq + (size_t)tok * (hq * D / 2) + col / 2) = w4;
    if ((d & 15) == 0) osf[sf_atom_offset((long long)tok, col >> 4, k64)] = s8;
}

template <int D, typename T, int KVS, int MINB>
static int launch_attn_variant(const CUtensorMap& tq, const CUtensorMap& tkv, const AttnParams& p, int qtiles, int nseq,
                               cudaStream_t stream) {
    constexpr int smem = 128 * D * 2 + 2 * KVS * kKvTile * D * 2 + 2 * 128 * kKvTile * 2 + 1024 + 512;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc5_kernel<D, T, KVS, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail("cudaFuncSetAttribute(attn_tc5)", e);
        configured = true;
    }
    dim3 grid(qtiles, p.hkv, nseq * p.splits);
    TELB_LAUNCH("attn_tc5_kernel", (attn_tc5_kernel<D, T, KVS, MINB>), dim3(grid), dim3(kAttnThreads), smem, stream, tq, tkv, p);
    TELB_CHECK_LAUNCH("attn_tc5_kernel");
    if (p.splits > 1) {
        const int rows = p.total_tokens * p.hq;
        TELB_LAUNCH("attn_combine_kernel", (attn_combine_kernel<D, T>), dim3(rows), dim3(D), 0, stream, p.ws_o, p.ws_lse, reinterpret_cast<T*>(p.out), rows, p.splits);
        TELB_CHECK_LAUNCH("attn_combine_kernel");
    }
    return 0;
}

static int g_attn_variant = 1;       // measured 4-8 % faster than the deep-ring variant on prefill shapes

template <int D, typename T>
static int launch_attn(const CUtensorMap& tq, const CUtensorMap& tkv, const AttnParams& p, int qtiles, int nseq, cudaStream_t stream) {
    // 256-wide heads (Gemma family): the Q tile alone is 64 KB and O takes 256 TMEM columns, so one CTA per SM with
    // single-stage K / V rings is the only shape that fits
    if constexpr (D > 128) return launch_attn_variant<D, T, 1, 1>(tq, tkv, p, qtiles, nseq, stream);
    if (g_attn_variant == 1) return launch_attn_variant<D, T, 1, 2>(tq, tkv, p, qtiles, nseq, stream);     // 2 CTAs / SM, single-stage rings
    return launch_attn_variant<D, T, 4, 1>(tq, tkv, p, qtiles, nseq, stream);                              // 1 CTA / SM, four-stage rings
}

}  // namespace telb

using namespace telb;

// Ring depth / residency variant of the tile attention kernel (0 or 1: see launch_attn); process-wide.
extern "C" int telb_set_attn_variant(int v) {
    if (v < 0 || v > 1) return fail("telb_set_attn_variant: variant must be 0 or 1");
    g_attn_variant = v;
    return 0;
}

// Merge `splits` partial results (ws_o [splits, rows, d] fp32, ws_lse [splits, rows]) into out [rows, d].
extern "C" int telb_attn_combine(const float* ws_o, const float* ws_lse, void* out, int rows, int splits, int d, int is_bf16,
                                 cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (d == 128) {
        if (is_bf16) TELB_LAUNCH("attn_combine_kernel", (attn_combine_kernel<128, __nv_bfloat16>), dim3(rows), dim3(128), 0, stream, ws_o, ws_lse, (__nv_bfloat16*)out, rows, splits);
        else TELB_LAUNCH("attn_combine_kernel", (attn_combine_kernel<128, __half>), dim3(rows), dim3(128), 0, stream, ws_o, ws_lse, (__half*)out, rows, splits);
    } else if (d == 64) {
        if (is_bf16) TELB_LAUNCH("attn_combine_kernel", (attn_combine_kernel<64, __nv_bfloat16>), dim3(rows), dim3(64), 0, stream, ws_o, ws_lse, (__nv_bfloat16*)out, rows, splits);
        else TELB_LAUNCH("attn_combine_kernel", (attn_combine_kernel<64, __half>), dim3(rows), dim3(64), 0, stream, ws_o, ws_lse, (__half*)out, rows, splits);
    } else if (d == 256) {
        if (is_bf16) TELB_LAUNCH("attn_combine_kernel", (attn_combine_kernel<256, __nv_bfloat16>), dim3(rows), dim3(256), 0, stream, ws_o, ws_lse, (__nv_bfloat16*)out, rows, splits);
        else TELB_LAUNCH("attn_combine_kernel", (attn_combine_kernel<256, __half>), dim3(rows), dim3(256), 0, stream, ws_o, ws_lse, (__half*)out, rows, splits);
    } else {
        return fail("telb_attn_combine: head_dim must be 64, 128 or 256");
    }
    TELB_CHECK_LAUNCH("attn_combine_kernel");
    return 0;
}

extern "C" int telb_nvfp4_k64_pad(int k);

// The merge with an NVFP4 result: packed codes oq [tokens, hq * d / 2] and atom-layout scales osf over hq * d columns.
extern "C" int telb_attn_combine_quant(const float* ws_o, const float* ws_lse, void* oq, void* osf, const float* ogs, int tokens, int hq,
                                       int splits, int d, int is_bf16, cudaStream_t stream) {
    const int rows = tokens * hq;
    if (rows <= 0) return 0;
    if (d != 128) return fail("telb_attn_combine_quant: head_dim must be 128");
    if (splits > 32) return fail("telb_attn_combine_quant: at most 32 splits");
    const int k64 = telb_nvfp4_k64_pad(hq * d);
    if (is_bf16) TELB_LAUNCH("attn_combine_quant_kernel", (attn_combine_quant_kernel<128, __nv_bfloat16>), dim3(rows), dim3(128), 0, stream, ws_o, ws_lse, (uint8_t*)oq, (uint8_t*)osf, ogs, rows, hq, splits, k64);
    else TELB_LAUNCH("attn_combine_quant_kernel", (attn_combine_quant_kernel<128, __half>), dim3(rows), dim3(128), 0, stream, ws_o, ws_lse, (uint8_t*)oq, (uint8_t*)osf, ogs, rows, hq, splits, k64);
    TELB_CHECK_LAUNCH("attn_combine_quant_kernel");
    return 0;
}

// q [T,Hq,D], kv_layer [pages,2,Hkv,P,D], out [T,Hq,D]; metadata as in the ragged step ABI.
// ws must hold splits*T*Hq*(D+1) floats when splits > 1 (pass splits = 1 to avoid scratch).
extern "C" int telb_paged_attention(const void* q, const void* kv_layer, void* out, const int* q_start,
                                    const int* q_len, const int* past_len, const int* page_table,
                                    const int* tree_mask, int mask_words, int num_seqs, int total_tokens,
                                    int max_q_len, int num_pages, int max_pages, int page_size, int hq, int hkv, int d,
                                    float scale, int window, int splits, float* ws, long long ws_floats, int is_bf16,
                                    int* status, const float* sinks, const float* skip_thr, int* skip_stats, cudaStream_t stream) {
    if (num_seqs <= 0 || total_tokens <= 0) return 0;
    if (d != 64 && d != 128 && d != 256) return fail("telb_paged_attention: head_dim must be 64, 128 or 256");
    if (page_size != 64 && page_size != 128) return fail("telb_paged_attention: page size must be 64 or 128");
    if (hq % hkv) return fail("telb_paged_attention: Hq must be a multiple of Hkv");
    const int group = hq / hkv;
    if (group > 128 || (128 % group)) return fail("telb_paged_attention: GQA ratio must divide 128");
    AttnParams p{};
    p.out = out;
    p.q_start = q_start;
    p.q_len = q_len;
    p.past_len = past_len;
    p.page_table = page_table;
    p.tree_mask = tree_mask;
    p.mask_words = mask_words;
    p.max_pages = max_pages;
    p.page_size = page_size;
    p.hq = hq;
    p.hkv = hkv;
    p.group = group;
    p.tq = 128 / group;
    p.total_tokens = total_tokens;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.out_bf16 = is_bf16;
    p.sinks = sinks;
    p.skip_thr = skip_thr;
    p.skip_stats = skip_stats;
    p.status = status;
    if (splits < 1) splits = 1;
    while (splits > 1 && (long long)splits * total_tokens * hq * (d + 1) > ws_floats) --splits;
    p.splits = splits;
    p.ws_o = ws;
    p.ws_lse = ws ? ws + (size_t)splits * total_tokens * hq * d : nullptr;
    const int qtiles = (max_q_len + p.tq - 1) / p.tq;
    const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap tq, tkv;
    {
        const uint64_t dims[3] = {(uint64_t)d, (uint64_t)hq, (uint64_t)total_tokens};
        const uint64_t strides[2] = {(uint64_t)d * 2, (uint64_t)hq * d * 2};
        const uint32_t box[3] = {64, (uint32_t)group, (uint32_t)p.tq};
        if (make_tmap_nd(&tq, dt, 3, q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    }
    {
        const uint64_t rows = (uint64_t)num_pages * 2 * hkv * page_size;
        if (make_tmap_2d(&tkv, dt, 2, kv_layer, rows, d, (uint64_t)d * 2, kKvTile, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    }
    if (d == 128) {
        if (is_bf16) return launch_attn<128, __nv_bfloat16>(tq, tkv, p, qtiles, num_seqs, stream);
        return launch_attn<128, __half>(tq, tkv, p, qtiles, num_seqs, stream);
    }
    if (d == 256) {
        if (is_bf16) return launch_attn<256, __nv_bfloat16>(tq, tkv, p, qtiles, num_seqs, stream);
        return launch_attn<256, __half>(tq, tkv, p, qtiles, num_seqs, stream);
    }
    if (is_bf16) return launch_attn<64, __nv_bfloat16>(tq, tkv, p, qtiles, num_seqs, stream);
    return launch_attn<64, __half>(tq, tkv, p, qtiles, num_seqs, stream);
}
