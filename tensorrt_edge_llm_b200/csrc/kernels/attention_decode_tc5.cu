// GQA decode attention over the paged KV cache, XQA-style, on tcgen05.
//
// A decode step has 1..4 new tokens per sequence, so the work is streaming K and V once.  The
// tile is transposed relative to the prefill kernel: 128 cached tokens sit on the MMA-M side
// and the (query token, head-in-group) pairs — at most 16 — are the MMA-N side:
//     Sᵀ[128 tok, 16] = K[128 tok, D] · Qᵀ          (K-major A straight from the cache pages)
//     Oᵀ[D, 16]      += Vᵀ[D, 128 tok] · Pᵀ          (V used as an MN-major A operand, P from smem)
// Each softmax thread owns one cached token, i.e. 16 scores, so the per-tile softmax is a few
// dozen instructions instead of a row-long loop; the column max is a warp `redux.sync.max.f32`
// plus one shared-memory exchange, and the column sums are kept as per-thread partials that are
// reduced once at the end.  O is rescaled lazily (only when a column max grows by more than 2^8).
//
// CTA = (KV head, sequence, KV split); 128-token tiles = 2 pages of 64 (or 1 of 128), fetched by
// TMA into a 3-stage ring.  Splits write normalised fp32 partials + log-sum-exp; the merge kernel
// of attention_tc5.cu combines them.
//
// Reference counterparts: kernelSrcs/fmha_decode_ctm/fmha_decode.py (CTM) and kernelSrcs/xqa/mha.cu.
#include <type_traits>

#include "host_utils.h"
#include "nvfp4_common.cuh"
#include "tc5_common.cuh"

namespace telb {

struct DecParams {
    void* out;
    // optional NVFP4 output for the projection that follows (splits == 1): packed codes [T, Hq * D / 2], atom-layout scales
    uint8_t* oq;
    uint8_t* osf;
    const float* ogs;
    int ok64;
    float* ws_o;
    float* ws_lse;
    const int* q_start;
    const int* q_len;
    const int* past_len;
    const int* page_table;
    int max_pages, page_size;
    int hq, hkv, group;
    int splits, total_tokens, window;
    int num_seqs, num_items;        // items = sequences x KV heads x splits, walked by persistent CTAs
    float scale_log2;
    const float* sinks;             // [Hq] fp32 per-head sink logits (natural-log units), or null
    // FP8 (E4M3) cache pages read directly (KV8 kernels): kv_scales[0] multiplies the scores (K dequantisation scale),
    // kv_scales[1] the output (V scale); probabilities enter the P·V product as E4M3 of 256 x p.
    const float* kv_scales;
    int* status;
    // Optional timeline of CTA 0: trace[role][tile][event] in ns since the CTA started (role 0 producer,
    // 1 MMA issuer, 2 softmax; 4 events per tile, 64 tiles at most).  Null in normal use.
    unsigned long long* trace;
};

// E4M3 x E4M3 MMA with fp32 accumulation (K = 32 per instruction); the instruction descriptor has the layout of the 16-bit
// kind with format code 0 (= E4M3) for both operands.
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

constexpr int kDecThreads = 192;
constexpr int kDecTile = 128;      // cached tokens per tile
constexpr int kDecN = 16;          // (query token, head) columns
constexpr int kTraceTiles = 64;

__device__ __forceinline__ void trace_at(const DecParams& p, unsigned long long t0, int role, int tile, int ev) {
    if (p.trace && blockIdx.x == 0 && tile < kTraceTiles)
        p.trace[(role * kTraceTiles + tile) * 4 + ev] = global_timer_ns() - t0;
}

__device__ __forceinline__ float warp_max_f32(float v) {
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}

// One unit of work: the cached tokens [j0, j0 + ntiles) x 128 of one (sequence, KV head).
struct DecItem {
    int seq, kvh, split, qlen, past, qrow0, j0, ntiles;
};

// Items are ordered KV head fastest, so CTAs that run side by side read neighbouring slabs of the same pages.
__device__ __forceinline__ DecItem decode_item(const DecParams& p, int item) {
    DecItem it;
    it.kvh = item % p.hkv;
    const int rest = item / p.hkv;
    it.split = rest % p.splits;
    it.seq = rest / p.splits;
    it.qlen = p.q_len[it.seq];
    it.past = p.past_len[it.seq];
    it.qrow0 = p.q_start[it.seq];
    const int kv_end = it.past + it.qlen;
    int tile_lo = 0;
    if (p.window > 0) tile_lo = max(0, it.past - p.window + 1) / kDecTile;
    const int tile_hi = (kv_end + kDecTile - 1) / kDecTile;
    const int per = (tile_hi - tile_lo + p.splits - 1) / p.splits;
    it.j0 = tile_lo + it.split * per;
    it.ntiles = it.qlen > 0 ? max(0, min(tile_hi, it.j0 + per) - it.j0) : 0;
    return it;
}

// KS / VS: depth of the K and V tile rings; MINB: CTAs that must fit on one SM (co-resident CTAs with shallow
// rings hide each other's per-tile synchronisation latency; one CTA with deep rings prefetches further).
// NC: how many of the 16 MMA columns can be live (query tokens x heads per KV head, rounded up to 4 / 8 / 16);
// the softmax registers and loops are sized by it.
//
// The grid is persistent: CTA b walks items b, b + gridDim.x, ...  The K/V rings, the four score buffers and the
// two P buffers keep cycling across item boundaries (flat tile counter), Q and the O accumulator are double
// buffered per item, so the next item's loads and scores overlap the previous item's epilogue and no CTA slot
// idles while another wave of CTAs starts up.
// KV8: the cache pages (and the Q and P operands) are E4M3 bytes: a 128-byte swizzle span holds 128 elements instead of 64, an
// MMA consumes 32 of them per instruction instead of 16, everything else (roles, rings, barriers, softmax) is shared.
template <int D, typename T, int KS, int VS, int MINB, int NC, bool KV8 = false>
__global__ void __launch_bounds__(kDecThreads, MINB)
attn_decode_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_kv, DecParams p) {
    constexpr int kEB = KV8 ? 1 : 2;                            // bytes per operand element
    constexpr int kSpan = 128 / kEB;                            // elements per 128-byte swizzle span
    constexpr int kMmaK = KV8 ? 32 : 16;                        // K elements per MMA
    constexpr int kDChunks = D / kSpan;
    constexpr int kChunkBytes = kDecTile * 128;                 // [128 tokens x one span of d]
    constexpr int kKvBytes = kDChunks * kChunkBytes;            // one K or V tile
    constexpr int kQBytes = kDChunks * kDecN * 128;
    constexpr int kPBytes = (kDecTile / kSpan) * kDecN * 128;   // Pᵀ: [16 cols x 128 tokens], one span of tokens per chunk
    constexpr int kSBufs = 4;                                   // score buffers S0..S3 @ 0, 16, 32, 48
    constexpr int kOCol = kSBufs * 16;                          // O accumulators O0, O1 (16 columns each)
    constexpr int kTmemCols = 128;
    constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* s_k = smem;
    uint8_t* s_v = s_k + KS * kKvBytes;
    uint8_t* s_q = s_v + VS * kKvBytes;                         // two Q buffers
    uint8_t* s_p = s_q + 2 * kQBytes;                           // two P buffers
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_p + 2 * kPBytes);
    uint64_t* q_full = bars;
    uint64_t* q_free = q_full + 2;
    uint64_t* k_full = q_free + 2;
    uint64_t* k_empty = k_full + KS;
    uint64_t* v_full = k_empty + KS;
    uint64_t* v_empty = v_full + VS;
    uint64_t* s_full = v_empty + VS;
    uint64_t* s_free = s_full + kSBufs;
    uint64_t* p_full = s_free + kSBufs;
    uint64_t* p_free = p_full + 2;
    uint64_t* o_full = p_free + 2;
    uint64_t* o_free = o_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_free + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* s_red = reinterpret_cast<float*>(tmem_slot + 4);     // [2 parities][4 warps][16] column maxima
    float* s_sum = s_red + 128;                                 // [4 warps][16] column sums (item epilogue)

    pdl_prologue();          // step metadata and Q/KV are produced by earlier kernels
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&q_full[s], 1);
            mbar_init(&q_free[s], 1);
            mbar_init(&p_full[s], 128);
            mbar_init(&p_free[s], 1);
            mbar_init(&o_full[s], 1);
            mbar_init(&o_free[s], 128);
        }
        for (int s = 0; s < KS; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
        }
        for (int s = 0; s < VS; ++s) {
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        for (int s = 0; s < kSBufs; ++s) {
            mbar_init(&s_full[s], 1);
            mbar_init(&s_free[s], 128);
        }
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tensormap(&tma_q);
        prefetch_tensormap(&tma_kv);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    for (int i = threadIdx.x; i < 2 * kPBytes / 16; i += blockDim.x) reinterpret_cast<uint4*>(s_p)[i] = make_uint4(0, 0, 0, 0);
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const unsigned long long t_start = p.trace ? global_timer_ns() : 0ull;

    if (warp == 0) {
        // ------------------------------ producer ------------------------------
        // The whole warp walks the tiles: every lane fetches the page ids of one tile ahead of time (one coalesced
        // read per 32 tiles instead of dependent global loads on the issuing thread), lane 0 issues the TMA copies.
        const int pages_per_tile = kDecTile / p.page_size;          // 2 for 64-token pages, 1 for 128
        const int rows_per_load = kDecTile / pages_per_tile;
        bool ok = true;
        int jg = 0, ig = 0;
        for (int item = blockIdx.x; item < p.num_items && ok; item += gridDim.x) {
            const DecItem it = decode_item(p, item);
            if (it.ntiles <= 0) continue;
            if (lane == 0) {
                // Q columns: (query token qi, head g) → row qi*G + g of a [16 x D] K-major tile
                ok = mbar_wait(&q_free[ig & 1], ((ig >> 1) & 1) ^ 1, abort_flag, p.status, kStatusProducerTimeout);
                if (ok) {
                    mbar_expect_tx(&q_full[ig & 1], kQBytes);
#pragma unroll
                    for (int c = 0; c < kDChunks; ++c)
                        tma_load_3d(s_q + (ig & 1) * kQBytes + c * (kDecN * 128), &tma_q, &q_full[ig & 1], c * kSpan, it.kvh * p.group, it.qrow0);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            for (int base = 0; base < it.ntiles && ok; base += 32) {
                int pg[2] = {0, 0};
                if (base + lane < it.ntiles) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int lp = (it.j0 + base + lane) * pages_per_tile + h;
                        int page = -1;
                        if (h < pages_per_tile && lp < p.max_pages) page = p.page_table[(size_t)it.seq * p.max_pages + lp];
                        pg[h] = page < 0 ? 0 : page;                     // masked anyway
                    }
                }
                const int cnt = min(32, it.ntiles - base);
                for (int jj = 0; jj < cnt && ok; ++jj, ++jg) {
                    const int page0 = __shfl_sync(0xffffffffu, pg[0], jj), page1 = __shfl_sync(0xffffffffu, pg[1], jj);
                    if (lane == 0) {
                        const int ks = jg % KS, vs = jg % VS;
                        const uint32_t kph = ((jg / KS) & 1) ^ 1, vph = ((jg / VS) & 1) ^ 1;
                        const int rows[2] = {((page0 * 2 + 0) * p.hkv + it.kvh) * p.page_size, ((page1 * 2 + 0) * p.hkv + it.kvh) * p.page_size};
                        ok = mbar_wait(&k_empty[ks], kph, abort_flag, p.status, kStatusProducerTimeout);
                        if (ok) {
                            trace_at(p, t_start, 0, jg, 0);         // K slot free, K loads issued next
                            mbar_expect_tx(&k_full[ks], kKvBytes);
                            for (int h = 0; h < pages_per_tile; ++h)
#pragma unroll
                                for (int c = 0; c < kDChunks; ++c)
                                    tma_load_2d(s_k + ks * kKvBytes + c * kChunkBytes + h * rows_per_load * 128, &tma_kv, &k_full[ks],
                                                c * kSpan, rows[h]);
                            ok = mbar_wait(&v_empty[vs], vph, abort_flag, p.status, kStatusProducerTimeout);
                        }
                        if (ok) {
                            trace_at(p, t_start, 0, jg, 1);         // V slot free, V loads issued next
                            mbar_expect_tx(&v_full[vs], kKvBytes);
                            for (int h = 0; h < pages_per_tile; ++h)
#pragma unroll
                                for (int c = 0; c < kDChunks; ++c)
                                    tma_load_2d(s_v + vs * kKvBytes + c * kChunkBytes + h * rows_per_load * 128, &tma_kv, &v_full[vs],
                                                c * kSpan, rows[h] + p.hkv * p.page_size);
                        }
                    }
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                }
            }
            ++ig;
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            // format code 0 is fp16 for the 16-bit kind and E4M3 for the 8-bit kind
            const uint32_t idesc_s = idesc_f16(128, kDecN, kBf16 && !KV8);                    // A = K (K-major), B = Q (K-major)
            const uint32_t idesc_o = idesc_f16(128, kDecN, kBf16 && !KV8, /*a_mn_major=*/true);   // A = Vᵀ (MN-major), B = Pᵀ (K-major)
            // Two cursors walk the same item list: scores (S = K Qᵀ) run up to kSBufs tiles ahead of P·V, so the
            // score MMA is never on the softmax → P·V dependency chain.
            struct Cursor {
                int item, ig, j, jg, ntiles;       // current item, its ordinal among non-empty items, tile in item, flat tile
            };
            auto advance = [&](Cursor& c) {        // move to the next non-empty item of this CTA (ntiles = 0 at the end)
                c.ntiles = 0;
                while (c.item < p.num_items) {
                    const DecItem it = decode_item(p, c.item);
                    if (it.ntiles > 0) {
                        c.ntiles = it.ntiles;
                        return;
                    }
                    c.item += gridDim.x;
                }
            };
            Cursor cs{(int)blockIdx.x, 0, 0, 0, 0}, cp{(int)blockIdx.x, 0, 0, 0, 0};
            advance(cs);
            advance(cp);
            bool ok = true;
            const long long spin0 = clock64();
            unsigned int idle = 0;
            while (ok && cp.ntiles > 0) {
                bool progressed = false;
                if (cs.ntiles > 0 && cs.jg < cp.jg + kSBufs && (cs.j > 0 || mbar_try_wait(&q_full[cs.ig & 1], (cs.ig >> 1) & 1)) &&
                    mbar_try_wait(&k_full[cs.jg % KS], (cs.jg / KS) & 1) && mbar_try_wait(&s_free[cs.jg % kSBufs], ((cs.jg / kSBufs) & 1) ^ 1)) {
                    tc_fence_after_sync();
                    trace_at(p, t_start, 1, cs.jg, 0);      // K tile landed and S buffer free: S = K Qᵀ issued
                    const int stage = cs.jg % KS;
                    const uint64_t dk = smem_desc_sw128(s_k + stage * kKvBytes);
                    const uint64_t dq = smem_desc_sw128(s_q + (cs.ig & 1) * kQBytes);
                    const uint32_t d_tmem = tmem_base + (cs.jg % kSBufs) * 16;
#pragma unroll
                    for (int k = 0; k < D / kMmaK; ++k) {          // four MMAs per 128-byte span, 32 bytes each
                        const int c = k >> 2, kk = k & 3;
                        const uint64_t da_ = dk + (uint64_t)((c * kChunkBytes) >> 4) + 2 * kk, db_ = dq + (uint64_t)((c * kDecN * 128) >> 4) + 2 * kk;
                        if constexpr (KV8) umma_f8(d_tmem, da_, db_, idesc_s, k > 0 ? 1u : 0u);
                        else umma_f16(d_tmem, da_, db_, idesc_s, k > 0 ? 1u : 0u);
                    }
                    umma_commit(&k_empty[stage]);
                    umma_commit(&s_full[cs.jg % kSBufs]);
                    ++cs.j;
                    ++cs.jg;
                    if (cs.j == cs.ntiles) {                // last score tile of the item: its Q buffer may be refilled
                        umma_commit(&q_free[cs.ig & 1]);
                        cs.item += gridDim.x;
                        ++cs.ig;
                        cs.j = 0;
                        advance(cs);
                    }
                    progressed = true;
                }
                if (cp.jg < cs.jg && mbar_try_wait(&p_full[cp.jg & 1], (cp.jg >> 1) & 1) && mbar_try_wait(&v_full[cp.jg % VS], (cp.jg / VS) & 1) &&
                    (cp.j > 0 || mbar_try_wait(&o_free[cp.ig & 1], ((cp.ig >> 1) & 1) ^ 1))) {
                    tc_fence_after_sync();
                    trace_at(p, t_start, 1, cp.jg, 1);      // P written and V tile landed: O += Vᵀ Pᵀ issued
                    const int stage = cp.jg % VS;
                    // A = Vᵀ: 64-wide d chunks are kChunkBytes apart (leading offset), 8-token groups 1024 B apart
                    const uint64_t dv = smem_desc_sw128_mn(s_v + stage * kKvBytes, kChunkBytes, 1024);
                    const uint64_t dp = smem_desc_sw128(s_p + (cp.jg & 1) * kPBytes);
                    const uint32_t d_o = tmem_base + kOCol + (cp.ig & 1) * 16;
#pragma unroll
                    for (int k = 0; k < kDecTile / kMmaK; ++k) {    // 16 (32) tokens per MMA: 2048 (4096) B of V rows, 32 B of a P row
                        const uint64_t da_ = dv + (uint64_t)((k * kMmaK * 128) >> 4), db_ = dp + (uint64_t)(((k >> 2) * (kDecN * 128)) >> 4) + 2 * (k & 3);
                        if constexpr (KV8) umma_f8(d_o, da_, db_, idesc_o, (cp.j > 0 || k > 0) ? 1u : 0u);
                        else umma_f16(d_o, da_, db_, idesc_o, (cp.j > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&v_empty[stage]);
                    umma_commit(&p_free[cp.jg & 1]);
                    ++cp.j;
                    ++cp.jg;
                    if (cp.j == cp.ntiles) {                // the item's accumulator is complete
                        umma_commit(&o_full[cp.ig & 1]);
                        cp.item += gridDim.x;
                        ++cp.ig;
                        cp.j = 0;
                        advance(cp);
                    }
                    progressed = true;
                }
                if (progressed) {
                    idle = 0;
                } else if ((++idle & 1023u) == 0) {         // bounded: give up after about two seconds without progress
                    if (*abort_flag) ok = false;
                    else if (idle > (1u << 20) && clock64() - spin0 > kSpinLimitCycles) {
                        *abort_flag = 1u;
                        if (p.status) atomicCAS(p.status, kStatusOk, kStatusMmaTimeout);
                        ok = false;
                    }
                }
            }
        }
    } else {
        // ------------------------------ softmax / epilogue ------------------------------
        const int quad = warp & 3;
        const int r = quad * 32 + lane;                 // cached token within the tile == TMEM lane (S); feature d (O)
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
        const int gshift = 31 - __clz(p.group);         // the group size is a power of two
        // FP8 pages: the K scale multiplies the scores, the V scale and the 1 / 256 of the scaled probabilities the output
        const float scale_log2 = KV8 ? p.scale_log2 * p.kv_scales[0] : p.scale_log2;
        const float o_scale = KV8 ? p.kv_scales[1] * (1.f / 256.f) : 1.f;
        bool ok = true;
        int jg = 0, ig = 0;
        for (int item = blockIdx.x; item < p.num_items && ok; item += gridDim.x) {
            const DecItem it = decode_item(p, item);
            if (it.qlen <= 0) continue;
            const int ncol = it.qlen * p.group;         // live columns (<= NC)
            float m_used[NC], l_part[NC];
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                m_used[c] = -INFINITY;
                l_part[c] = 0.f;
            }
            const uint32_t o_addr = lane_addr + kOCol + (ig & 1) * 16;
            for (int j = 0; j < it.ntiles && ok; ++j, ++jg) {
                const int b = jg & 1;                   // P buffer
                const int sb = jg % kSBufs;             // score buffer
                if (!mbar_wait(&s_full[sb], (jg / kSBufs) & 1, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
                tc_fence_after_sync();
                if (threadIdx.x == 64) trace_at(p, t_start, 2, jg, 0);     // scores ready
                uint32_t raw[NC];
                tmem_ld_n<NC>(lane_addr + sb * 16, raw);
                tmem_ld_wait();
                tc_fence_before_sync();
                mbar_arrive(&s_free[sb]);
                const int tk = (it.j0 + j) * kDecTile + r;     // absolute cache slot of this thread's token
                float s[NC];
                float* red = s_red + b * 64;
                // Only the live columns (query tokens x heads of this sequence) are processed; `ncol`
                // is uniform across the CTA, so the guards below do not diverge.
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    if (c < ncol) {
                        const int qi = c >> gshift;
                        bool vis = tk <= it.past + qi;
                        if (p.window > 0) vis = vis && tk > it.past + qi - p.window;
                        s[c] = vis ? __uint_as_float(raw[c]) * scale_log2 : -INFINITY;
                        const float wm = warp_max_f32(s[c]);
                        if (lane == c) red[(warp - 2) * 16 + c] = wm;
                    } else {
                        s[c] = -INFINITY;
                    }
                }
                named_barrier_sync(1, 128);
                if (threadIdx.x == 64) trace_at(p, t_start, 2, jg, 1);     // column maxima exchanged
                bool any_need = false;
                float f[NC];
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    f[c] = 1.f;
                    if (c < ncol) {
                        const float mt = fmaxf(fmaxf(red[c], red[16 + c]), fmaxf(red[32 + c], red[48 + c]));
                        const float m_new = fmaxf(m_used[c], mt);
                        if (m_new > m_used[c] + 8.0f) {               // uniform across the CTA
                            f[c] = (m_used[c] == -INFINITY) ? 0.f : exp2f(m_used[c] - m_new);
                            l_part[c] *= f[c];
                            m_used[c] = m_new;
                            any_need = true;
                        }
                    }
                }
                // P buffer b is free once the P·V two tiles back has completed.  This wait is taken for every use of the
                // buffer, so its parity is exact; it also pins how far the tensor pipe can lag behind this warp.
                if (!mbar_wait(&p_free[b], ((jg >> 1) & 1) ^ 1, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
                if (j > 0 && any_need) {
                    // O may only be rescaled after the previous tile's P·V has landed: that is the next completion of the
                    // other P buffer's barrier (a parity wait on a barrier polled only now and then could alias).
                    if (!mbar_wait(&p_free[b ^ 1], ((jg - 1) >> 1) & 1, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
                    tc_fence_after_sync();
                    uint32_t o[NC];
                    tmem_ld_n<NC>(o_addr, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < NC; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * f[c]);
                    tmem_st_n<NC>(o_addr, o);
                    tmem_st_wait();
                    tc_fence_before_sync();
                }
                // Pᵀ[c][token]: row c is 128 tokens = two 128-byte swizzled chunks of 64 tokens.  Dead columns hold the
                // zeros written at start-up.
                // one 128-byte span of row c holds kSpan tokens; element bytes kEB
                uint8_t* pbase = s_p + b * kPBytes + (r / kSpan) * (kDecN * 128);
                const int tl = r % kSpan;
                constexpr int kPer16 = 16 / kEB;               // tokens per 16-byte swizzle unit
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    uint8_t* dst = pbase + (c >> 3) * 1024 + (c & 7) * 128 + ((((tl / kPer16) ^ (c & 7)) & 7) << 4) + (tl % kPer16) * kEB;
                    if (c < ncol) {
                        const float mref = m_used[c] == -INFINITY ? 0.f : m_used[c];
                        const float e = exp2f(s[c] - mref);
                        l_part[c] += e;
                        if constexpr (KV8) *dst = __nv_cvt_float_to_fp8(e * 256.f, __NV_SATFINITE, __NV_E4M3);
                        else *reinterpret_cast<T*>(dst) = Cvt<T>::from_f(e);
                    } else if (c < kDecN) {
                        // a shorter sequence may follow a longer one in this CTA: clear columns it no longer uses
                        if constexpr (KV8) *dst = 0;
                        else *reinterpret_cast<T*>(dst) = Cvt<T>::from_f(0.f);
                    }
                }
                fence_proxy_async_smem();
                mbar_arrive(&p_full[b]);
                if (threadIdx.x == 64) trace_at(p, t_start, 2, jg, 2);     // probabilities published
            }
            if (!ok) break;
            // ---- item epilogue: column sums across the 128 threads, then O / l ----
            named_barrier_sync(1, 128);
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                float v = l_part[c];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == c) s_sum[(warp - 2) * 16 + c] = v;
            }
            named_barrier_sync(1, 128);
            uint32_t o[NC];
            if (it.ntiles > 0) {
                if (!mbar_wait(&o_full[ig & 1], (ig >> 1) & 1, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
                tc_fence_after_sync();
                tmem_ld_n<NC>(o_addr, o);
                tmem_ld_wait();
                tc_fence_before_sync();
                mbar_arrive(&o_free[ig & 1]);           // the accumulator may be overwritten by the item after next
            }
            if (r < D) {
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    if (c < ncol) {
                        const float l = s_sum[c] + s_sum[16 + c] + s_sum[32 + c] + s_sum[48 + c];
                        const int qi = c >> gshift, g = c - (qi << gshift);
                        const size_t tok = (size_t)it.qrow0 + qi;
                        const int head = it.kvh * p.group + g;
                        const bool have = it.ntiles > 0 && l > 0.f;
                        float inv = have ? 1.f / l : 0.f;
                        float lse = have ? m_used[c] + log2f(l) : -INFINITY;
                        if (p.sinks != nullptr && it.split == 0) {
                            // the sink is one more logit with no value row: it only grows the denominator (first split only)
                            const float z = p.sinks[head] * 1.44269504f;
                            if (have) {
                                const float m2 = fmaxf(m_used[c], z);
                                const float os = exp2f(m_used[c] - m2);
                                const float l2 = l * os + exp2f(z - m2);
                                inv = os / l2;
                                lse = m2 + log2f(l2);
                            } else {
                                lse = z;
                            }
                        }
                        const float val = have ? __uint_as_float(o[c]) * inv * o_scale : 0.f;
                        if (p.splits == 1 && p.oq != nullptr) {
                            // the output projection reads NVFP4: quantise here (16 consecutive dims = 16 consecutive lanes),
                            // with the rounding of the 16-bit store the unfused path would have made first
                            const float gs = *p.ogs;
                            uint8_t s8;
                            const uint32_t w4 = nvfp4_quantize_lane16(Cvt<T>::to_f(Cvt<T>::from_f(val)), gs, 1.f / gs, s8);
                            const int col = head * D + r;
                            if ((lane & 7) == 0) *reinterpret_cast<uint32_t*>(p.oq + tok * (size_t)(p.hq * D / 2) + col / 2) = w4;
                            if ((lane & 15) == 0) p.osf[sf_atom_offset((long long)tok, col >> 4, p.ok64)] = s8;
                        } else if (p.splits == 1) {
                            reinterpret_cast<T*>(p.out)[(tok * p.hq + head) * D + r] = Cvt<T>::from_f(val);
                        } else {
                            p.ws_o[(((size_t)it.split * p.total_tokens + tok) * p.hq + head) * D + r] = val;
                            if (r == 0) p.ws_lse[((size_t)it.split * p.total_tokens + tok) * p.hq + head] = lse;
                        }
                    }
                }
            }
            if (it.ntiles > 0) ++ig;
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

template <int D, typename T, int KS, int VS, int MINB, int NC, bool KV8 = false>
static int launch_decode_variant(const CUtensorMap& tq, const CUtensorMap& tkv, const DecParams& p, int nseq, cudaStream_t stream) {
    constexpr int kv = (D / (KV8 ? 128 : 64)) * kDecTile * 128;
    constexpr int smem = (KS + VS) * kv + 2 * 4096 + 2 * 2 * kDecN * 128 + 1024 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<D, T, KS, VS, MINB, NC, KV8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail("cudaFuncSetAttribute(attn_decode)", e);
        configured = true;
    }
    const int slots = MINB * sm_count();
    const int grid = p.num_items < slots ? p.num_items : slots;
    TELB_LAUNCH("attn_decode_kernel", (attn_decode_kernel<D, T, KS, VS, MINB, NC, KV8>), dim3(grid), dim3(kDecThreads), smem, stream, tq, tkv, p);
    TELB_CHECK_LAUNCH("attn_decode_kernel");
    return 0;
}

static int g_decode_variant = 1;      // measured fastest at batch 8..64 with 1k context

template <int D, typename T, int NC>
static int launch_decode_nc(const CUtensorMap& tq, const CUtensorMap& tkv, const DecParams& p, int nseq, cudaStream_t stream) {
    switch (g_decode_variant) {
        case 1: return launch_decode_variant<D, T, 1, 1, 2, NC>(tq, tkv, p, nseq, stream);     // 2 CTAs / SM, single-stage rings
        case 2: return launch_decode_variant<D, T, 2, 2, 1, NC>(tq, tkv, p, nseq, stream);     // 1 CTA / SM, two-stage rings
        default: return launch_decode_variant<D, T, 3, 3, 1, NC>(tq, tkv, p, nseq, stream);    // 1 CTA / SM, three-stage rings
    }
}

// FP8 pages: half the bytes per tile, so two CTAs per SM hold two-stage rings
template <int D, typename T>
static int launch_decode_fp8(const CUtensorMap& tq, const CUtensorMap& tkv, const DecParams& p, int nseq, int max_cols, cudaStream_t stream) {
    if (max_cols <= 4) return launch_decode_variant<D, T, 2, 2, 2, 4, true>(tq, tkv, p, nseq, stream);
    if (max_cols <= 8) return launch_decode_variant<D, T, 2, 2, 2, 8, true>(tq, tkv, p, nseq, stream);
    return launch_decode_variant<D, T, 2, 2, 2, 16, true>(tq, tkv, p, nseq, stream);
}

template <int D, typename T>
static int launch_decode(const CUtensorMap& tq, const CUtensorMap& tkv, const DecParams& p, int nseq, int max_cols, cudaStream_t stream) {
    if (max_cols <= 4) return launch_decode_nc<D, T, 4>(tq, tkv, p, nseq, stream);
    if (max_cols <= 8) return launch_decode_nc<D, T, 8>(tq, tkv, p, nseq, stream);
    return launch_decode_nc<D, T, 16>(tq, tkv, p, nseq, stream);
}

}  // namespace telb

using namespace telb;

extern "C" int telb_attn_combine(const float* ws_o, const float* ws_lse, void* out, int rows, int splits, int d, int is_bf16,
                                 cudaStream_t stream);
extern "C" int telb_attn_combine_quant(const float* ws_o, const float* ws_lse, void* oq, void* osf, const float* ogs, int tokens, int hq,
                                       int splits, int d, int is_bf16, cudaStream_t stream);
extern "C" int telb_nvfp4_k64_pad(int k);

// Ring depth / residency variant of the decode kernel (0, 1 or 2: see launch_decode); process-wide.
extern "C" int telb_set_decode_variant(int v) {
    if (v < 0 || v > 2) return fail("telb_set_decode_variant: variant must be 0, 1 or 2");
    g_decode_variant = v;
    return 0;
}

extern "C" int telb_paged_attention_decode_traced(const void* q, const void* kv_layer, void* out, const int* q_start,
                                                  const int* q_len, const int* past_len, const int* page_table, int num_seqs,
                                                  int total_tokens, int max_q_len, int num_pages, int max_pages, int page_size,
                                                  int hq, int hkv, int d, float scale, int window, int splits, float* ws,
                                                  long long ws_floats, int is_bf16, int* status, unsigned long long* trace,
                                                  const float* sinks, cudaStream_t stream);

// Decode-shaped steps only: max_q_len * (Hq/Hkv) <= 16.  Same tensors as telb_paged_attention.
extern "C" int telb_paged_attention_decode(const void* q, const void* kv_layer, void* out, const int* q_start,
                                           const int* q_len, const int* past_len, const int* page_table, int num_seqs,
                                           int total_tokens, int max_q_len, int num_pages, int max_pages, int page_size,
                                           int hq, int hkv, int d, float scale, int window, int splits, float* ws,
                                           long long ws_floats, int is_bf16, int* status, cudaStream_t stream) {
    return telb_paged_attention_decode_traced(q, kv_layer, out, q_start, q_len, past_len, page_table, num_seqs, total_tokens, max_q_len,
                                              num_pages, max_pages, page_size, hq, hkv, d, scale, window, splits, ws, ws_floats, is_bf16,
                                              status, nullptr, nullptr, stream);
}

static int decode_impl(const void* q, const void* kv_layer, void* out, void* oq, void* osf, const float* ogs, const int* q_start,
                       const int* q_len, const int* past_len, const int* page_table, int num_seqs, int total_tokens, int max_q_len,
                       int num_pages, int max_pages, int page_size, int hq, int hkv, int d, float scale, int window, int splits, float* ws,
                       long long ws_floats, int is_bf16, int* status, unsigned long long* trace, const float* sinks, const float* kv_scales,
                       cudaStream_t stream);

// Same call with a timeline buffer (3 x 64 x 4 u64, zeroed by the caller) filled by the first CTA.
extern "C" int telb_paged_attention_decode_traced(const void* q, const void* kv_layer, void* out, const int* q_start,
                                                  const int* q_len, const int* past_len, const int* page_table, int num_seqs,
                                                  int total_tokens, int max_q_len, int num_pages, int max_pages, int page_size,
                                                  int hq, int hkv, int d, float scale, int window, int splits, float* ws,
                                                  long long ws_floats, int is_bf16, int* status, unsigned long long* trace,
                                                  const float* sinks, cudaStream_t stream) {
    return decode_impl(q, kv_layer, out, nullptr, nullptr, nullptr, q_start, q_len, past_len, page_table, num_seqs, total_tokens, max_q_len,
                       num_pages, max_pages, page_size, hq, hkv, d, scale, window, splits, ws, ws_floats, is_bf16, status, trace, sinks, nullptr, stream);
}

// Decode attention whose output is written as NVFP4 only (packed codes out_xq [T, Hq * D / 2], atom-layout scales out_sf over
// rows T and Hq * D columns, pre-zeroed by the caller where padding exists): the input of the output projection, so a decode
// layer has no separate quantisation kernel between attention and o_proj.
extern "C" int telb_paged_attention_decode_quant(const void* q, const void* kv_layer, void* out_xq, void* out_sf, const float* out_global_scale,
                                                 const int* q_start, const int* q_len, const int* past_len, const int* page_table,
                                                 int num_seqs, int total_tokens, int max_q_len, int num_pages, int max_pages, int page_size,
                                                 int hq, int hkv, int d, float scale, int window, int splits, float* ws, long long ws_floats,
                                                 int is_bf16, int* status, const float* sinks, cudaStream_t stream) {
    if (!out_xq || !out_sf || !out_global_scale) return fail("telb_paged_attention_decode_quant: output buffers and scale are required");
    return decode_impl(q, kv_layer, nullptr, out_xq, out_sf, out_global_scale, q_start, q_len, past_len, page_table, num_seqs, total_tokens,
                       max_q_len, num_pages, max_pages, page_size, hq, hkv, d, scale, window, splits, ws, ws_floats, is_bf16, status, nullptr, sinks, nullptr, stream);
}

// Decode attention over FP8 (E4M3) cache pages read in place: `q8` is the query tensor cast to E4M3 [T, Hq, D], `kv_layer` the
// FP8 layer [pages, 2, Hkv, P, D], `kv_scales` the layer's (K, V) dequantisation scales on the device.  The output is 16-bit
// (`out`) or, when `out_xq` is given, NVFP4 for the projection that follows.  `is_bf16` names the output / activation type.
extern "C" int telb_paged_attention_decode_fp8(const void* q8, const void* kv_layer, void* out, void* out_xq, void* out_sf,
                                               const float* out_global_scale, const float* kv_scales, const int* q_start, const int* q_len,
                                               const int* past_len, const int* page_table, int num_seqs, int total_tokens, int max_q_len,
                                               int num_pages, int max_pages, int page_size, int hq, int hkv, int d, float scale, int window,
                                               int splits, float* ws, long long ws_floats, int is_bf16, int* status, const float* sinks,
                                               cudaStream_t stream) {
    if (!kv_scales) return fail("telb_paged_attention_decode_fp8: the K / V scales are required");
    if (!out && !out_xq) return fail("telb_paged_attention_decode_fp8: no output buffer");
    if (out_xq && (!out_sf || !out_global_scale)) return fail("telb_paged_attention_decode_fp8: NVFP4 output needs its scale buffers");
    return decode_impl(q8, kv_layer, out, out_xq, out_sf, out_global_scale, q_start, q_len, past_len, page_table, num_seqs, total_tokens,
                       max_q_len, num_pages, max_pages, page_size, hq, hkv, d, scale, window, splits, ws, ws_floats, is_bf16, status, nullptr,
                       sinks, kv_scales, stream);
}

static int decode_impl(const void* q, const void* kv_layer, void* out, void* oq, void* osf, const float* ogs, const int* q_start,
                       const int* q_len, const int* past_len, const int* page_table, int num_seqs, int total_tokens, int max_q_len,
                       int num_pages, int max_pages, int page_size, int hq, int hkv, int d, float scale, int window, int splits, float* ws,
                       long long ws_floats, int is_bf16, int* status, unsigned long long* trace, const float* sinks, const float* kv_scales,
                       cudaStream_t stream) {
    if (num_seqs <= 0 || total_tokens <= 0) return 0;
    if (d != 128) return fail("telb_paged_attention_decode: head_dim must be 128");
    if (page_size != 64 && page_size != 128) return fail("telb_paged_attention_decode: page size must be 64 or 128");
    if (hq % hkv) return fail("telb_paged_attention_decode: Hq must be a multiple of Hkv");
    const int group = hq / hkv;
    if (max_q_len * group > kDecN) return fail("telb_paged_attention_decode: q_len * (Hq/Hkv) must be <= 16");
    if (kDecN % group) return fail("telb_paged_attention_decode: Hq/Hkv must divide 16");
    DecParams p{};
    p.out = out;
    p.oq = static_cast<uint8_t*>(oq);
    p.osf = static_cast<uint8_t*>(osf);
    p.ogs = ogs;
    p.ok64 = telb_nvfp4_k64_pad(hq * d);
    p.sinks = sinks;
    p.kv_scales = kv_scales;
    p.q_start = q_start;
    p.q_len = q_len;
    p.past_len = past_len;
    p.page_table = page_table;
    p.max_pages = max_pages;
    p.page_size = page_size;
    p.hq = hq;
    p.hkv = hkv;
    p.group = group;
    p.total_tokens = total_tokens;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = status;
    p.trace = trace;
    p.num_seqs = num_seqs;
    if (splits < 1) splits = 1;
    if (splits > 32) splits = 32;
    while (splits > 1 && (long long)splits * total_tokens * hq * (d + 1) > ws_floats) --splits;
    p.splits = splits;
    p.num_items = num_seqs * hkv * splits;
    p.ws_o = ws;
    p.ws_lse = ws ? ws + (size_t)splits * total_tokens * hq * d : nullptr;
    const bool fp8 = kv_scales != nullptr;
    const CUtensorMapDataType dt = fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : (is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
    const uint64_t eb = fp8 ? 1 : 2;                  // bytes per element of Q and of the cache
    const uint32_t span = fp8 ? 128 : 64;             // elements per 128-byte swizzle span
    CUtensorMap tq, tkv;
    {
        // Q viewed as [tokens][Hq][D]; one box = (one span of features, G heads, 16/G tokens) → 16 rows of 128 B
        const uint64_t dims[3] = {(uint64_t)d, (uint64_t)hq, (uint64_t)total_tokens};
        const uint64_t strides[2] = {(uint64_t)d * eb, (uint64_t)hq * d * eb};
        const uint32_t box[3] = {span, (uint32_t)group, (uint32_t)(kDecN / group)};
        if (make_tmap_nd(&tq, dt, 3, q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    }
    {
        const uint64_t rows = (uint64_t)num_pages * 2 * hkv * page_size;
        const uint32_t box_rows = page_size == 64 ? 64 : 128;
        if (make_tmap_2d(&tkv, dt, (int)eb, kv_layer, rows, d, (uint64_t)d * eb, box_rows, span, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    }
    int rc;
    if (fp8)
        rc = is_bf16 ? launch_decode_fp8<128, __nv_bfloat16>(tq, tkv, p, num_seqs, max_q_len * group, stream)
                     : launch_decode_fp8<128, __half>(tq, tkv, p, num_seqs, max_q_len * group, stream);
    else
        rc = is_bf16 ? launch_decode<128, __nv_bfloat16>(tq, tkv, p, num_seqs, max_q_len * group, stream)
                     : launch_decode<128, __half>(tq, tkv, p, num_seqs, max_q_len * group, stream);
    if (rc) return rc;
    if (splits > 1 && oq) return telb_attn_combine_quant(p.ws_o, p.ws_lse, oq, osf, ogs, total_tokens, hq, splits, d, is_bf16, stream);
    if (splits > 1) return telb_attn_combine(p.ws_o, p.ws_lse, out, total_tokens * hq, splits, d, is_bf16, stream);
    return 0;
}
