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
#include "tc5_common.cuh"

namespace telb {

struct DecParams {
    void* out;
    float* ws_o;
    float* ws_lse;
    const int* q_start;
    const int* q_len;
    const int* past_len;
    const int* page_table;
    int max_pages, page_size;
    int hq, hkv, group;
    int splits, total_tokens, window;
    float scale_log2;
    int* status;
};

constexpr int kDecThreads = 192;
constexpr int kDecTile = 128;      // cached tokens per tile
constexpr int kDecN = 16;          // (query token, head) columns

__device__ __forceinline__ float warp_max_f32(float v) {
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}

// KS / VS: depth of the K and V tile rings; MINB: CTAs that must fit on one SM (two co-resident CTAs with
// shallow rings hide each other's per-tile synchronisation latency; one CTA with deep rings prefetches further).
// NC: how many of the 16 MMA columns can be live (query tokens x heads per KV head, rounded up to 4 / 8 / 16);
// the softmax registers and loops are sized by it.
template <int D, typename T, int KS, int VS, int MINB, int NC>
__global__ void __launch_bounds__(kDecThreads, MINB)
attn_decode_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_kv, DecParams p) {
    constexpr int kDChunks = D / 64;
    constexpr int kChunkBytes = kDecTile * 128;                 // [128 tokens x 64 d]
    constexpr int kKvBytes = kDChunks * kChunkBytes;            // one K or V tile
    constexpr int kQBytes = kDChunks * kDecN * 128;
    constexpr int kPBytes = 2 * kDecN * 128;                    // Pᵀ: [16 cols x 128 tokens] bf16, two 64-token chunks
    constexpr int kTmemCols = 64;                               // S0 @0, S1 @16, O @32 (16 columns each)
    constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* s_k = smem;
    uint8_t* s_v = s_k + KS * kKvBytes;
    uint8_t* s_q = s_v + VS * kKvBytes;
    uint8_t* s_p = s_q + ((kQBytes + 1023) & ~1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_p + 2 * kPBytes);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;
    uint64_t* k_empty = k_full + KS;
    uint64_t* v_full = k_empty + KS;
    uint64_t* v_empty = v_full + VS;
    uint64_t* s_full = v_empty + VS;
    uint64_t* s_free = s_full + 2;
    uint64_t* p_full = s_free + 2;
    uint64_t* p_free = p_full + 2;
    uint64_t* o_bar = p_free + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_bar + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* s_red = reinterpret_cast<float*>(tmem_slot + 4);     // [2 parities][4 warps][16] column maxima, then sums

    pdl_prologue();          // step metadata and Q/KV are produced by earlier kernels
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int kvh = blockIdx.x;
    const int seq = blockIdx.y / p.splits;
    const int split = blockIdx.y - seq * p.splits;
    const int qlen = p.q_len[seq];
    const int past = p.past_len[seq];
    const int qrow0 = p.q_start[seq];
    if (qlen <= 0) return;

    const int kv_end = past + qlen;
    int tile_lo = 0;
    if (p.window > 0) tile_lo = max(0, past - p.window + 1) / kDecTile;
    const int tile_hi_all = (kv_end + kDecTile - 1) / kDecTile;
    const int per = (tile_hi_all - tile_lo + p.splits - 1) / p.splits;
    const int j0 = tile_lo + split * per;
    const int j1 = min(tile_hi_all, j0 + per);
    const int ntiles = max(0, j1 - j0);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < KS; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
        }
        for (int s = 0; s < VS; ++s) {
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
    for (int i = threadIdx.x; i < 2 * kPBytes / 16; i += blockDim.x) reinterpret_cast<uint4*>(s_p)[i] = make_uint4(0, 0, 0, 0);
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------ producer ------------------------------
        if (lane == 0 && ntiles > 0) {
            // Q columns: (query token qi, head g) → row qi*G + g of a [16 x D] K-major tile
            mbar_expect_tx(q_full, kQBytes);
#pragma unroll
            for (int c = 0; c < kDChunks; ++c)
                tma_load_3d(s_q + c * (kDecN * 128), &tma_q, q_full, c * 64, kvh * p.group, qrow0);
            const int pages_per_tile = kDecTile / p.page_size;          // 2 for 64-token pages, 1 for 128
            const int rows_per_load = kDecTile / pages_per_tile;
            for (int j = 0; j < ntiles; ++j) {
                const int ks = j % KS, vs = j % VS;
                const uint32_t kph = ((j / KS) & 1) ^ 1, vph = ((j / VS) & 1) ^ 1;
                const int tile = j0 + j;
                int rows[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    int page = -1;
                    const int lp = tile * pages_per_tile + h;
                    if (h < pages_per_tile && lp < p.max_pages) page = p.page_table[(size_t)seq * p.max_pages + lp];
                    if (page < 0) page = 0;                              // masked anyway
                    rows[h] = ((page * 2 + 0) * p.hkv + kvh) * p.page_size;
                }
                if (!mbar_wait(&k_empty[ks], kph, abort_flag, p.status, kStatusProducerTimeout)) break;
                mbar_expect_tx(&k_full[ks], kKvBytes);
                for (int h = 0; h < pages_per_tile; ++h)
#pragma unroll
                    for (int c = 0; c < kDChunks; ++c)
                        tma_load_2d(s_k + ks * kKvBytes + c * kChunkBytes + h * rows_per_load * 128, &tma_kv, &k_full[ks],
                                    c * 64, rows[h]);
                if (!mbar_wait(&v_empty[vs], vph, abort_flag, p.status, kStatusProducerTimeout)) break;
                mbar_expect_tx(&v_full[vs], kKvBytes);
                for (int h = 0; h < pages_per_tile; ++h)
#pragma unroll
                    for (int c = 0; c < kDChunks; ++c)
                        tma_load_2d(s_v + vs * kKvBytes + c * kChunkBytes + h * rows_per_load * 128, &tma_kv, &v_full[vs],
                                    c * 64, rows[h] + p.hkv * p.page_size);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0 && ntiles > 0) {
            const uint32_t idesc_s = idesc_f16(128, kDecN, kBf16);                    // A = K (K-major), B = Q (K-major)
            const uint32_t idesc_o = idesc_f16(128, kDecN, kBf16, /*a_mn_major=*/true);   // A = Vᵀ (MN-major), B = Pᵀ (K-major)
            auto issue_s = [&](int j) {
                const int stage = j % KS;
                const uint64_t dk = smem_desc_sw128(s_k + stage * kKvBytes);
                const uint64_t dq = smem_desc_sw128(s_q);
                const uint32_t d_tmem = tmem_base + (j & 1) * 16;
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const int c = k >> 2, kk = k & 3;
                    umma_f16(d_tmem, dk + (uint64_t)((c * kChunkBytes) >> 4) + 2 * kk, dq + (uint64_t)((c * kDecN * 128) >> 4) + 2 * kk,
                             idesc_s, k > 0 ? 1u : 0u);
                }
                umma_commit(&k_empty[stage]);
                umma_commit(&s_full[j & 1]);
            };
            bool ok = mbar_wait(q_full, 0, abort_flag, p.status, kStatusMmaTimeout) &&
                      mbar_wait(&k_full[0], 0, abort_flag, p.status, kStatusMmaTimeout);
            if (ok) {
                tc_fence_after_sync();
                issue_s(0);
            }
            for (int j = 0; j < ntiles && ok; ++j) {
                if (j + 1 < ntiles) {
                    const int jn = j + 1;
                    ok = mbar_wait(&k_full[jn % KS], (jn / KS) & 1, abort_flag, p.status, kStatusMmaTimeout) &&
                         mbar_wait(&s_free[jn & 1], ((jn >> 1) & 1) ^ 1, abort_flag, p.status, kStatusMmaTimeout);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_s(jn);
                }
                const int stage = j % VS;
                ok = mbar_wait(&p_full[j & 1], (j >> 1) & 1, abort_flag, p.status, kStatusMmaTimeout) &&
                     mbar_wait(&v_full[stage], (j / VS) & 1, abort_flag, p.status, kStatusMmaTimeout);
                if (!ok) break;
                tc_fence_after_sync();
                // A = Vᵀ: 64-wide d chunks are kChunkBytes apart (leading offset), 8-token groups 1024 B apart
                const uint64_t dv = smem_desc_sw128_mn(s_v + stage * kKvBytes, kChunkBytes, 1024);
                const uint64_t dp = smem_desc_sw128(s_p + (j & 1) * kPBytes);
#pragma unroll
                for (int k = 0; k < kDecTile / 16; ++k)     // 16 tokens per MMA: 2048 B of V rows, 32 B of a P row
                    umma_f16(tmem_base + 32, dv + (uint64_t)((k * 2048) >> 4), dp + (uint64_t)(((k >> 2) * (kDecN * 128)) >> 4) + 2 * (k & 3),
                             idesc_o, (j > 0 || k > 0) ? 1u : 0u);
                umma_commit(&v_empty[stage]);
                umma_commit(&p_free[j & 1]);
                umma_commit(o_bar);
            }
        }
    } else {
        // ------------------------------ softmax / epilogue ------------------------------
        const int quad = warp & 3;
        const int r = quad * 32 + lane;                 // cached token within the tile == TMEM lane (S); feature d (O)
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
        const int ncol = qlen * p.group;                // live columns (<= 16)
        const int gshift = 31 - __clz(p.group);         // the group size is a power of two
        float m_used[NC], l_part[NC];
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            m_used[c] = -INFINITY;
            l_part[c] = 0.f;
        }
        bool ok = true;
        for (int j = 0; j < ntiles && ok; ++j) {
            const int b = j & 1;
            if (!mbar_wait(&s_full[b], (j >> 1) & 1, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
            tc_fence_after_sync();
            uint32_t raw[NC];
            tmem_ld_n<NC>(lane_addr + b * 16, raw);
            tmem_ld_wait();
            tc_fence_before_sync();
            mbar_arrive(&s_free[b]);
            const int tk = (j0 + j) * kDecTile + r;     // absolute cache slot of this thread's token
            float s[NC];
            float* red = s_red + b * 64;
            // Only the live columns (query tokens x heads of this sequence) are processed; `ncol`
            // is uniform across the CTA, so the guards below do not diverge.
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                if (c < ncol) {
                    const int qi = c >> gshift;
                    bool vis = tk <= past + qi;
                    if (p.window > 0) vis = vis && tk > past + qi - p.window;
                    s[c] = vis ? __uint_as_float(raw[c]) * p.scale_log2 : -INFINITY;
                    const float wm = warp_max_f32(s[c]);
                    if (lane == c) red[(warp - 2) * 16 + c] = wm;
                } else {
                    s[c] = -INFINITY;
                }
            }
            named_barrier_sync(1, 128);
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
            // P buffer b is free once PV(j-2) has completed.  This wait is taken for every use of the buffer, so its
            // parity is exact; it also pins how far the tensor pipe can lag behind this warp.
            if (!mbar_wait(&p_free[b], ((j >> 1) & 1) ^ 1, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
            if (j > 0 && any_need) {
                // O may only be rescaled after PV(j-1) has landed: that is the next completion of the other P
                // buffer's barrier (a parity wait on a barrier that is polled only now and then could alias).
                if (!mbar_wait(&p_free[b ^ 1], ((j - 1) >> 1) & 1, abort_flag, p.status, kStatusEpilogueTimeout)) { ok = false; break; }
                tc_fence_after_sync();
                uint32_t o[NC];
                tmem_ld_n<NC>(lane_addr + 32, o);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < NC; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * f[c]);
                tmem_st_n<NC>(lane_addr + 32, o);
                tmem_st_wait();
                tc_fence_before_sync();
            }
            // Pᵀ[c][token]: row c is 128 tokens = two 128-byte swizzled chunks of 64 tokens.  Dead
            // columns keep whatever the buffer holds; their outputs are never read.
            uint8_t* pbase = s_p + b * kPBytes + (r >> 6) * (kDecN * 128);
            const int tl = r & 63;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                if (c < ncol) {
                    const float mref = m_used[c] == -INFINITY ? 0.f : m_used[c];
                    const float e = exp2f(s[c] - mref);
                    l_part[c] += e;
                    T* dst = reinterpret_cast<T*>(pbase + (c >> 3) * 1024 + (c & 7) * 128 + ((((tl >> 3) ^ (c & 7)) & 7) << 4) + (tl & 7) * 2);
                    *dst = Cvt<T>::from_f(e);
                }
            }
            fence_proxy_async_smem();
            mbar_arrive(&p_full[b]);
        }
        // ---- epilogue: column sums across the 128 threads, then O / l ----
        float* red = s_red;         // reuse: [4 warps][16]
        named_barrier_sync(1, 128);
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            float v = l_part[c];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == c) red[(warp - 2) * 16 + c] = v;
        }
        named_barrier_sync(1, 128);
        // every PV has completed once the last tile's commit has: commits complete in issue order
        if (ok && ntiles > 0)
            ok = mbar_wait(&p_free[(ntiles - 1) & 1], ((ntiles - 1) >> 1) & 1, abort_flag, p.status, kStatusEpilogueTimeout);
        if (ok) {
            tc_fence_after_sync();
            uint32_t o[NC];
            if (ntiles > 0) {
                tmem_ld_n<NC>(lane_addr + 32, o);
                tmem_ld_wait();
            }
            if (r < D) {
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    if (c < ncol) {
                        const float l = red[c] + red[16 + c] + red[32 + c] + red[48 + c];
                        const float val = (ntiles > 0 && l > 0.f) ? __uint_as_float(o[c]) / l : 0.f;
                        const int qi = c >> gshift, g = c - (qi << gshift);
                        const size_t tok = (size_t)qrow0 + qi;
                        const int head = kvh * p.group + g;
                        if (p.splits == 1) {
                            reinterpret_cast<T*>(p.out)[(tok * p.hq + head) * D + r] = Cvt<T>::from_f(val);
                        } else {
                            p.ws_o[(((size_t)split * p.total_tokens + tok) * p.hq + head) * D + r] = val;
                            if (r == 0)
                                p.ws_lse[((size_t)split * p.total_tokens + tok) * p.hq + head] =
                                    (ntiles > 0 && l > 0.f) ? m_used[c] + log2f(l) : -INFINITY;
                        }
                    }
                }
            }
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

template <int D, typename T, int KS, int VS, int MINB, int NC>
static int launch_decode_variant(const CUtensorMap& tq, const CUtensorMap& tkv, const DecParams& p, int nseq, cudaStream_t stream) {
    constexpr int kv = (D / 64) * kDecTile * 128;
    constexpr int smem = (KS + VS) * kv + 4096 + 2 * 2 * kDecN * 128 + 1024 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<D, T, KS, VS, MINB, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail("cudaFuncSetAttribute(attn_decode)", e);
        configured = true;
    }
    dim3 grid(p.hkv, nseq * p.splits);
    TELB_LAUNCH("attn_decode_kernel", (attn_decode_kernel<D, T, KS, VS, MINB, NC>), dim3(grid), dim3(kDecThreads), smem, stream, tq, tkv, p);
    TELB_CHECK_LAUNCH("attn_decode_kernel");
    return 0;
}

static int g_decode_variant = 1;      // measured fastest at batch 8..64 with 1k context

template <int D, typename T, int NC>
static int launch_decode_nc(const CUtensorMap& tq, const CUtensorMap& tkv, const DecParams& p, int nseq, cudaStream_t stream) {
    switch (g_decode_variant) {
        case 1: return launch_decode_variant<D, T, 1, 1, 2, NC>(tq, tkv, p, nseq, stream);     // 2 CTAs / SM, single-stage rings
        case 2: return launch_decode_variant<D, T, 2, 1, 2, NC>(tq, tkv, p, nseq, stream);     // 2 CTAs / SM, K prefetched one tile ahead
        default: return launch_decode_variant<D, T, 3, 3, 1, NC>(tq, tkv, p, nseq, stream);    // 1 CTA / SM, three-stage rings
    }
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

// Ring depth / residency variant of the decode kernel (0, 1 or 2: see launch_decode); process-wide.
extern "C" int telb_set_decode_variant(int v) {
    if (v < 0 || v > 2) return fail("telb_set_decode_variant: variant must be 0, 1 or 2");
    g_decode_variant = v;
    return 0;
}

// Decode-shaped steps only: max_q_len * (Hq/Hkv) <= 16.  Same tensors as telb_paged_attention.
extern "C" int telb_paged_attention_decode(const void* q, const void* kv_layer, void* out, const int* q_start,
                                           const int* q_len, const int* past_len, const int* page_table, int num_seqs,
                                           int total_tokens, int max_q_len, int num_pages, int max_pages, int page_size,
                                           int hq, int hkv, int d, float scale, int window, int splits, float* ws,
                                           long long ws_floats, int is_bf16, int* status, cudaStream_t stream) {
    if (num_seqs <= 0 || total_tokens <= 0) return 0;
    if (d != 128) return fail("telb_paged_attention_decode: head_dim must be 128");
    if (page_size != 64 && page_size != 128) return fail("telb_paged_attention_decode: page size must be 64 or 128");
    if (hq % hkv) return fail("telb_paged_attention_decode: Hq must be a multiple of Hkv");
    const int group = hq / hkv;
    if (max_q_len * group > kDecN) return fail("telb_paged_attention_decode: q_len * (Hq/Hkv) must be <= 16");
    if (kDecN % group) return fail("telb_paged_attention_decode: Hq/Hkv must divide 16");
    DecParams p{};
    p.out = out;
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
    if (splits < 1) splits = 1;
    if (splits > 32) splits = 32;
    while (splits > 1 && (long long)splits * total_tokens * hq * (d + 1) > ws_floats) --splits;
    p.splits = splits;
    p.ws_o = ws;
    p.ws_lse = ws ? ws + (size_t)splits * total_tokens * hq * d : nullptr;
    const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap tq, tkv;
    {
        // Q viewed as [tokens][Hq][D]; one box = (64 features, G heads, 16/G tokens) → 16 rows of 128 B
        const uint64_t dims[3] = {(uint64_t)d, (uint64_t)hq, (uint64_t)total_tokens};
        const uint64_t strides[2] = {(uint64_t)d * 2, (uint64_t)hq * d * 2};
        const uint32_t box[3] = {64, (uint32_t)group, (uint32_t)(kDecN / group)};
        if (make_tmap_nd(&tq, dt, 3, q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    }
    {
        const uint64_t rows = (uint64_t)num_pages * 2 * hkv * page_size;
        const uint32_t box_rows = page_size == 64 ? 64 : 128;
        if (make_tmap_2d(&tkv, dt, 2, kv_layer, rows, d, (uint64_t)d * 2, box_rows, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    }
    const int rc = is_bf16 ? launch_decode<128, __nv_bfloat16>(tq, tkv, p, num_seqs, max_q_len * group, stream)
                           : launch_decode<128, __half>(tq, tkv, p, num_seqs, max_q_len * group, stream);
    if (rc) return rc;
    if (splits > 1) return telb_attn_combine(p.ws_o, p.ws_lse, out, total_tokens * hq, splits, d, is_bf16, stream);
    return 0;
}
