// NVFP4 block-scaled GEMM for prefill-size M with 256-wide output tiles, as a single CTA (128 x 256) or as a
// CTA pair (`tcgen05.mma.cta_group::2`, 256 x 256 per pair):
//     out[M,N] = (xq ⊙ sfx)[M,K] · (wq ⊙ sfw)[N,K]ᵀ · alpha[N]  (+ bias, + residual)
//
// Why a second kernel next to gemm_nvfp4_tc5.cu: with 128 x 128 tiles the block-scaled tensor pipe waits for
// shared memory to fill — a K step of 256 moves 36 KB from L2 per 8.4 MFLOP, which at the fp4 rate asks for
// more L2 → SM bandwidth than the chip has.  A pair of CTAs on neighbouring SMs that issues one 256 x 256 MMA
// needs, per CTA and K step, only its own 128 A rows, HALF of the B tile (the tensor cores of both SMs read
// both halves in place) and the scales: 38 KB per 16.8 MFLOP, 1.9x the arithmetic per byte.  The single-CTA
// form (54 KB per 16.8 MFLOP) is kept as the fallback when clusters of two cannot be scheduled.
//
// No TMA load in this file uses cluster multicast (this kernel runs inside tensor-parallel steps at world
// sizes above one): each CTA fetches its own A rows, its own half of B and its own copy of the scales.  The
// only cluster-scoped operations are `tcgen05.commit ... multicast::cluster` (an mbarrier arrive in both CTAs
// of the pair), remote `mbarrier.arrive` and the cluster barrier.
//
// TMEM plan (512 columns): two 256-column fp32 accumulators cannot sit beside the scale-factor columns, so
// the second accumulator starts at column 128 and overlaps the first by 128 columns.  The epilogue of a tile
// drains the half that the next tile's accumulator needs first and signals it (`tovl`), so the next main loop
// starts while the other half is still being converted and stored:
//     columns [0,256) accumulator 0, [128,384) accumulator 1, [384,480) two scale buffers of 48 columns.
//
// Pair protocol: both CTAs run the same tile sequence.  Each CTA's producer warp fills its own stage ring
// with `cp.async.bulk.tensor ... .cta_group::2` loads (no multicast) whose byte counts complete on the
// LEADER's "stage full" barrier, armed by the leader for both CTAs' bytes; the scale atoms travel as tiled
// loads over a [atoms, 512 B] view of the scale buffers for the same reason.  CTA 0 (the leader) issues every
// `tcgen05.cp` / `tcgen05.mma` (with `.cta_group::2` they act on both CTAs' shared memory and TMEM).  Stage
// release and "accumulator full" reach both CTAs through the multicast commit; "accumulator drained" comes
// back from all 256 epilogue threads of the pair as arrives on the leader's barriers.  Every wait is bounded,
// as in the other kernels.
//
// Fusions carried over from the 128-wide kernel: reduce-scatter epilogue (rows leave as 128-byte lines to
// their owner rank's buffer), all-gather prologue (the producer waits for the rows' owner flags), SwiGLU +
// NVFP4 quantisation of the next GEMM's input on 64-row gate / up interleaved weights.
//
// Reference counterparts: CuTe-DSL `gemm_blackwell_nvfp4_ws.py` and the 256 x 256 two-CTA registrations of
// kernelSrcs/build_cutedsl.py:2164-2332; this kernel is written from the PTX up.
#include "gemm_common.cuh"
#include "nvfp4_common.cuh"

namespace telb {

constexpr int kWBN = 256;
constexpr int kWAcc1 = 128;                 // first column of accumulator 1
constexpr int kWSf0 = 384;                  // first scale-factor column
constexpr int kWSfCols = 48;                // SFA 16 + SFB 32 per buffer
constexpr int kWTmemCols = 512;

template <bool PAIR>
struct WideCfg {
    static constexpr int kTileM = PAIR ? 256 : 128;
    static constexpr int kBRows = PAIR ? 128 : 256;          // B rows one CTA keeps in shared memory
    static constexpr int kATile = 128 * 128;
    static constexpr int kBTile = kBRows * 128;
    static constexpr int kSfA = 2048;
    static constexpr int kSfB = 4096;
    static constexpr int kStage = kATile + kBTile + kSfA + kSfB;
    static constexpr int kStages = PAIR ? 5 : 3;
    static constexpr int kNumBars = 3 * kStages + 6;
    static constexpr int kSmem = kStages * kStage + 1024 + 256 + kRsStageBytes;
};

__device__ __forceinline__ uint32_t cluster_ctarank_w() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_w() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the barrier at the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t* bar, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(bar)), "r"(rank));
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
// Shared-memory address of `ptr`'s counterpart in CTA `rank` of the cluster (shared::cluster window).
__device__ __forceinline__ uint32_t cluster_addr_of(const void* ptr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(ptr)), "r"(rank));
    return remote;
}
// Tiled TMA load of a CTA pair (no multicast): the data lands in THIS CTA's shared memory, the byte count completes on the
// mbarrier at `bar_cluster_addr`, which may belong to the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
// ---- cta_group::2 forms ------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_nvfp4_2(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t tmem_sfa,
                                             uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
}
__device__ __forceinline__ void tmem_cp_sf2(uint32_t tmem_dst, uint64_t desc_src) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(desc_src) : "memory");
}
// One arrive on `bar` in every CTA of `mask` once all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit2(uint64_t* bar, uint16_t mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

struct WideTile {
    int a0, b0, tb;        // first row of the (pair) tile, first column, column-tile index
};
template <int TILE_M>
__device__ __forceinline__ WideTile wide_tile(const GemmParams& p, int t) {
    const int per_group = kRasterGroup * p.tiles_b;
    const int group = t / per_group;
    const int within = t - group * per_group;
    const int gfirst = group * kRasterGroup;
    const int gsize = min(kRasterGroup, p.tiles_a - gfirst);
    WideTile w;
    w.a0 = (gfirst + within % gsize) * TILE_M;
    w.tb = within / gsize;
    w.b0 = w.tb * kWBN;
    return w;
}

template <bool PAIR>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_nvfp4_wide_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                       const __grid_constant__ CUtensorMap tma_sfa, const __grid_constant__ CUtensorMap tma_sfb,
                       const uint8_t* __restrict__ sf_a, const uint8_t* __restrict__ sf_b, int sf_k64_a, int sf_k64_b, GemmParams p) {
    using Cfg = WideCfg<PAIR>;
    constexpr int STAGES = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::kStage);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* peer_full = empty_bar + STAGES;          // leader only: the other CTA's stage is full
    uint64_t* tfull_bar = peer_full + STAGES;
    uint64_t* tempty_bar = tfull_bar + 2;
    uint64_t* tovl_bar = tempty_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tovl_bar + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    uint8_t* rs_stage = smem + STAGES * Cfg::kStage + 256;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t crank = PAIR ? cluster_ctarank_w() : 0u;
    const bool leader = crank == 0;
    const int ncta = PAIR ? 2 : 1;
    const int cid = blockIdx.x / ncta, ncl = gridDim.x / ncta;
    const int total_tiles = p.tiles_a * p.tiles_b;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
            mbar_init(&peer_full[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tfull_bar[s], 1);
            mbar_init(&tempty_bar[s], 128 * ncta);
            mbar_init(&tovl_bar[s], 128 * ncta);
        }
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tensormap(&tma_a);
        prefetch_tensormap(&tma_b);
        if constexpr (PAIR) {
            prefetch_tensormap(&tma_sfa);
            prefetch_tensormap(&tma_sfb);
        }
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            tmem_alloc2(tmem_slot, kWTmemCols);
            tmem_relinquish2();
        } else {
            tmem_alloc(tmem_slot, kWTmemCols);
            tmem_relinquish();
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_w();       // both CTAs' barriers and TMEM exist before anything crosses the pair
    tc_fence_after_sync();
    pdl_prologue();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- producer: this CTA's A rows, its part of B, its scale atoms ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const int ag_e = p.ag_flags ? *p.ag_epoch : 0;
            const int last_a_tile = (p.rows_a - 1) / 128, last_b_tile = (p.rows_b - 1) / 128;
            for (int t = cid; t < total_tiles && ok; t += ncl) {
                const WideTile w = wide_tile<Cfg::kTileM>(p, t);
                const int a0 = w.a0 + (int)crank * 128;
                const int brow = w.b0 + (PAIR ? (int)crank * 128 : 0);
                if (p.ag_flags && a0 < p.rows_a && !ag_wait_rows(p, a0, ag_e, abort_flag)) break;
                const int ta = min(a0 / 128, last_a_tile);
                const int tb0 = min(w.b0 / 128, last_b_tile), tb1 = min(w.b0 / 128 + 1, last_b_tile);
                for (int kb = 0; kb < p.kb_total; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + stage * Cfg::kStage;
                    uint8_t* sb = sa + Cfg::kATile;
                    uint8_t* ssa = sb + Cfg::kBTile;
                    uint8_t* ssb = ssa + Cfg::kSfA;
                    if constexpr (PAIR) {
                        // every load of both CTAs completes on the LEADER's barrier (armed by the leader for both stages'
                        // bytes), so the issuer learns that the pair's operands are in place without a relay hop; the scale
                        // atoms travel as tiled loads too (rows of 512 bytes), since only those can signal the peer's barrier
                        const uint32_t fb = cluster_addr_of(&full_bar[stage], 0);
                        if (leader) mbar_expect_tx(&full_bar[stage], 2 * Cfg::kStage);
                        tma_load_2d_pair(sa, &tma_a, fb, kb * 128, a0);
                        tma_load_2d_pair(sb, &tma_b, fb, kb * 128, brow);
                        tma_load_2d_pair(ssa, &tma_sfa, fb, 0, ta * sf_k64_a + kb * 4);
                        tma_load_2d_pair(ssb, &tma_sfb, fb, 0, tb0 * sf_k64_b + kb * 4);
                        tma_load_2d_pair(ssb + 2048, &tma_sfb, fb, 0, tb1 * sf_k64_b + kb * 4);
                    } else {
                        mbar_expect_tx(&full_bar[stage], Cfg::kStage);
                        tma_load_2d(sa, &tma_a, &full_bar[stage], kb * 128, a0);
                        tma_load_2d(sb, &tma_b, &full_bar[stage], kb * 128, brow);
                        bulk_load(ssa, sf_a + ((size_t)ta * sf_k64_a + (size_t)kb * 4) * 512, 2048, &full_bar[stage]);
                        bulk_load(ssb, sf_b + ((size_t)tb0 * sf_k64_b + (size_t)kb * 4) * 512, 2048, &full_bar[stage]);
                        bulk_load(ssb + 2048, sf_b + ((size_t)tb1 * sf_k64_b + (size_t)kb * 4) * 512, 2048, &full_bar[stage]);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            // ---------------- UMMA issuer (leader CTA) ----------------
            const uint32_t idesc = idesc_nvfp4(Cfg::kTileM, kWBN);
            int stage = 0;
            uint32_t phase = 0, sf_par = 0;
            bool ok = true;
            int i = 0;
            for (int t = cid; t < total_tiles && ok; t += ncl, ++i) {
                const int acc = i & 1;
                const uint32_t use_par = (uint32_t)(i >> 1) & 1u;
                // the accumulator's previous tile is fully drained, and the previous tile's overlapping half is drained
                if (!mbar_wait(&tempty_bar[acc], use_par ^ 1, abort_flag, p.status, kStatusMmaTimeout)) break;
                if (i > 0 && !mbar_wait(&tovl_bar[acc ^ 1], (uint32_t)((i - 1) >> 1) & 1u, abort_flag, p.status, kStatusMmaTimeout)) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (acc ? kWAcc1 : 0);
                for (int kb = 0; kb < p.kb_total; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kStatusMmaTimeout)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint8_t* sa = smem + stage * Cfg::kStage;
                    const uint8_t* sb = sa + Cfg::kATile;
                    const uint8_t* ssa = sb + Cfg::kBTile;
                    const uint8_t* ssb = ssa + Cfg::kSfA;
                    const uint32_t t_sfa = tmem_base + kWSf0 + sf_par * kWSfCols;
                    const uint32_t t_sfb = t_sfa + 16;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if constexpr (PAIR) {
                            tmem_cp_sf2(t_sfa + q * 4, smem_desc_sf(ssa + q * 512));
                            tmem_cp_sf2(t_sfb + q * 8, smem_desc_sf(ssb + q * 512));
                            tmem_cp_sf2(t_sfb + q * 8 + 4, smem_desc_sf(ssb + 2048 + q * 512));
                        } else {
                            tmem_cp_sf(t_sfa + q * 4, smem_desc_sf(ssa + q * 512));
                            tmem_cp_sf(t_sfb + q * 8, smem_desc_sf(ssb + q * 512));
                            tmem_cp_sf(t_sfb + q * 8 + 4, smem_desc_sf(ssb + 2048 + q * 512));
                        }
                    }
                    const uint64_t da = smem_desc_sw128(sa);
                    const uint64_t db = smem_desc_sw128(sb);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t accum = (kb > 0 || q > 0) ? 1u : 0u;
                        if constexpr (PAIR) umma_nvfp4_2(d_tmem, da + 2 * q, db + 2 * q, idesc, t_sfa + q * 4, t_sfb + q * 8, accum);
                        else umma_nvfp4(d_tmem, da + 2 * q, db + 2 * q, idesc, t_sfa + q * 4, t_sfb + q * 8, accum);
                    }
                    if constexpr (PAIR) umma_commit2(&empty_bar[stage], 3);
                    else umma_commit(&empty_bar[stage]);
                    sf_par ^= 1;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                if constexpr (PAIR) umma_commit2(&tfull_bar[acc], 3);
                else umma_commit(&tfull_bar[acc]);
            }
        }
    } else {
        // ---------------- epilogue (warps 2-5): lane quadrant q owns accumulator rows 32 q .. 32 q + 31 ----------------
        const int quad = warp & 3;
        const int lrow = quad * 32 + lane;
        int i = 0;
        for (int t = cid; t < total_tiles; t += ncl, ++i) {
            const WideTile w = wide_tile<Cfg::kTileM>(p, t);
            const int acc = i & 1;
            const uint32_t use_par = (uint32_t)(i >> 1) & 1u;
            if (!mbar_wait(&tfull_bar[acc], use_par, abort_flag, p.status, kStatusEpilogueTimeout)) break;
            tc_fence_after_sync();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + (acc ? kWAcc1 : 0);
            const int row = w.a0 + (int)crank * 128 + lrow;
            const bool row_ok = row < p.rows_a;
            const int b0 = w.b0;
#pragma unroll 1
            for (int hh = 0; hh < 2; ++hh) {
                // accumulator 0 gives up its upper half first (accumulator 1 begins there), accumulator 1 its lower half
                const int h = acc ? hh : (hh ^ 1);
                const int hb0 = b0 + h * 128;                      // first output column of this half
                const uint32_t h_addr = t_addr + h * 128;
                if (p.sw_xq != nullptr) {
                    // columns [0,64) of the half: gate features f0 .. f0+63, columns [64,128): the matching up features
                    const float gs = *p.sw_gs;
                    const float inv_gs = 1.f / gs;
                    const int f0 = (w.tb * 2 + h) * 64;
#pragma unroll 1
                    for (int c = 0; c < 2; ++c) {
                        uint32_t rg[32], ru[32];
                        tmem_ld_x32(h_addr + c * 32, rg);
                        tmem_ld_x32(h_addr + 64 + c * 32, ru);
                        tmem_ld_wait();
                        if (row_ok && hb0 + 128 <= p.rows_b) {
#pragma unroll
                            for (int hf = 0; hf < 2; ++hf) {
                                float y[16];
                                float amax = 0.f;
#pragma unroll
                                for (int k = 0; k < 16; ++k) {
                                    const int j = hf * 16 + k;
                                    float g = __uint_as_float(rg[j]), u = __uint_as_float(ru[j]);
                                    if (p.alpha) {
                                        g *= p.alpha[hb0 + c * 32 + j];
                                        u *= p.alpha[hb0 + 64 + c * 32 + j];
                                    }
                                    // the same roundings as the unfused chain: 16-bit GEMM output, 16-bit activation, then quantise
                                    if (p.out_bf16) {
                                        g = Cvt<__nv_bfloat16>::to_f(Cvt<__nv_bfloat16>::from_f(g));
                                        u = Cvt<__nv_bfloat16>::to_f(Cvt<__nv_bfloat16>::from_f(u));
                                        y[k] = Cvt<__nv_bfloat16>::to_f(Cvt<__nv_bfloat16>::from_f(g / (1.f + __expf(-g)) * u));
                                    } else {
                                        g = Cvt<__half>::to_f(Cvt<__half>::from_f(g));
                                        u = Cvt<__half>::to_f(Cvt<__half>::from_f(u));
                                        y[k] = Cvt<__half>::to_f(Cvt<__half>::from_f(g / (1.f + __expf(-g)) * u));
                                    }
                                    amax = fmaxf(amax, fabsf(y[k]));
                                }
                                uint8_t s8;
                                const uint2 packed = nvfp4_quantize_block16(y, amax, gs, inv_gs, s8);
                                const int blk = (f0 + c * 32 + hf * 16) >> 4;
                                *reinterpret_cast<uint2*>(p.sw_xq + (size_t)row * p.sw_ld + blk * 8) = packed;
                                p.sw_sf[sf_atom_offset((long long)row, blk, p.sw_k64_pad)] = s8;
                            }
                        }
                    }
                } else if (p.rs_world > 1) {
                    // reduce-scatter: two 32-column chunks are transposed through a per-warp slab of shared memory and leave
                    // as whole 128-byte lines to the owner rank's partial buffer, four rows per store instruction
                    uint8_t* slab = rs_stage + quad * (32 * kRsStageRowBytes);
                    const int seg = lane & 7, rsub = lane >> 3;
#pragma unroll 1
                    for (int c = 0; c < 4; c += 2) {
#pragma unroll
                        for (int s2 = 0; s2 < 2; ++s2) {
                            uint32_t r[32];
                            tmem_ld_x32(h_addr + (c + s2) * 32, r);
                            tmem_ld_wait();
                            float v[32];
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                            uint4 u[4];
                            const int col0 = min(hb0 + (c + s2) * 32, max(p.rows_b - 32, 0));   // clamp: columns past N are not stored
                            if (p.out_bf16) pack_chunk<__nv_bfloat16>(p, v, col0, u);
                            else pack_chunk<__half>(p, v, col0, u);
                            uint4* dst = reinterpret_cast<uint4*>(slab + lane * kRsStageRowBytes + s2 * 64);
#pragma unroll
                            for (int q = 0; q < 4; ++q) dst[q] = u[q];
                        }
                        __syncwarp();
                        const int colseg = hb0 + c * 32 + seg * 8;
#pragma unroll
                        for (int rr = 0; rr < 32; rr += 4) {
                            const int lr = rr + rsub;
                            const int grow = w.a0 + (int)crank * 128 + quad * 32 + lr;
                            if (grow < p.rows_a && colseg + 8 <= p.rows_b) {
                                const int d = grow / p.rs_rows_per_rank;
                                const size_t orow = (size_t)p.rs_rank * p.rs_rows_per_rank + (grow - d * p.rs_rows_per_rank);
                                const uint4 val = *reinterpret_cast<const uint4*>(slab + lr * kRsStageRowBytes + seg * 16);
                                uint16_t* base = reinterpret_cast<uint16_t*>(p.rs_out[d]);
                                *reinterpret_cast<uint4*>(base + orow * (size_t)p.ldc_lane + colseg) = val;
                            }
                        }
                        __syncwarp();
                    }
                } else {
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t r[32];
                        tmem_ld_x32(h_addr + c * 32, r);
                        tmem_ld_wait();
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                        const int col0 = hb0 + c * 32;
                        const int nvalid = min(32, p.rows_b - col0);
                        if (row_ok && nvalid > 0) {
                            if (p.out_bf16) epilogue_store<__nv_bfloat16>(p, v, row, col0, nvalid);
                            else epilogue_store<__half>(p, v, row, col0, nvalid);
                        }
                    }
                }
                tc_fence_before_sync();
                if (hh == 0) {
                    if constexpr (PAIR) mbar_arrive_cluster(&tovl_bar[acc], 0);
                    else mbar_arrive(&tovl_bar[acc]);
                } else {
                    if constexpr (PAIR) mbar_arrive_cluster(&tempty_bar[acc], 0);
                    else mbar_arrive(&tempty_bar[acc]);
                }
            }
        }
        // the peer stores of the reduce-scatter epilogue are performed system-wide before the kernel ends, so the
        // "GEMM finished" flag the next kernel publishes can never overtake them
        if (p.rs_world > 1) __threadfence_system();
    }

    if (*abort_flag) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_w();       // the other CTA's tensor core may still be reading this CTA's tiles / TMEM
    if (warp == 1) {
        tc_fence_after_sync();
        if constexpr (PAIR) tmem_dealloc2(tmem_base, kWTmemCols);
        else tmem_dealloc(tmem_base, kWTmemCols);
    }
}

template <bool PAIR>
static int launch_wide(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsfa, const CUtensorMap& tsfb, const uint8_t* sfa,
                       const uint8_t* sfb, int k64a, int k64b, const GemmParams& p, cudaStream_t stream) {
    using Cfg = WideCfg<PAIR>;
    auto kern = gemm_nvfp4_wide_kernel<PAIR>;
    static int max_clusters = 0;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem);
        if (e != cudaSuccess) return fail("cudaFuncSetAttribute(gemm_nvfp4_wide)", e);
        if (PAIR) {
            // how many pairs can be resident at once: a pair needs two free SMs of one TPC / GPC, so it is queried, not assumed
            cudaLaunchConfig_t q{};
            q.gridDim = dim3(sm_count() / 2 * 2, 1, 1);
            q.blockDim = dim3(kGemmThreads, 1, 1);
            q.dynamicSmemBytes = Cfg::kSmem;
            cudaLaunchAttribute a[1];
            a[0].id = cudaLaunchAttributeClusterDimension;
            a[0].val.clusterDim.x = 2;
            a[0].val.clusterDim.y = 1;
            a[0].val.clusterDim.z = 1;
            q.attrs = a;
            q.numAttrs = 1;
            int n = 0;
            e = cudaOccupancyMaxActiveClusters(&n, kern, &q);
            if (e != cudaSuccess || n <= 0) {
                cudaGetLastError();
                n = sm_count() / 2;
            }
            max_clusters = n;
            if (getenv("TELB_DEBUG_CLUSTERS")) fprintf(stderr, "[telb] gemm_nvfp4_wide: %d CTA pairs can be resident (of %d SMs)\n", n, sm_count());
        } else {
            max_clusters = sm_count();
        }
        configured = true;
    }
    const int total = p.tiles_a * p.tiles_b;
    const int clusters = total < max_clusters ? total : max_clusters;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(clusters * (PAIR ? 2 : 1), 1, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    int na = 0;
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    if (pdl_enabled()) ++na;
    if (PAIR) {
        attrs[na].id = cudaLaunchAttributeClusterDimension;
        attrs[na].val.clusterDim.x = 2;
        attrs[na].val.clusterDim.y = 1;
        attrs[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, tsfa, tsfb, sfa, sfb, k64a, k64b, p);
    if (e != cudaSuccess) return fail("cudaLaunchKernelEx(gemm_nvfp4_wide)", e);
    return 0;
}

}  // namespace telb

using namespace telb;

// Which large-M NVFP4 kernel runs: 0 = 128 x 128 tiles (gemm_nvfp4_tc5.cu), 1 = 128 x 256 single CTA, 2 = 256 x 256 CTA pair.
// TELB_NVFP4_WIDE overrides the default.
static int g_wide_mode = -1;
extern "C" int telb_nvfp4_wide_mode() {
    if (g_wide_mode < 0) {
        const char* e = getenv("TELB_NVFP4_WIDE");
        g_wide_mode = (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 1;
    }
    return g_wide_mode;
}
// Tests and benchmarks switch kernels inside one process; returns the previous mode.
extern "C" int telb_set_nvfp4_wide_mode(int mode) {
    const int old = telb_nvfp4_wide_mode();
    if (mode >= 0 && mode <= 2) g_wide_mode = mode;
    return old;
}

// Large-M layout only (M > 128 is the caller's business; any M works).  `p` arrives with the epilogue / fusion fields set;
// this fills the tile geometry and launches.  pair = 0 → single CTA, 1 → CTA pair.
extern "C" int telb_gemm_nvfp4_wide_launch(const void* xq, const void* x_sf, const void* wq, const void* w_sf, int M, int N, int K,
                                           const void* params_blob, int pair, cudaStream_t stream) {
    GemmParams p = *static_cast<const GemmParams*>(params_blob);
    if (K % 32) return fail("telb_gemm_nvfp4_wide: K must be a multiple of 32");
    if (N % 8) return fail("telb_gemm_nvfp4_wide: N must be a multiple of 8");
    const uint64_t kbytes = (uint64_t)K / 2;
    p.k = K;
    p.kb_total = (K + 255) / 256;
    p.rows_a = M;
    p.rows_b = N;
    p.ldc_lane = N;
    p.ldc_col = 1;
    p.feat_on_lane = 0;
    p.splits = 1;
    p.kb_per_split = p.kb_total;
    const int tile_m = pair ? 256 : 128;
    p.tiles_a = (M + tile_m - 1) / tile_m;
    p.tiles_b = (N + kWBN - 1) / kWBN;
    const int k64 = ((K + 255) / 256) * 4;
    CUtensorMap ta, tb;
    if (make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, M, kbytes, kbytes, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    if (make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, N, kbytes, kbytes, pair ? 128 : 256, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    // the pair kernel fetches scale atoms with tiled loads: the scale buffers seen as rows of 512 bytes (128 x u32), four atoms
    // (one 256-element K step of one 128-row tile) per box
    CUtensorMap tsa = ta, tsb = tb;
    if (pair) {
        const uint64_t atoms_a = (uint64_t)((M + 127) / 128) * k64, atoms_b = (uint64_t)((N + 127) / 128) * k64;
        if (make_tmap_2d(&tsa, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, x_sf, atoms_a, 128, 512, 4, 128, CU_TENSOR_MAP_SWIZZLE_NONE)) return -1;
        if (make_tmap_2d(&tsb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, w_sf, atoms_b, 128, 512, 4, 128, CU_TENSOR_MAP_SWIZZLE_NONE)) return -1;
    }
    return pair ? launch_wide<true>(ta, tb, tsa, tsb, (const uint8_t*)x_sf, (const uint8_t*)w_sf, k64, k64, p, stream)
                : launch_wide<false>(ta, tb, tsa, tsb, (const uint8_t*)x_sf, (const uint8_t*)w_sf, k64, k64, p, stream);
}
