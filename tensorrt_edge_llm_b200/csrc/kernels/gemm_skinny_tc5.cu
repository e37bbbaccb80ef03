// Decode-size GEMM (M <= 128 tokens):  out[M,N] = x[M,K] · w[N,K]ᵀ · alpha (+bias, +residual),
// for 16-bit weights and for NVFP4 block-scaled weights/activations.
//
// A decode step is bound by streaming the weights once, and each projection is only a few
// microseconds of HBM traffic, so the design minimises the latency chain rather than FLOPs:
//   * operands are swapped: the 128-row MMA-M side holds weight rows, the token batch is MMA-N;
//   * K is split across the CTAs of a thread-block cluster (1 x S x 1); each CTA accumulates its
//     K-slice in TMEM, parks the fp32 partial tile in its own shared memory, and after one cluster
//     barrier every CTA reduces a slice of the token columns by reading its peers' shared memory
//     (distributed shared memory) — no global workspace, no atomics, no CTA waiting on a flag;
//   * ~96 KiB of shared memory per CTA so two CTAs share an SM and a 192-tile projection is one wave;
//   * programmatic dependent launch: the kernel is launched while its predecessor drains, issues
//     its weight-tile TMA loads immediately (weights never depend on the predecessor) and executes
//     `griddepcontrol.wait` only before touching activations or writing outputs.
// No TMA load here uses cluster multicast: every CTA fetches its own K-slice.
//
// Tensor-parallel fusion at decode size (both optional, same contract as the large-M kernels):
//   * reduce-scatter epilogue: the output row of token t belongs to rank t / rows_per_rank and is stored straight
//     into that rank's partial buffer over peer memory (256 contiguous bytes per warp and token), so the
//     row-parallel projection needs no copy-in, no pull and only 1/world of a one-shot all-reduce's bytes;
//   * all-gather prologue: the activation rows were pushed into this GPU's memory by their owner ranks; the
//     producer warp waits (bounded) for the owners' flags after `griddepcontrol.wait`, while the weight
//     tiles of the first ring pass are already in flight.
//
// Reference counterparts: TensorRT decode tactics; kernelSrcs/nvfp4A16BlackwellGemv (SM110-only
// CUDA-core GEMV) and `gemm_blackwell_nvfp4_ws_*_tn64` at TP=2.
#include "gemm_common.cuh"

namespace telb {

struct SkinnyParams {
    int n_out, m_tok, k;             // out features, tokens, reduction length
    int kb_total, kb_per_rank, ranks;
    void* out;                       // [m_tok, n_out] 16-bit
    const void* bias;                // [n_out] 16-bit or null
    const float* alpha;              // [n_out] or null
    const void* residual;            // [m_tok, n_out] or null
    int out_bf16;
    const uint8_t* sf_w;             // NVFP4 scale atoms of the weights / activations
    const uint8_t* sf_x;
    int sf_k64;
    int* status;
    // reduce-scatter epilogue (rs_world > 1): token t → rs_out[t / rs_rows_per_rank], row rs_rank * rs_rows_per_rank + t % rs_rows_per_rank
    void* rs_out[8];
    int rs_world, rs_rank, rs_rows_per_rank;
    // all-gather prologue (ag_flags != null): rank o pushed tokens [o * ag_rows_per_rank, ...) and then set ag_flags[o] = *ag_epoch
    const int* ag_flags;
    const int* ag_epoch;
    int ag_world, ag_rows_per_rank;
};

// Where the four features starting at `feat` of token `tok` are stored: the local output, or the owner rank's partial buffer.
template <typename T>
__device__ __forceinline__ T* skinny_out_ptr(const SkinnyParams& p, int tok, int feat) {
    if (p.rs_world > 1) {
        const int d = tok / p.rs_rows_per_rank;
        return reinterpret_cast<T*>(p.rs_out[d]) + ((size_t)p.rs_rank * p.rs_rows_per_rank + (tok - d * p.rs_rows_per_rank)) * p.n_out + feat;
    }
    return reinterpret_cast<T*>(p.out) + (size_t)tok * p.n_out + feat;
}

__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// 16-byte load from the same shared-memory offset in CTA `rank` of the cluster.  Not volatile: the
// loads of one reduction step are independent and must be free to overlap; ordering against the
// producers is provided by the cluster barriers around the reduction.
__device__ __forceinline__ float4 ld_dsmem_f32x4(uint32_t local_smem_addr, uint32_t rank) {
    uint32_t remote;
    float4 v;
    asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
    asm("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote));
    return v;
}

template <int KIND, int BN>
struct SkinnyCfg {
    static constexpr int kBKBytes = 128;                                     // one swizzle atom per row
    static constexpr int kWTile = kBM * 128;
    static constexpr int kXTile = BN * 128;
    static constexpr int kSf = KIND == 1 ? 2 * 2048 : 0;
    static constexpr int kStage = kWTile + kXTile + kSf;
    static constexpr int kRed = BN * kBM * 4;                                // fp32 partial tile
    static constexpr int kBudget = 98304;
    static constexpr int kStagesRaw = kBudget / kStage;
    static constexpr int kStages = kStagesRaw > 8 ? 8 : (kStagesRaw < 2 ? 2 : kStagesRaw);
    static constexpr int kSmemData = kStages * kStage > kRed ? kStages * kStage : kRed;
    static constexpr int kAccCols = BN < 32 ? 32 : BN;
    static constexpr int kTmemNeed = kAccCols + (KIND == 1 ? 2 * 32 : 0);
    static constexpr int kTmemCols = kTmemNeed <= 32 ? 32 : kTmemNeed <= 64 ? 64 : kTmemNeed <= 128 ? 128 : 256;
};

// KIND 0: bf16/fp16 operands (K per stage = 64), KIND 1: NVFP4 (K per stage = 256).
template <int KIND, int BN, typename T>
__global__ void __launch_bounds__(kGemmThreads, 2)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x, SkinnyParams p) {
    using Cfg = SkinnyCfg<KIND, BN>;
    constexpr int STAGES = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::kSmemData);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tfull_bar = empty_bar + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull_bar + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* s_alpha = reinterpret_cast<float*>(tmem_slot + 4);      // per-feature scale / bias of this 128-row tile
    float* s_bias = s_alpha + kBM;
    float* red = reinterpret_cast<float*>(smem);          // aliases the stage ring once the main loop is done

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int a0 = blockIdx.x * kBM;
    const int rank = p.ranks > 1 ? (int)cluster_rank() : 0;
    const int kb0 = rank * p.kb_per_rank;
    const int kb1 = min(p.kb_total, kb0 + p.kb_per_rank);
    const int nkb = max(0, kb1 - kb0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(tfull_bar, 1);
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tensormap(&tma_w);
        prefetch_tensormap(&tma_x);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    pdl_launch_dependents();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // Weight tiles (and their scales) of the first ring pass do not depend on the previous
            // kernel: issue them before waiting for it.
            const int pre = min(nkb, STAGES);
            for (int j = 0; j < pre; ++j) {
                uint8_t* sw = smem + j * Cfg::kStage;
                mbar_expect_tx(&full_bar[j], Cfg::kStage);
                tma_load_2d(sw, &tma_w, &full_bar[j], (kb0 + j) * (KIND == 1 ? 128 : 64), a0);
                if constexpr (KIND == 1)
                    bulk_load(sw + Cfg::kWTile + Cfg::kXTile, p.sf_w + ((size_t)blockIdx.x * p.sf_k64 + (size_t)(kb0 + j) * 4) * 512,
                              2048, &full_bar[j]);
            }
            pdl_wait();
            bool x_ready = true;
            if (p.ag_flags) {
                // the rows of every owner rank below m_tok must have arrived (peers wrote them with plain stores; the
                // tiles are read by TMA / bulk copies, hence the proxy fence)
                const int e = *p.ag_epoch;
                const int o1 = min((p.m_tok - 1) / p.ag_rows_per_rank, p.ag_world - 1);
                for (int o = 0; o <= o1 && x_ready; ++o) {
                    const uint64_t t0 = global_timer_ns();
                    uint32_t it = 0;
                    while (ld_acquire_sys_s32(p.ag_flags + o) - e < 0) {
                        if ((++it & 63u) == 0 && (*abort_flag || global_timer_ns() - t0 > kWaitLimitNs)) {
                            *abort_flag = 1;
                            if (p.status) atomicCAS(p.status, kStatusOk, kStatusPeerTimeout);
                            x_ready = false;
                            break;
                        }
                    }
                }
                asm volatile("fence.proxy.async;" ::: "memory");
            }
            for (int j = 0; j < pre && x_ready; ++j) {
                uint8_t* sx = smem + j * Cfg::kStage + Cfg::kWTile;
                tma_load_2d(sx, &tma_x, &full_bar[j], (kb0 + j) * (KIND == 1 ? 128 : 64), 0);
                if constexpr (KIND == 1)
                    bulk_load(sx + Cfg::kXTile + 2048, p.sf_x + (size_t)(kb0 + j) * 4 * 512, 2048, &full_bar[j]);
            }
            int stage = pre % STAGES;
            uint32_t phase = pre >= STAGES ? 1 : 0;
            for (int j = pre; j < nkb && x_ready; ++j) {
                if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) break;
                uint8_t* sw = smem + stage * Cfg::kStage;
                mbar_expect_tx(&full_bar[stage], Cfg::kStage);
                tma_load_2d(sw, &tma_w, &full_bar[stage], (kb0 + j) * (KIND == 1 ? 128 : 64), a0);
                tma_load_2d(sw + Cfg::kWTile, &tma_x, &full_bar[stage], (kb0 + j) * (KIND == 1 ? 128 : 64), 0);
                if constexpr (KIND == 1) {
                    bulk_load(sw + Cfg::kWTile + Cfg::kXTile, p.sf_w + ((size_t)blockIdx.x * p.sf_k64 + (size_t)(kb0 + j) * 4) * 512,
                              2048, &full_bar[stage]);
                    bulk_load(sw + Cfg::kWTile + Cfg::kXTile + 2048, p.sf_x + (size_t)(kb0 + j) * 4 * 512, 2048, &full_bar[stage]);
                }
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && nkb > 0) {
            const uint32_t idesc = KIND == 1 ? idesc_nvfp4(kBM, BN) : idesc_f16(kBM, BN, p.out_bf16 != 0);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int j = 0; j < nkb; ++j) {
                if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kStatusMmaTimeout)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint8_t* sw = smem + stage * Cfg::kStage;
                const uint64_t dw = smem_desc_sw128(sw);
                const uint64_t dx = smem_desc_sw128(sw + Cfg::kWTile);
                if constexpr (KIND == 1) {
                    const uint32_t t_sfw = tmem_base + Cfg::kAccCols + (j & 1) * 32;
                    const uint32_t t_sfx = t_sfw + 16;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        tmem_cp_sf(t_sfw + i * 4, smem_desc_sf(sw + Cfg::kWTile + Cfg::kXTile + i * 512));
                        tmem_cp_sf(t_sfx + i * 4, smem_desc_sf(sw + Cfg::kWTile + Cfg::kXTile + 2048 + i * 512));
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        umma_nvfp4(tmem_base, dw + 2 * i, dx + 2 * i, idesc, t_sfw + i * 4, t_sfx + i * 4, (j > 0 || i > 0) ? 1u : 0u);
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) umma_f16(tmem_base, dw + 2 * i, dx + 2 * i, idesc, (j > 0 || i > 0) ? 1u : 0u);
                }
                umma_commit(&empty_bar[stage]);
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (ok) umma_commit(tfull_bar);
        }
    }

    // ---- epilogue ------------------------------------------------------------------------------
    const bool is_epi = warp >= 2;
    const int quad = warp & 3;
    const int lrow = quad * 32 + lane;
    const int feat = a0 + lrow;
    const bool feat_ok = is_epi && feat < p.n_out;
    float alpha = 1.f, bias = 0.f;
    if (feat_ok) {                                   // static per-feature constants: fetch while the MMAs run
        if (p.alpha) alpha = __ldg(&p.alpha[feat]);
        if (p.bias) bias = Cvt<T>::to_f(reinterpret_cast<const T*>(p.bias)[feat]);
    }
    if (is_epi) {
        s_alpha[lrow] = alpha;
        s_bias[lrow] = bias;
    }
    bool have_acc = false;
    if (is_epi && nkb > 0) {
        have_acc = mbar_wait(tfull_bar, 0, abort_flag, p.status, kStatusEpilogueTimeout);
        tc_fence_after_sync();
    }
    const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    T* outp = reinterpret_cast<T*>(p.out);
    const T* resp = reinterpret_cast<const T*>(p.residual);
    const bool scatter = p.rs_world > 1;          // host side guarantees n_out % 4 == 0 and no residual

    if (p.ranks == 1 && (p.m_tok > 8 || scatter) && (p.n_out & 3) == 0) {
        // Many token columns: a lane owns one feature, so direct stores would be 2-byte pieces 2 * n_out apart.  The
        // tile is transposed through shared memory instead (the stage ring is free once the MMAs have completed) and
        // leaves as 8-byte stores, 256 contiguous bytes per token and warp.
        __syncthreads();
        if (is_epi) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (c0 >= p.m_tok) break;
                uint32_t r[16];
                if (have_acc) {
                    tmem_ld_x16(t_addr + c0, r);
                    tmem_ld_wait();
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) red[(c0 + j) * kBM + lrow] = have_acc ? __uint_as_float(r[j]) : 0.f;
            }
            named_barrier_sync(1, 128);
            pdl_wait();
            const int etid = (warp - 2) * 32 + lane;
            const int items = min(BN, p.m_tok) * 32;
            for (int it = etid; it < items; it += 128) {
                const int c = it >> 5;
                const int fg = (it & 31) * 4;
                const int f0 = a0 + fg;
                if (f0 + 3 >= p.n_out) continue;
                const float4 acc4 = *reinterpret_cast<const float4*>(&red[c * kBM + fg]);
                float v[4] = {acc4.x, acc4.y, acc4.z, acc4.w};
                const size_t o = (size_t)c * p.n_out + f0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    v[i] = v[i] * s_alpha[fg + i] + s_bias[fg + i];
                    if (resp) v[i] += Cvt<T>::to_f(resp[o + i]);
                }
                uint2 u;
                u.x = Cvt<T>::pack2(v[0], v[1]);
                u.y = Cvt<T>::pack2(v[2], v[3]);
                *reinterpret_cast<uint2*>(skinny_out_ptr<T>(p, c, f0)) = u;
            }
            // peer stores are performed system-wide before this thread moves on, so the "GEMM finished" flag that
            // the next kernel publishes can never overtake them
            if (scatter) __threadfence_system();
        }
    } else if (p.ranks == 1) {
        if (is_epi) {
            pdl_wait();
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (c0 >= p.m_tok) break;
                uint32_t r[16];
                if (have_acc) {
                    tmem_ld_x16(t_addr + c0, r);
                    tmem_ld_wait();
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int tok = c0 + j;
                    if (feat_ok && tok < p.m_tok) {
                        float v = (have_acc ? __uint_as_float(r[j]) : 0.f) * alpha + bias;
                        const size_t o = (size_t)tok * p.n_out + feat;
                        if (resp) v += Cvt<T>::to_f(resp[o]);
                        outp[o] = Cvt<T>::from_f(v);
                    }
                }
            }
        }
    } else {
        // 1. park the partial tile in shared memory: red[col][lane]
        __syncthreads();            // every role is done with the stage ring (MMAs completed → tfull)
        if (is_epi) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (c0 >= p.m_tok) break;
                uint32_t r[16];
                if (have_acc) {
                    tmem_ld_x16(t_addr + c0, r);
                    tmem_ld_wait();
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) red[(c0 + j) * kBM + lrow] = have_acc ? __uint_as_float(r[j]) : 0.f;
            }
        }
        cluster_sync_all();
        // 2. reduce my slice of the token columns across the cluster: one work item is (token column,
        //    four consecutive features); its `ranks` 16-byte peer loads are issued together.
        if (is_epi) {
            pdl_wait();
            const int etid = (warp - 2) * 32 + lane;
            const int mcols = min(BN, p.m_tok);
            const int per = (mcols + p.ranks - 1) / p.ranks;
            const int c_lo = rank * per, c_hi = min(mcols, c_lo + per);
            const int items = max(0, c_hi - c_lo) * 32;
            const bool vec_out = (p.n_out & 3) == 0;
            for (int it = etid; it < items; it += 128) {
                const int c = c_lo + (it >> 5);
                const int fg = (it & 31) * 4;
                const uint32_t addr = smem_u32(&red[c * kBM + fg]);
                float4 part[8];
#pragma unroll
                for (int rk = 0; rk < 8; ++rk)
                    part[rk] = rk < p.ranks ? ld_dsmem_f32x4(addr, rk) : make_float4(0.f, 0.f, 0.f, 0.f);
                float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int rk = 0; rk < 8; ++rk) {
                    v[0] += part[rk].x;
                    v[1] += part[rk].y;
                    v[2] += part[rk].z;
                    v[3] += part[rk].w;
                }
                const int f0 = a0 + fg;
                const size_t o = (size_t)c * p.n_out + f0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (f0 + i < p.n_out) {
                        v[i] = v[i] * s_alpha[fg + i] + s_bias[fg + i];
                        if (resp) v[i] += Cvt<T>::to_f(resp[o + i]);
                    }
                }
                if (vec_out && f0 + 3 < p.n_out) {
                    uint2 u;
                    u.x = Cvt<T>::pack2(v[0], v[1]);
                    u.y = Cvt<T>::pack2(v[2], v[3]);
                    *reinterpret_cast<uint2*>(skinny_out_ptr<T>(p, c, f0)) = u;
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (f0 + i < p.n_out) outp[o + i] = Cvt<T>::from_f(v[i]);
                }
            }
            if (scatter) __threadfence_system();
        }
        cluster_sync_all();         // peers may still be reading this CTA's partial tile
    }

    if (*abort_flag) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

template <int KIND, int BN, typename T>
static int launch_skinny(const CUtensorMap& tw, const CUtensorMap& tx, const SkinnyParams& p, cudaStream_t stream) {
    using Cfg = SkinnyCfg<KIND, BN>;
    constexpr int smem = Cfg::kSmemData + 1024 + 256 + 2 * kBM * 4;
    static bool configured = false;
    auto kern = gemm_skinny_kernel<KIND, BN, T>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail("cudaFuncSetAttribute(gemm_skinny)", e);
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 0);
        (void)e;
        cudaGetLastError();
        configured = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((p.n_out + kBM - 1) / kBM, p.ranks, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    int na = 0;
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    if (pdl_enabled()) ++na;
    if (p.ranks > 1) {
        attrs[na].id = cudaLaunchAttributeClusterDimension;
        attrs[na].val.clusterDim.x = 1;
        attrs[na].val.clusterDim.y = p.ranks;
        attrs[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw, tx, p);
    if (e != cudaSuccess) return fail("cudaLaunchKernelEx(gemm_skinny)", e);
    return 0;
}

// Cluster size (K ranks).  A cluster lives inside one GPC, so what counts is how many clusters of a given size are
// resident at once: with two CTAs per SM and at least 16 usable SMs in each of the 8 GPCs that is 8 * (32 / r)
// (48 clusters of 6 or 8 do not fit and run as two waves, 48 clusters of 4 do).  Among the sizes that divide the
// work the estimate below — waves x (K steps per rank + fixed launch-to-first-byte cost) + reduction cost per rank —
// picks the cheapest; its constants come from timing the Qwen3-8B decode projections with HBM-resident weights.
static int choose_ranks(int tiles, int kb_total, int force) {
    if (force > 0) return force > 8 ? 8 : (force > kb_total ? kb_total : force);
    static const int cand[6] = {1, 2, 3, 4, 6, 8};
    int best_r = 1;
    float best = 1e30f;
    for (int i = 0; i < 6; ++i) {
        const int r = cand[i];
        if (r > kb_total) break;
        const int capacity = 8 * (32 / r);
        const int waves = (tiles + capacity - 1) / capacity;
        const int steps = (kb_total + r - 1) / r;
        const float est = waves * (steps * 0.35f + 4.0f) + r * 0.15f;
        if (est < best - 1e-3f) {
            best = est;
            best_r = r;
        }
    }
    return best_r;
}

template <int KIND>
static int dispatch_skinny(const CUtensorMap& tw, const CUtensorMap& tx, const SkinnyParams& p, int bn, cudaStream_t stream) {
#define TELB_SK(BN_)                                                                          \
    return p.out_bf16 ? launch_skinny<KIND, BN_, __nv_bfloat16>(tw, tx, p, stream)            \
                      : launch_skinny<KIND, BN_, __half>(tw, tx, p, stream)
    switch (bn) {
        case 16: TELB_SK(16);
        case 32: TELB_SK(32);
        case 64: TELB_SK(64);
        default: TELB_SK(128);
    }
#undef TELB_SK
}

}  // namespace telb

using namespace telb;

extern "C" int telb_nvfp4_k64_pad(int k);

// kind 0: x, w are 16-bit [M,K], [N,K].  kind 1: packed E2M1 [M,K/2], [N,K/2] with atom-layout scales.
// `fusion` (may be null) adds the reduce-scatter epilogue and / or the all-gather prologue described at the top.
extern "C" int telb_gemm_skinny_fused(int kind, const void* x, const void* x_sf, const void* w, const void* w_sf, void* out, int M,
                                      int N, int K, const float* alpha, const void* bias, const void* residual, int is_bf16,
                                      int* status, int force_ranks, const TelbGemmFusion* fusion, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (M > 128) return fail("telb_gemm_skinny: M must be <= 128");
    if (fusion && fusion->rs_world > 1) {
        if (residual) return fail("telb_gemm_skinny: reduce-scatter epilogue takes no residual");
        if (N % 4) return fail("telb_gemm_skinny: reduce-scatter epilogue needs N % 4 == 0");
        if (fusion->rs_world > 8 || fusion->rs_rows_per_rank <= 0 || (long long)fusion->rs_rows_per_rank * fusion->rs_world < M)
            return fail("telb_gemm_skinny: reduce-scatter rows_per_rank * world must cover M (world <= 8)");
    }
    const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
    SkinnyParams p{};
    p.n_out = N;
    p.m_tok = M;
    p.k = K;
    p.out = out;
    p.bias = bias;
    p.alpha = alpha;
    p.residual = residual;
    p.out_bf16 = is_bf16;
    p.status = status;
    if (fusion) {
        for (int i = 0; i < 8; ++i) p.rs_out[i] = fusion->rs_out[i];
        p.rs_world = fusion->rs_world;
        p.rs_rank = fusion->rs_rank;
        p.rs_rows_per_rank = fusion->rs_rows_per_rank;
        p.ag_flags = fusion->ag_flags;
        p.ag_epoch = fusion->ag_epoch;
        p.ag_world = fusion->ag_world;
        p.ag_rows_per_rank = fusion->ag_rows_per_rank;
        if (p.ag_flags && (p.ag_world < 1 || p.ag_rows_per_rank <= 0)) return fail("telb_gemm_skinny: bad all-gather description");
    }
    CUtensorMap tw, tx;
    if (kind == 1) {
        if (K % 32) return fail("telb_gemm_skinny: NVFP4 needs K % 32 == 0");
        p.kb_total = (K + 255) / 256;
        p.sf_w = (const uint8_t*)w_sf;
        p.sf_x = (const uint8_t*)x_sf;
        p.sf_k64 = telb_nvfp4_k64_pad(K);
        const uint64_t kbytes = (uint64_t)K / 2;
        if (make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w, N, kbytes, kbytes, kBM, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
        if (make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x, M, kbytes, kbytes, bn, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    } else {
        if (K % 8) return fail("telb_gemm_skinny: K must be a multiple of 8");
        p.kb_total = (K + 63) / 64;
        const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        if (make_tmap_2d(&tw, dt, 2, w, N, K, (uint64_t)K * 2, kBM, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
        if (make_tmap_2d(&tx, dt, 2, x, M, K, (uint64_t)K * 2, bn, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    }
    const int tiles = (N + kBM - 1) / kBM;
    int ranks = choose_ranks(tiles, p.kb_total, force_ranks);
    p.kb_per_rank = (p.kb_total + ranks - 1) / ranks;
    p.ranks = (p.kb_total + p.kb_per_rank - 1) / p.kb_per_rank;
    return kind == 1 ? dispatch_skinny<1>(tw, tx, p, bn, stream) : dispatch_skinny<0>(tw, tx, p, bn, stream);
}

extern "C" int telb_gemm_skinny(int kind, const void* x, const void* x_sf, const void* w, const void* w_sf, void* out, int M,
                                int N, int K, const float* alpha, const void* bias, const void* residual, int is_bf16,
                                int* status, int force_ranks, cudaStream_t stream) {
    return telb_gemm_skinny_fused(kind, x, x_sf, w, w_sf, out, M, N, K, alpha, bias, residual, is_bf16, status, force_ranks, nullptr, stream);
}
