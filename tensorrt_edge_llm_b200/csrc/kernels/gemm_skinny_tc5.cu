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
// INT4 group-wise weights (KIND 2, W4A16): the packed 4-bit tile of a K step (4 KB for 128 output rows x 64 inputs) arrives
// by TMA next to the activation tile; the four warps that later run the epilogue expand it — (q − 8) · scale per
// group — into the 16-bit, 128-byte-swizzled operand tile the MMA reads, so HBM and L2 only ever see 4-bit weights.
//
// Reference counterparts: TensorRT decode tactics; int4 group-wise GEMM / GEMV of
// cpp/kernels/int4GroupwiseGemmKernels/int4WoqGemmCuda.cu:98-124 and int4WoQGemvCuda.cu:225-253 (mma.sync / CUDA cores);
// kernelSrcs/nvfp4A16BlackwellGemv (SM110-only
// CUDA-core GEMV) and `gemm_blackwell_nvfp4_ws_*_tn64` at TP=2.
#include <type_traits>

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
    // INT4 group-wise weights (KIND 2): per-(row, group) scales, 16-bit, [n_out, k / group]
    const void* w_scale;
    int group, groups_per_row;
    // SwiGLU + NVFP4 output (weights whose gate / up rows alternate in blocks of 64, m_tok <= 64): instead of the 16-bit
    // [m_tok, n_out] result the epilogue stores quantised silu(gate) * up [m_tok, n_out / 2] — packed codes into sw_xq
    // (row pitch sw_ld bytes) and block scales into the atom-layout buffer sw_sf.
    uint8_t* sw_xq;
    uint8_t* sw_sf;
    const float* sw_gs;
    int sw_ld, sw_k64_pad;
};

// 16 SwiGLU outputs of one token from a 128-feature tile row `v` (64 gate features followed by their 64 up features, fp32
// sums already scaled): the same roundings as the unfused chain — 16-bit GEMM output, 16-bit activation — then quantise.
template <typename T>
__device__ __forceinline__ void skinny_swiglu_block(const SkinnyParams& p, const float* v, int tok, int a0, int b) {
    float y[16];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float g = Cvt<T>::to_f(Cvt<T>::from_f(v[16 * b + i]));
        const float u = Cvt<T>::to_f(Cvt<T>::from_f(v[64 + 16 * b + i]));
        y[i] = Cvt<T>::to_f(Cvt<T>::from_f(g / (1.f + __expf(-g)) * u));
        amax = fmaxf(amax, fabsf(y[i]));
    }
    const float gs = *p.sw_gs;
    uint8_t s8;
    const uint2 packed = nvfp4_quantize_block16(y, amax, gs, 1.f / gs, s8);
    const int blk = (a0 / 2 + 16 * b) >> 4;                         // 16-element block index along the intermediate dimension
    *reinterpret_cast<uint2*>(p.sw_xq + (size_t)tok * p.sw_ld + blk * 8) = packed;
    p.sw_sf[sf_atom_offset((long long)tok, blk, p.sw_k64_pad)] = s8;
}

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
    static constexpr int kSf = KIND == 1 ? 2 * 2048 : (KIND == 2 ? 4096 : 0);      // NVFP4 scale atoms, or the packed INT4 tile
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

// Eight 4-bit codes of one output row (the low or the high nibbles of eight packed bytes) → eight 16-bit values (q − 8) · scale.
// No integer-to-float conversion: a code OR-ed into the mantissa of a 16-bit constant is the number (C + q) exactly
// (C = 128 for bf16, 1024 for fp16); subtracting (C + 8) is exact too, and one multiply by the scale rounds once.
// A 32-bit word holds the codes of inputs k, k+1, k+2, k+3 in its four bytes: the masked word pairs (k, k+2) and
// (k+1, k+3), and two byte permutes restore the input order.
template <typename T>
__device__ __forceinline__ uint4 int4_expand8(uint32_t w0, uint32_t w1, int shift, float scale) {
    constexpr bool kBf = std::is_same<T, __nv_bfloat16>::value;
    constexpr uint32_t kMagic = kBf ? 0x43004300u : 0x64006400u;          // 128.0 | 128.0   or   1024.0 | 1024.0
    constexpr uint32_t kOff = kBf ? 0x43084308u : 0x64086408u;            // 136.0 | 136.0   or   1032.0 | 1032.0
    const uint32_t a0 = ((w0 >> shift) & 0x000F000Fu) | kMagic, a1 = ((w0 >> (shift + 8)) & 0x000F000Fu) | kMagic;
    const uint32_t b0 = ((w1 >> shift) & 0x000F000Fu) | kMagic, b1 = ((w1 >> (shift + 8)) & 0x000F000Fu) | kMagic;
    uint32_t v[4] = {__byte_perm(a0, a1, 0x5410), __byte_perm(a0, a1, 0x7632), __byte_perm(b0, b1, 0x5410), __byte_perm(b0, b1, 0x7632)};
    uint4 u;
    uint32_t* o = reinterpret_cast<uint32_t*>(&u);
    if constexpr (kBf) {
        const __nv_bfloat162 s2 = __float2bfloat162_rn(scale);
        const __nv_bfloat162 off = *reinterpret_cast<const __nv_bfloat162*>(&kOff);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 r = __hmul2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&v[i]), off), s2);
            o[i] = *reinterpret_cast<const uint32_t*>(&r);
        }
    } else {
        const __half2 s2 = __float2half2_rn(scale);
        const __half2 off = *reinterpret_cast<const __half2*>(&kOff);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 r = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&v[i]), off), s2);
            o[i] = *reinterpret_cast<const uint32_t*>(&r);
        }
    }
    return u;
}

// KIND 0: bf16/fp16 operands (K per stage = 64), KIND 1: NVFP4 (K per stage = 256), KIND 2: INT4 group-wise weights
// expanded to 16 bits in shared memory (K per stage = 64).
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
    uint64_t* raw_bar = tfull_bar + 1;                 // KIND 2: the packed tile and the activations of a stage have landed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(raw_bar + STAGES);
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
            mbar_init(&full_bar[s], KIND == 2 ? 128 : 1);      // KIND 2: the 128 expanding threads fill the operand tile
            mbar_init(&empty_bar[s], 1);
            mbar_init(&raw_bar[s], 1);
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
                if constexpr (KIND == 2) {
                    // packed 4-bit tile: 64 byte rows (two output rows each) x 64 input columns, into the stage's staging area
                    mbar_expect_tx(&raw_bar[j], 4096 + Cfg::kXTile);
                    tma_load_2d(sw + Cfg::kWTile + Cfg::kXTile, &tma_w, &raw_bar[j], (kb0 + j) * 64, a0 / 2);
                } else {
                    mbar_expect_tx(&full_bar[j], Cfg::kStage);
                    tma_load_2d(sw, &tma_w, &full_bar[j], (kb0 + j) * (KIND == 1 ? 128 : 64), a0);
                }
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
                tma_load_2d(sx, &tma_x, KIND == 2 ? &raw_bar[j] : &full_bar[j], (kb0 + j) * (KIND == 1 ? 128 : 64), 0);
                if constexpr (KIND == 1)
                    bulk_load(sx + Cfg::kXTile + 2048, p.sf_x + (size_t)(kb0 + j) * 4 * 512, 2048, &full_bar[j]);
            }
            int stage = pre % STAGES;
            uint32_t phase = pre >= STAGES ? 1 : 0;
            for (int j = pre; j < nkb && x_ready; ++j) {
                if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) break;
                uint8_t* sw = smem + stage * Cfg::kStage;
                if constexpr (KIND == 2) {
                    mbar_expect_tx(&raw_bar[stage], 4096 + Cfg::kXTile);
                    tma_load_2d(sw + Cfg::kWTile + Cfg::kXTile, &tma_w, &raw_bar[stage], (kb0 + j) * 64, a0 / 2);
                    tma_load_2d(sw + Cfg::kWTile, &tma_x, &raw_bar[stage], (kb0 + j) * 64, 0);
                } else {
                    mbar_expect_tx(&full_bar[stage], Cfg::kStage);
                    tma_load_2d(sw, &tma_w, &full_bar[stage], (kb0 + j) * (KIND == 1 ? 128 : 64), a0);
                    tma_load_2d(sw + Cfg::kWTile, &tma_x, &full_bar[stage], (kb0 + j) * (KIND == 1 ? 128 : 64), 0);
                }
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
            const uint32_t idesc = KIND == 1 ? idesc_nvfp4(kBM, BN) : idesc_f16(kBM, BN, p.out_bf16 != 0);     // KIND 2 multiplies 16-bit tiles
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

    if constexpr (KIND == 2) {
        if (warp >= 2) {
            // ---- expand the packed 4-bit tiles: thread t serves byte row t / 2 (output rows 2 (t/2), 2 (t/2) + 1) and the
            //      input-column half t % 2 (32 columns = four 16-byte chunks per output row) ----
            const int t = (warp - 2) * 32 + lane;
            const int pr = t >> 1, kh = t & 1;
            const int row0 = 2 * pr, grow = a0 + row0;
            const T* sc = reinterpret_cast<const T*>(p.w_scale);
            int stage = 0, cur_group = -1;
            uint32_t phase = 0;
            float s0 = 0.f, s1 = 0.f;
            for (int j = 0; j < nkb; ++j) {
                const int grp = ((kb0 + j) * 64) / p.group;
                if (grp != cur_group) {                        // a group spans one or more K steps: fetch its two scales once
                    cur_group = grp;
                    s0 = grow < p.n_out ? Cvt<T>::to_f(sc[(size_t)grow * p.groups_per_row + grp]) : 0.f;
                    s1 = grow + 1 < p.n_out ? Cvt<T>::to_f(sc[(size_t)(grow + 1) * p.groups_per_row + grp]) : 0.f;
                }
                if (!mbar_wait(&raw_bar[stage], phase, abort_flag, p.status, kStatusEpilogueTimeout)) break;
                uint8_t* sw = smem + stage * Cfg::kStage;
                const uint4* src = reinterpret_cast<const uint4*>(sw + Cfg::kWTile + Cfg::kXTile + pr * 64 + kh * 32);
                const uint4 pa = src[0], pb = src[1];
                const uint32_t w[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int chunk = kh * 4 + c;
                    const int r0 = row0, r1 = row0 + 1;
                    *reinterpret_cast<uint4*>(sw + (r0 >> 3) * 1024 + (r0 & 7) * 128 + ((chunk ^ (r0 & 7)) << 4)) =
                        int4_expand8<T>(w[2 * c], w[2 * c + 1], 0, s0);
                    *reinterpret_cast<uint4*>(sw + (r1 >> 3) * 1024 + (r1 & 7) * 128 + ((chunk ^ (r1 & 7)) << 4)) =
                        int4_expand8<T>(w[2 * c], w[2 * c + 1], 4, s1);
                }
                fence_proxy_async_smem();
                mbar_arrive(&full_bar[stage]);
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            }
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

    if (p.ranks == 1 && (p.m_tok > 8 || scatter || p.sw_xq != nullptr) && (p.n_out & 3) == 0) {
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
            if (p.sw_xq != nullptr) {
                // SwiGLU + quantise: one item = (token, block of 16 outputs); the tile row is scaled in place first
                const int mt = min(BN, p.m_tok);
                for (int it = etid; it < mt * kBM; it += 128) red[it] = red[it] * s_alpha[it & (kBM - 1)] + s_bias[it & (kBM - 1)];
                named_barrier_sync(1, 128);
                for (int it = etid; it < mt * 4; it += 128) skinny_swiglu_block<T>(p, red + (it >> 2) * kBM, it >> 2, a0, it & 3);
            }
            const int items = p.sw_xq != nullptr ? 0 : min(BN, p.m_tok) * 32;
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
            float* fin = red + BN * kBM;            // SwiGLU mode: this CTA's reduced token columns [per][128], local only
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
                if (p.sw_xq != nullptr) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) fin[(c - c_lo) * kBM + fg + i] = v[i] * s_alpha[fg + i] + s_bias[fg + i];
                    continue;
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
            if (p.sw_xq != nullptr) {
                named_barrier_sync(1, 128);
                for (int it = etid; it < max(0, c_hi - c_lo) * 4; it += 128)
                    skinny_swiglu_block<T>(p, fin + (it >> 2) * kBM, c_lo + (it >> 2), a0, it & 3);
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

// Whole-matrix expansion of INT4 group-wise weights to 16 bits (prefill-size GEMMs run on the dense tensor-core kernel
// over a temporary expanded copy; decode-size GEMMs expand tile by tile inside gemm_skinny_kernel and never need it).
template <typename T>
__global__ void int4_expand_kernel(const uint8_t* __restrict__ wq, const T* __restrict__ scales, T* __restrict__ out, int n, int k,
                                   int group) {
    pdl_prologue();
    const long long chunks = (long long)(n / 2) * (k / 8);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < chunks; i += (long long)gridDim.x * blockDim.x) {
        const int pr = (int)(i / (k / 8)), c = (int)(i - (long long)pr * (k / 8));
        const uint2 w = *reinterpret_cast<const uint2*>(wq + (size_t)pr * k + c * 8);
        const int grp = c * 8 / group;
        const float s0 = Cvt<T>::to_f(scales[(size_t)(2 * pr) * (k / group) + grp]);
        const float s1 = Cvt<T>::to_f(scales[(size_t)(2 * pr + 1) * (k / group) + grp]);
        *reinterpret_cast<uint4*>(out + (size_t)(2 * pr) * k + c * 8) = int4_expand8<T>(w.x, w.y, 0, s0);
        *reinterpret_cast<uint4*>(out + (size_t)(2 * pr + 1) * k + c * 8) = int4_expand8<T>(w.x, w.y, 4, s1);
    }
}

template <int KIND, int BN, typename T>
static int launch_skinny(const CUtensorMap& tw, const CUtensorMap& tx, const SkinnyParams& p, cudaStream_t stream) {
    using Cfg = SkinnyCfg<KIND, BN>;
    constexpr int smem = Cfg::kSmemData + 1024 + 384 + 2 * kBM * 4;
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
struct SkinnySwiglu {
    uint8_t* xq;
    uint8_t* sf;
    const float* gs;
};

static int gemm_skinny_impl(int kind, const void* x, const void* x_sf, const void* w, const void* w_sf, void* out, int M,
                            int N, int K, const float* alpha, const void* bias, const void* residual, int is_bf16,
                            int* status, int force_ranks, const TelbGemmFusion* fusion, int group, cudaStream_t stream,
                            const SkinnySwiglu* sw = nullptr) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (sw && (M > 64 || N % 128 || residual)) return fail("telb_gemm_skinny: the SwiGLU epilogue needs M <= 64, N % 128 == 0 and no residual");
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
    if (sw) {
        p.sw_xq = sw->xq;
        p.sw_sf = sw->sf;
        p.sw_gs = sw->gs;
        p.sw_ld = N / 4;                              // (N / 2 outputs) / 2 bytes per row
        p.sw_k64_pad = telb_nvfp4_k64_pad(N / 2);
    }
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
    if (kind == 2) {
        // w: packed INT4 [N / 2, K] bytes (row r: output rows 2r low nibble, 2r + 1 high nibble); w_sf: 16-bit scales [N, K / group]
        if (N % 2 || K % 64) return fail("telb_gemm_skinny: INT4 weights need an even N and K % 64 == 0");
        if (group < 64 || group % 64 || K % group) return fail("telb_gemm_skinny: INT4 group size must be a multiple of 64 that divides K");
        p.kb_total = K / 64;
        p.w_scale = w_sf;
        p.group = group;
        p.groups_per_row = K / group;
        const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        if (make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w, N / 2, K, K, 64, 64, CU_TENSOR_MAP_SWIZZLE_NONE)) return -1;
        if (make_tmap_2d(&tx, dt, 2, x, M, K, (uint64_t)K * 2, bn, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    } else if (kind == 1) {
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
    if (kind == 2) return dispatch_skinny<2>(tw, tx, p, bn, stream);
    return kind == 1 ? dispatch_skinny<1>(tw, tx, p, bn, stream) : dispatch_skinny<0>(tw, tx, p, bn, stream);
}

extern "C" int telb_gemm_skinny_fused(int kind, const void* x, const void* x_sf, const void* w, const void* w_sf, void* out, int M,
                                      int N, int K, const float* alpha, const void* bias, const void* residual, int is_bf16,
                                      int* status, int force_ranks, const TelbGemmFusion* fusion, cudaStream_t stream) {
    if (kind != 0 && kind != 1) return fail("telb_gemm_skinny_fused: kind must be 0 (16-bit) or 1 (NVFP4)");
    return gemm_skinny_impl(kind, x, x_sf, w, w_sf, out, M, N, K, alpha, bias, residual, is_bf16, status, force_ranks, fusion, 0, stream);
}

// Decode-size gate/up projection with SwiGLU + NVFP4 quantisation in the epilogue (M <= 64): w holds 2 * inter rows in which
// blocks of 64 gate rows alternate with the 64 matching up rows; the result is quantised silu(gate) * up [M, inter] as packed
// codes out_xq [M, inter / 2] and atom-layout scales out_sf (pre-zeroed by the caller when inter % 256 leaves padding).
extern "C" int telb_gemm_skinny_swiglu(int kind, const void* x, const void* x_sf, const void* w, const void* w_sf, const float* alpha,
                                       void* out_xq, void* out_sf, const float* out_global_scale, int M, int N, int K, int is_bf16,
                                       int* status, const TelbGemmFusion* fusion, cudaStream_t stream) {
    if (kind != 0 && kind != 1) return fail("telb_gemm_skinny_swiglu: kind must be 0 (16-bit) or 1 (NVFP4)");
    if (fusion && fusion->rs_world > 1) return fail("telb_gemm_skinny_swiglu: no reduce-scatter on a column-parallel projection");
    SkinnySwiglu sw{static_cast<uint8_t*>(out_xq), static_cast<uint8_t*>(out_sf), out_global_scale};
    return gemm_skinny_impl(kind, x, x_sf, w, w_sf, nullptr, M, N, K, alpha, nullptr, nullptr, is_bf16, status, 0, fusion, 0, stream, &sw);
}

// W4A16 decode-size GEMM: out[M, N] = x[M, K] · dequant(wq, scales)[N, K]ᵀ (+ bias, + residual), M <= 128.  wq is the
// ModelOpt-prepacked INT4 layout [N / 2, K] (byte row r holds output rows 2r in the low and 2r + 1 in the high nibbles,
// codes offset by 8), scales [N, K / group] in the activation dtype.  The 4-bit codes are expanded inside the kernel.
extern "C" int telb_gemm_skinny_int4(const void* x, const void* wq, const void* scales, void* out, int M, int N, int K, int group,
                                     const void* bias, const void* residual, int is_bf16, int* status, int force_ranks,
                                     cudaStream_t stream) {
    return gemm_skinny_impl(2, x, nullptr, wq, scales, out, M, N, K, nullptr, bias, residual, is_bf16, status, force_ranks, nullptr, group, stream);
}

// wq [N / 2, K] packed INT4 + scales [N, K / group] → out [N, K] 16-bit, (q − 8) · scale.
extern "C" int telb_int4_awq_expand(const void* wq, const void* scales, void* out, int N, int K, int group, int is_bf16,
                                    cudaStream_t stream) {
    if (N <= 0 || K <= 0) return 0;
    if (N % 2 || K % 8 || group <= 0 || group % 8 || K % group) return fail("telb_int4_awq_expand: even N, K % 8 == 0 and a group that divides K are required");
    const long long chunks = (long long)(N / 2) * (K / 8);
    long long blocks = (chunks + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (is_bf16)
        TELB_LAUNCH("int4_expand_kernel", (int4_expand_kernel<__nv_bfloat16>), dim3((int)blocks), dim3(256), 0, stream, (const uint8_t*)wq,
                    (const __nv_bfloat16*)scales, (__nv_bfloat16*)out, N, K, group);
    else
        TELB_LAUNCH("int4_expand_kernel", (int4_expand_kernel<__half>), dim3((int)blocks), dim3(256), 0, stream, (const uint8_t*)wq,
                    (const __half*)scales, (__half*)out, N, K, group);
    return 0;
}

extern "C" int telb_gemm_skinny(int kind, const void* x, const void* x_sf, const void* w, const void* w_sf, void* out, int M,
                                int N, int K, const float* alpha, const void* bias, const void* residual, int is_bf16,
                                int* status, int force_ranks, cudaStream_t stream) {
    return telb_gemm_skinny_fused(kind, x, x_sf, w, w_sf, out, M, N, K, alpha, bias, residual, is_bf16, status, force_ranks, nullptr, stream);
}
