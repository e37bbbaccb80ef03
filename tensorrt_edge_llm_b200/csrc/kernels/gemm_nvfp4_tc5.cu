// NVFP4 block-scaled GEMM on 5th-generation tensor cores:
//     out[M,N] = (xq ⊙ sfx)[M,K] · (wq ⊙ sfw)[N,K]ᵀ · alpha[N]  (+ bias, + residual)
// Operands are E2M1 values packed two per byte (low nibble = even K index) with one UE4M3 scale per
// 16 K-elements; `tcgen05.mma.kind::mxf4nvf4.block_scale.block16` applies the scales inside the
// tensor core and accumulates fp32 in TMEM.  alpha folds the two fp32 global scales
// (activation `input_scale` x weight `weight_scale_2`) per output feature.
//
// Scale factors arrive in the 512-byte atom layout the tensor core consumes (128 rows x 4 scales,
// byte = (r%32)*16 + (r/32)*4 + k): global memory holds [row tile of 128][K/64][512 B], so one
// pipeline stage (K = 256) of scales for a 128-row tile is a single contiguous 2 KiB bulk copy;
// `tcgen05.cp` then moves each atom from shared memory into TMEM next to the accumulators.
//
// Structure, roles, split-K and bounded waits are those of the 16-bit kernel (gemm_tc5.cu): large
// M keeps activations on the MMA-M side with a 128-wide weight tile, small M swaps the operands so
// the 128-row side streams weights.
//
// Reference counterparts: CuTe-DSL `gemm_blackwell_nvfp4_ws.py` (kernelSrcs/gemm_cutedsl/) and the
// scale repack of cpp/kernels/multiDeviceKernels/scaleConvert.cu; the activation quantiser below
// corresponds to cpp/kernels/moe/fp4SupportKernels/fp4Quantize.cu and the math of
// tensorrt_edgellm/models/ops.py:826-909.
#include "gemm_common.cuh"
#include "nvfp4_common.cuh"

namespace telb {

constexpr int kFp4BK = 256;                         // K elements per stage = 128 packed bytes
constexpr int kFp4ATileBytes = kBM * 128;           // 16 KiB
constexpr int kSfStageBytes = 2048;                 // 128 rows x 16 scales

template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                  const uint8_t* __restrict__ sf_a, const uint8_t* __restrict__ sf_b, int sf_k64_a, int sf_k64_b,
                  GemmParams p) {
    constexpr int kBGroups = BN > 128 ? BN / 128 : 1;            // 128-row scale groups of the B tile
    constexpr int kBTileBytes = BN * 128;
    constexpr int kSfBBytes = kBGroups * kSfStageBytes;
    constexpr int kStageBytes = kFp4ATileBytes + kBTileBytes + kSfStageBytes + kSfBBytes;
    constexpr int kAccStride = BN < 32 ? 32 : BN;
    constexpr int kSfACols = 16;                                  // 4 MMAs x 4 columns
    constexpr int kSfBCols = 16 * kBGroups;
    constexpr int kSfTmem0 = 2 * kAccStride;                      // scale columns start after the accumulators
    constexpr int kTmemNeed = 2 * kAccStride + 2 * (kSfACols + kSfBCols);
    constexpr int kTmemCols = kTmemNeed <= 64 ? 64 : kTmemNeed <= 128 ? 128 : kTmemNeed <= 256 ? 256 : 512;
    static_assert(kTmemNeed <= 512, "tile does not fit in TMEM");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * kStageBytes);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tfull_bar = empty_bar + STAGES;
    uint64_t* tempty_bar = tfull_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* last_flag = tmem_slot + 2;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int total_tiles = p.tiles_a * p.tiles_b * p.splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tfull_bar[s], 1);
            mbar_init(&tempty_bar[s], 128);
        }
        *abort_flag = 0;
        *last_flag = 0;
        mbar_fence_init();
        prefetch_tensormap(&tma_a);
        prefetch_tensormap(&tma_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    pdl_prologue();          // everything above is independent of earlier kernels
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- producer: operand tiles by TMA, scale atoms by bulk copy ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const int ag_e = p.ag_flags ? *p.ag_epoch : 0;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const TileCoord tc = decode_tile(p, t);
                if (tc.skip) continue;
                const int ta = tc.a0 / kBM;
                const int b0 = (tc.brow >= 0 ? tc.brow : 0) + tc.b0 * BN;      // row of the B tensor
                if (p.ag_flags && !ag_wait_rows(p, tc.a0, ag_e, abort_flag)) break;
                for (int kb = tc.kb0; kb < tc.kb1; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + stage * kStageBytes;
                    uint8_t* sb = sa + kFp4ATileBytes;
                    uint8_t* ssa = sb + kBTileBytes;
                    uint8_t* ssb = ssa + kSfStageBytes;
                    mbar_expect_tx(&full_bar[stage], kStageBytes);
                    tma_load_2d(sa, &tma_a, &full_bar[stage], kb * 128, tc.a0);
                    tma_load_2d(sb, &tma_b, &full_bar[stage], kb * 128, b0);
                    bulk_load(ssa, sf_a + ((size_t)ta * sf_k64_a + (size_t)kb * 4) * 512, kSfStageBytes, &full_bar[stage]);
#pragma unroll
                    for (int g = 0; g < kBGroups; ++g)
                        bulk_load(ssb + g * kSfStageBytes, sf_b + ((size_t)(b0 / 128 + g) * sf_k64_b + (size_t)kb * 4) * 512,
                                  kSfStageBytes, &full_bar[stage]);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- UMMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = idesc_nvfp4(kBM, BN);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            uint32_t sf_par = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const TileCoord tc = decode_tile(p, t);
                if (tc.skip) continue;
                if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, kStatusMmaTimeout)) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * kAccStride;
                for (int kb = tc.kb0; kb < tc.kb1; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kStatusMmaTimeout)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint8_t* sa = smem + stage * kStageBytes;
                    const uint8_t* sb = sa + kFp4ATileBytes;
                    const uint8_t* ssa = sb + kBTileBytes;
                    const uint8_t* ssb = ssa + kSfStageBytes;
                    const uint32_t t_sfa = tmem_base + kSfTmem0 + sf_par * (kSfACols + kSfBCols);
                    const uint32_t t_sfb = t_sfa + kSfACols;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        tmem_cp_sf(t_sfa + i * 4, smem_desc_sf(ssa + i * 512));
#pragma unroll
                        for (int g = 0; g < kBGroups; ++g)
                            tmem_cp_sf(t_sfb + (i * kBGroups + g) * 4, smem_desc_sf(ssb + g * kSfStageBytes + i * 512));
                    }
                    const uint64_t da = smem_desc_sw128(sa);
                    const uint64_t db = smem_desc_sw128(sb);
#pragma unroll
                    for (int i = 0; i < 4; ++i)     // 64 E2M1 elements = 32 bytes = 2 descriptor units
                        umma_nvfp4(d_tmem, da + 2 * i, db + 2 * i, idesc, t_sfa + i * 4, t_sfb + i * 4 * kBGroups,
                                   (kb > tc.kb0 || i > 0) ? 1u : 0u);
                    umma_commit(&empty_bar[stage]);
                    sf_par ^= 1;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit(&tfull_bar[acc]);
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
        }
    } else {
        gemm_epilogue_role<BN>(p, tmem_base, tfull_bar, tempty_bar, abort_flag, last_flag, total_tiles, kAccStride,
                               smem + STAGES * kStageBytes + 256,
                               reinterpret_cast<float*>(smem + STAGES * kStageBytes + 256 + kRsStageBytes));
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

template <int BN, int STAGES>
static int launch_nvfp4(const CUtensorMap& ta, const CUtensorMap& tb, const uint8_t* sfa, const uint8_t* sfb, int k64a,
                        int k64b, const GemmParams& p, cudaStream_t stream) {
    constexpr int kBGroups = BN > 128 ? BN / 128 : 1;
    constexpr int kStageBytes = kFp4ATileBytes + BN * 128 + kSfStageBytes + kBGroups * kSfStageBytes;
    constexpr int smem = STAGES * kStageBytes + 1024 + 256 + kRsStageBytes + kAlphaStageBytes;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_nvfp4_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail("cudaFuncSetAttribute(gemm_nvfp4)", e);
        configured = true;
    }
    const int total = p.tiles_a * p.tiles_b * p.splits;
    const int grid = total < sm_count() ? total : sm_count();
    TELB_LAUNCH("gemm_nvfp4_kernel", (gemm_nvfp4_kernel<BN, STAGES>), dim3(grid), dim3(kGemmThreads), smem, stream, ta, tb, sfa, sfb, k64a, k64b, p);
    TELB_CHECK_LAUNCH("gemm_nvfp4_kernel");
    return 0;
}

// ---- activation quantiser ---------------------------------------------------------------------
// x [M,K] 16-bit → packed E2M1 [M,K/2] + UE4M3 scales in the atom layout ([ceil(M/128)][k64_pad][512]).
// One thread per 16-element block.  scale = e4m3(amax / 6 / global), value = rn_e2m1(x / (scale*global)).
template <typename T>
__global__ void nvfp4_quantize_kernel(const T* __restrict__ x, uint8_t* __restrict__ xq, uint8_t* __restrict__ sf,
                                      const float* __restrict__ global_scale, long long rows, int k, int k64_pad) {
    pdl_prologue();
    const int blocks_per_row = k / 16;
    const long long total = rows * blocks_per_row;
    const float gs = *global_scale;
    const float inv_gs = 1.f / gs;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long r = idx / blocks_per_row;
        const int kb = (int)(idx - r * blocks_per_row);
        const uint4* src = reinterpret_cast<const uint4*>(x + r * k + kb * 16);
        uint4 u0 = src[0], u1 = src[1];
        float v[16];
        const T* e0 = reinterpret_cast<const T*>(&u0);
        const T* e1 = reinterpret_cast<const T*>(&u1);
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = Cvt<T>::to_f(e0[i]);
            v[8 + i] = Cvt<T>::to_f(e1[i]);
            amax = fmaxf(amax, fmaxf(fabsf(v[i]), fabsf(v[8 + i])));
        }
        uint8_t s8;
        const uint2 packed = nvfp4_quantize_block16(v, amax, gs, inv_gs, s8);
        *reinterpret_cast<uint2*>(xq + r * (k / 2) + kb * 8) = packed;
        sf[sf_atom_offset(r, kb, k64_pad)] = s8;
    }
}

// Row-major scales [rows, k/16] (as stored in checkpoints) → atom layout, zero padded.
__global__ void nvfp4_swizzle_sf_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, long long rows, int kblocks,
                                        int k64_pad) {
    pdl_prologue();
    const long long total = rows * kblocks;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long r = idx / kblocks;
        const int kb = (int)(idx - r * kblocks);
        out[sf_atom_offset(r, kb, k64_pad)] = in[idx];
    }
}

}  // namespace telb

using namespace telb;

extern "C" int telb_gemm_skinny(int kind, const void* x, const void* x_sf, const void* w, const void* w_sf, void* out, int M,
                                int N, int K, const float* alpha, const void* bias, const void* residual, int is_bf16,
                                int* status, int force_ranks, cudaStream_t stream);
extern "C" int telb_gemm_skinny_fused(int kind, const void* x, const void* x_sf, const void* w, const void* w_sf, void* out, int M,
                                      int N, int K, const float* alpha, const void* bias, const void* residual, int is_bf16,
                                      int* status, int force_ranks, const telb::TelbGemmFusion* fusion, cudaStream_t stream);

extern "C" int telb_nvfp4_wide_mode();
extern "C" int telb_gemm_nvfp4_wide_launch(const void* xq, const void* x_sf, const void* wq, const void* w_sf, int M, int N, int K,
                                           const void* params_blob, int pair, cudaStream_t stream);

// Number of 64-element K groups the scale buffers are padded to (whole 256-element stages).
extern "C" int telb_nvfp4_k64_pad(int k) { return ((k + 255) / 256) * 4; }

// Bytes of an atom-layout scale buffer for `rows` x `k`.
extern "C" long long telb_nvfp4_sf_bytes(long long rows, int k) {
    return ((rows + 127) / 128) * (long long)telb_nvfp4_k64_pad(k) * 512;
}

extern "C" int telb_nvfp4_swizzle_scales(const void* sf_rowmajor, void* sf_atoms, long long rows, int k,
                                         cudaStream_t stream) {
    if (k % 16) return fail("telb_nvfp4_swizzle_scales: K must be a multiple of 16");
    cudaError_t e = cudaMemsetAsync(sf_atoms, 0, (size_t)telb_nvfp4_sf_bytes(rows, k), stream);
    if (e != cudaSuccess) return fail("cudaMemsetAsync", e);
    const long long total = rows * (k / 16);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    TELB_LAUNCH("nvfp4_swizzle_sf_kernel", (nvfp4_swizzle_sf_kernel), dim3((int)blocks), dim3(256), 0, stream, (const uint8_t*)sf_rowmajor, (uint8_t*)sf_atoms, rows, k / 16, telb_nvfp4_k64_pad(k));
    TELB_CHECK_LAUNCH("nvfp4_swizzle_sf_kernel");
    return 0;
}

// The scale buffer must have been zeroed once if rows % 128 != 0 or K % 256 != 0 (padding is never written).
extern "C" int telb_nvfp4_quantize(const void* x, void* xq, void* sf_atoms, const float* global_scale, long long rows,
                                   int k, int is_bf16, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (k % 16) return fail("telb_nvfp4_quantize: K must be a multiple of 16");
    const long long total = rows * (k / 16);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (is_bf16)
        TELB_LAUNCH("nvfp4_quantize_kernel", (nvfp4_quantize_kernel<__nv_bfloat16>), dim3((int)blocks), dim3(256), 0, stream, (const __nv_bfloat16*)x, (uint8_t*)xq, (uint8_t*)sf_atoms, global_scale, rows, k, telb_nvfp4_k64_pad(k));
    else
        TELB_LAUNCH("nvfp4_quantize_kernel", (nvfp4_quantize_kernel<__half>), dim3((int)blocks), dim3(256), 0, stream, (const __half*)x, (uint8_t*)xq, (uint8_t*)sf_atoms, global_scale, rows, k, telb_nvfp4_k64_pad(k));
    TELB_CHECK_LAUNCH("nvfp4_quantize_kernel");
    return 0;
}

struct SwigluOut {
    uint8_t* xq;
    uint8_t* sf;
    const float* gs;
    int ld, k64_pad;
};

// out[M,N] = dequant(xq, x_sf)[M,K] · dequant(wq, w_sf)[N,K]^T * alpha[N] (+bias +residual); K % 32 == 0.
static int gemm_nvfp4_impl(const void* xq, const void* x_sf, const void* wq, const void* w_sf, void* out, int M, int N,
                           int K, const float* alpha, const void* bias, const void* residual, int out_bf16, void* ws,
                           long long ws_bytes, int* counters, int n_counters, int* status, int mode, int force_splits,
                           const TelbGemmFusion* fusion, cudaStream_t stream, const SwigluOut* sw = nullptr) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (K % 32) return fail("telb_gemm_nvfp4: K must be a multiple of 32");
    if (fusion && fusion->rs_world > 1 && residual) return fail("telb_gemm_nvfp4: reduce-scatter epilogue takes no residual");
    // decode-size steps keep the swapped-operand kernel when a collective is fused in (it has the same epilogue / prologue)
    if (fusion && M <= 128 && !sw && (fusion->rs_world <= 1 || N % 4 == 0))
        return telb_gemm_skinny_fused(1, xq, x_sf, wq, w_sf, out, M, N, K, alpha, bias, residual, out_bf16, status, 0, fusion, stream);
    if (fusion) mode = 1;         // otherwise the fused collectives run in the large-M layout
    if (mode == 0 && M <= 128)
        return telb_gemm_skinny(1, xq, x_sf, wq, w_sf, out, M, N, K, alpha, bias, residual, out_bf16, status, 0, stream);
    const bool swapped = mode == 2 || (mode == 0 && M <= 128);
    GemmParams p{};
    apply_fusion(p, fusion);
    if (sw) {
        p.sw_xq = sw->xq;
        p.sw_sf = sw->sf;
        p.sw_gs = sw->gs;
        p.sw_ld = sw->ld;
        p.sw_k64_pad = sw->k64_pad;
    }
    // prefill-size problems run on 256-wide tiles (a CTA pair per 256 x 256 tile, or one CTA per 128 x 256 tile)
    const int wide = telb_nvfp4_wide_mode();
    if (!swapped && wide > 0 && N >= 256 && N % 8 == 0 && M > 128) {
        p.c = out;
        p.bias = bias;
        p.alpha = alpha;
        p.residual = residual;
        p.out_bf16 = out_bf16;
        p.status = status;
        return telb_gemm_nvfp4_wide_launch(xq, x_sf, wq, w_sf, M, N, K, &p, wide == 2 ? 1 : 0, stream);
    }
    p.k = K;
    p.kb_total = (K + kFp4BK - 1) / kFp4BK;
    p.c = out;
    p.bias = bias;
    p.alpha = alpha;
    p.residual = residual;
    p.out_bf16 = out_bf16;
    p.ws = static_cast<float*>(ws);
    p.counters = counters;
    p.status = status;
    const int k64 = telb_nvfp4_k64_pad(K);
    CUtensorMap ta, tb;
    int bn;
    const uint8_t *sfa, *sfb;
    const uint64_t kbytes = (uint64_t)K / 2;
    if (swapped) {
        bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
        if (M > 128) return fail("telb_gemm_nvfp4: swapped layout needs M <= 128");
        p.rows_a = N;
        p.rows_b = M;
        p.ldc_lane = 1;
        p.ldc_col = N;
        p.feat_on_lane = 1;
        sfa = (const uint8_t*)w_sf;
        sfb = (const uint8_t*)x_sf;
        if (make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, N, kbytes, kbytes, kBM, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
        if (make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, M, kbytes, kbytes, bn, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    } else {
        bn = 128;
        p.rows_a = M;
        p.rows_b = N;
        p.ldc_lane = N;
        p.ldc_col = 1;
        p.feat_on_lane = 0;
        sfa = (const uint8_t*)x_sf;
        sfb = (const uint8_t*)w_sf;
        if (make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, M, kbytes, kbytes, kBM, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
        if (make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, N, kbytes, kbytes, bn, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    }
    p.tiles_a = (p.rows_a + kBM - 1) / kBM;
    p.tiles_b = (p.rows_b + bn - 1) / bn;
    const int tiles = p.tiles_a * p.tiles_b;
    int splits = 1;
    if (swapped && ws && counters) {
        splits = choose_splits(tiles, p.kb_total, force_splits);
        while (splits > 1 && ((long long)tiles * splits * bn * kBM * 4 > ws_bytes || tiles > n_counters)) --splits;
        if (splits < 1) splits = 1;
    }
    p.kb_per_split = (p.kb_total + splits - 1) / splits;
    p.splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;
    switch (bn) {
        case 16: return launch_nvfp4<16, 8>(ta, tb, sfa, sfb, k64, k64, p, stream);
        case 32: return launch_nvfp4<32, 8>(ta, tb, sfa, sfb, k64, k64, p, stream);
        case 64: return launch_nvfp4<64, 7>(ta, tb, sfa, sfb, k64, k64, p, stream);
        default: return launch_nvfp4<128, 5>(ta, tb, sfa, sfb, k64, k64, p, stream);
    }
}

extern "C" int telb_gemm_nvfp4(const void* xq, const void* x_sf, const void* wq, const void* w_sf, void* out, int M, int N,
                               int K, const float* alpha, const void* bias, const void* residual, int out_bf16, void* ws,
                               long long ws_bytes, int* counters, int n_counters, int* status, int mode, int force_splits,
                               cudaStream_t stream) {
    return gemm_nvfp4_impl(xq, x_sf, wq, w_sf, out, M, N, K, alpha, bias, residual, out_bf16, ws, ws_bytes, counters, n_counters,
                           status, mode, force_splits, nullptr, stream);
}

// Same GEMM with a tensor-parallel collective fused in: a reduce-scatter epilogue (rows stored into
// their owner's partial buffer over peer memory) and / or an all-gather prologue (the producer waits
// for the rows other ranks push into this GPU's copy of the activations).  `out` is unused by the
// reduce-scatter form.
extern "C" int telb_gemm_nvfp4_fused(const void* xq, const void* x_sf, const void* wq, const void* w_sf, void* out, int M, int N,
                                     int K, const float* alpha, const void* bias, int out_bf16, int* status,
                                     const TelbGemmFusion* fusion, cudaStream_t stream) {
    return gemm_nvfp4_impl(xq, x_sf, wq, w_sf, out, M, N, K, alpha, bias, nullptr, out_bf16, nullptr, 0, nullptr, 0, status, 1, 1,
                           fusion, stream);
}

// Gate/up projection with the SwiGLU + NVFP4 quantisation done in the epilogue: wq holds 2 * inter rows in which blocks
// of 64 gate rows alternate with the 64 matching up rows (alpha in the same order); the result is
// quantised silu(gate) * up [M, inter] as packed codes out_xq [M, inter / 2] and atom-layout scales out_sf (pre-zeroed
// by the caller when M % 128 or inter % 256 leave padding).  Large-M layout only (M > 128).
extern "C" int telb_gemm_nvfp4_swiglu(const void* xq, const void* x_sf, const void* wq, const void* w_sf, const float* alpha,
                                      void* out_xq, void* out_sf, const float* out_global_scale, int M, int N, int K, int out_bf16,
                                      int* status, const TelbGemmFusion* fusion, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (N % 128 || K % 32) return fail("telb_gemm_nvfp4_swiglu: N must be a multiple of 128 and K of 32");
    if (fusion && fusion->rs_world > 1) return fail("telb_gemm_nvfp4_swiglu: no reduce-scatter on a column-parallel projection");
    if (M <= 128) return fail("telb_gemm_nvfp4_swiglu: the fused epilogue exists for the large-M layout (M > 128)");
    SwigluOut sw{static_cast<uint8_t*>(out_xq), static_cast<uint8_t*>(out_sf), out_global_scale, N / 4 /* inter / 2 bytes per row */,
                 telb_nvfp4_k64_pad(N / 2)};
    return gemm_nvfp4_impl(xq, x_sf, wq, w_sf, nullptr, M, N, K, alpha, nullptr, nullptr, out_bf16, nullptr, 0, nullptr, 0, status, 1, 1,
                           fusion, stream, &sw);
}

// Grouped NVFP4 GEMM for mixture-of-experts (see telb_gemm_f16_grouped): xq [rows_pad, K/2] with
// atom-layout scales over the padded row space, wq [experts * N, K/2] with scales over experts * N rows.
static int gemm_nvfp4_grouped_impl(const void* xq, const void* x_sf, const void* wq, const void* w_sf, void* out, int rows_pad, int N, int K,
                                   int experts, const int* tile_expert, const float* alpha, int out_bf16, int* status, cudaStream_t stream,
                                   const SwigluOut* sw);

extern "C" int telb_gemm_nvfp4_grouped(const void* xq, const void* x_sf, const void* wq, const void* w_sf, void* out,
                                       int rows_pad, int N, int K, int experts, const int* tile_expert, const float* alpha,
                                       int out_bf16, int* status, cudaStream_t stream) {
    return gemm_nvfp4_grouped_impl(xq, x_sf, wq, w_sf, out, rows_pad, N, K, experts, tile_expert, alpha, out_bf16, status, stream, nullptr);
}

// Grouped gate/up projection with SwiGLU and the NVFP4 quantisation of the second expert GEMM's input in the epilogue.
// Every expert's N = 2 * inter weight rows alternate in blocks of 64 (gate features f .. f+63, then the matching up
// features); the output is packed codes out_xq [rows_pad, inter / 2] with atom-layout scales over rows_pad rows and inter
// columns (padding rows of a tile are not written).  Reference counterpart: the activation-fusion grouped GEMM of
// kernelSrcs/nvfp4_moe_cutedsl/blockscaled_contiguous_gather_grouped_gemm_act_fusion.py.
extern "C" int telb_gemm_nvfp4_grouped_swiglu(const void* xq, const void* x_sf, const void* wq, const void* w_sf, void* out_xq, void* out_sf,
                                              const float* out_global_scale, int rows_pad, int N, int K, int experts, const int* tile_expert,
                                              const float* alpha, int out_bf16, int* status, cudaStream_t stream) {
    if (N % 128) return fail("telb_gemm_nvfp4_grouped_swiglu: 2 * inter must be a multiple of 128");
    if (!out_xq || !out_sf || !out_global_scale) return fail("telb_gemm_nvfp4_grouped_swiglu: output buffers and scale are required");
    SwigluOut sw{static_cast<uint8_t*>(out_xq), static_cast<uint8_t*>(out_sf), out_global_scale, N / 4, telb_nvfp4_k64_pad(N / 2)};
    return gemm_nvfp4_grouped_impl(xq, x_sf, wq, w_sf, nullptr, rows_pad, N, K, experts, tile_expert, alpha, out_bf16, status, stream, &sw);
}

static int gemm_nvfp4_grouped_impl(const void* xq, const void* x_sf, const void* wq, const void* w_sf, void* out, int rows_pad, int N, int K,
                                   int experts, const int* tile_expert, const float* alpha, int out_bf16, int* status, cudaStream_t stream,
                                   const SwigluOut* sw) {
    if (rows_pad <= 0) return 0;
    if (K % 32 || rows_pad % kBM || N % 128) return fail("telb_gemm_nvfp4_grouped: K % 32, rows_pad % 128 and N % 128 must be 0");
    GemmParams p{};
    p.k = K;
    p.kb_total = (K + kFp4BK - 1) / kFp4BK;
    p.c = out;
    p.alpha = alpha;
    p.out_bf16 = out_bf16;
    p.status = status;
    p.rows_a = rows_pad;
    p.rows_b = N;
    p.ldc_lane = N;
    p.ldc_col = 1;
    p.tile_expert = tile_expert;
    p.group_rows_b = N;
    if (sw) {
        p.sw_xq = sw->xq;
        p.sw_sf = sw->sf;
        p.sw_gs = sw->gs;
        p.sw_ld = sw->ld;
        p.sw_k64_pad = sw->k64_pad;
    }
    const uint64_t kbytes = (uint64_t)K / 2;
    CUtensorMap ta, tb;
    if (make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, rows_pad, kbytes, kbytes, kBM, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    if (make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, (uint64_t)experts * N, kbytes, kbytes, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    p.tiles_a = rows_pad / kBM;
    p.tiles_b = N / 128;
    p.splits = 1;
    p.kb_per_split = p.kb_total;
    const int k64 = telb_nvfp4_k64_pad(K);
    return launch_nvfp4<128, 5>(ta, tb, (const uint8_t*)x_sf, (const uint8_t*)w_sf, k64, k64, p, stream);
}
