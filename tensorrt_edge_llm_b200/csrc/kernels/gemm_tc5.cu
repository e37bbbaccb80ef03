// 16-bit (bf16 / fp16) GEMM on 5th-generation tensor cores:  out[M,N] = x[M,K] · w[N,K]ᵀ
// (+ bias, × per-column alpha, + residual), fp32 accumulation in TMEM.
//
// One persistent, warp-specialised kernel serves both regimes:
//   * large M (prefill): x is the MMA-M operand (128-row tiles), w the MMA-N operand (256 rows);
//   * small M (decode):  operands are swapped so the 128-row MMA-M side always streams weights,
//     the token batch is the MMA-N side (16..128), and K is split across CTAs so that all SMs
//     pull weights from HBM.  Split partial tiles meet in an fp32 workspace; the CTA that
//     arrives last at the tile's counter sums them and runs the epilogue (no CTA ever waits on
//     another CTA).
// Roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = UMMA issuer + TMEM owner,
// warps 2-5 = epilogue (one TMEM lane quadrant each).  Accumulators are double-buffered in TMEM
// so the epilogue of tile i overlaps the main loop of tile i+1.
//
// Reference counterpart: the dense projections are TensorRT MatMul tactics inside the engine and
// CuTe-DSL `gemm_blackwell.py` for auxiliary GEMMs (kernelSrcs/gemm_cutedsl/); this kernel is
// written from the PTX up and shares no code with either.
#include "gemm_common.cuh"

namespace telb {

template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc5_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, GemmParams p) {
    constexpr int kBTileBytes = BN * kBK * 2;
    constexpr int kStageBytes = kATileBytes + kBTileBytes;
    constexpr int kAccStride = BN < 32 ? 32 : BN;          // TMEM columns per accumulator buffer
    constexpr int kTmemCols = 2 * kAccStride;               // power of two for every BN used here

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
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const int ag_e = p.ag_flags ? *p.ag_epoch : 0;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const TileCoord tc = decode_tile(p, t);
                if (tc.skip) continue;
                const int brow = (tc.brow >= 0 ? tc.brow : 0) + tc.b0 * BN;
                if (p.ag_flags && !ag_wait_rows(p, tc.a0, ag_e, abort_flag)) break;
                for (int kb = tc.kb0; kb < tc.kb1; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + stage * kStageBytes;
                    mbar_expect_tx(&full_bar[stage], kStageBytes);
                    tma_load_2d(sa, &tma_a, &full_bar[stage], kb * kBK, tc.a0);
                    tma_load_2d(sa + kATileBytes, &tma_b, &full_bar[stage], kb * kBK, brow);
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
            const uint32_t idesc = idesc_f16(kBM, BN, p.out_bf16 != 0);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
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
                    const uint64_t da = smem_desc_sw128(sa);
                    const uint64_t db = smem_desc_sw128(sa + kATileBytes);
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k)   // 16 elements = 32 bytes = 2 descriptor units
                        umma_f16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > tc.kb0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty_bar[stage]);
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

    // ---------------- common exit ----------------
    if (*abort_flag) {
        // Give copies that are still in flight time to land before shared memory is handed back.
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
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
    constexpr int kStageBytes = kATileBytes + BN * kBK * 2;
    constexpr int smem = STAGES * kStageBytes + 1024 /*align slack*/ + 256 /*barriers*/ + kRsStageBytes + kAlphaStageBytes;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc5_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail("cudaFuncSetAttribute(gemm_tc5)", e);
        configured = true;
    }
    const int total = p.tiles_a * p.tiles_b * p.splits;
    const int grid = total < sm_count() ? total : sm_count();
    TELB_LAUNCH("gemm_tc5_kernel", (gemm_tc5_kernel<BN, STAGES>), dim3(grid), dim3(kGemmThreads), smem, stream, ta, tb, p);
    TELB_CHECK_LAUNCH("gemm_tc5_kernel");
    return 0;
}

}  // namespace telb

using namespace telb;

extern "C" int telb_gemm_skinny(int kind, const void* x, const void* x_sf, const void* w, const void* w_sf, void* out, int M,
                                int N, int K, const float* alpha, const void* bias, const void* residual, int is_bf16,
                                int* status, int force_ranks, cudaStream_t stream);
extern "C" int telb_gemm_skinny_fused(int kind, const void* x, const void* x_sf, const void* w, const void* w_sf, void* out, int M,
                                      int N, int K, const float* alpha, const void* bias, const void* residual, int is_bf16,
                                      int* status, int force_ranks, const telb::TelbGemmFusion* fusion, cudaStream_t stream);

extern "C" const char* telb_last_error() { return g_last_error; }

// out[M,N] = x[M,K] · w[N,K]^T  (16-bit row-major operands, K % 8 == 0).
//   bias / alpha : per output column (may be null);  residual : [M,N] like out (may be null)
//   ws / counters: split-K scratch, used only by the small-M path (ws_bytes may be 0 → no split)
//   mode         : 0 = choose, 1 = force large-M layout, 2 = force swapped layout
static int gemm_f16_impl(const void* x, const void* w, void* out, int M, int N, int K, const void* bias,
                         const float* alpha, const void* residual, int is_bf16, void* ws, long long ws_bytes,
                         int* counters, int n_counters, int* status, int mode, int force_splits,
                         const TelbGemmFusion* fusion, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (fusion && fusion->rs_world > 1 && residual) return fail("telb_gemm_f16: reduce-scatter epilogue takes no residual");
    if (K % 8) return fail("telb_gemm_f16: K must be a multiple of 8");
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return fail("telb_gemm_f16: operands must be 16-byte aligned");
    // decode-size steps keep the swapped-operand kernel when a collective is fused in (it has the same epilogue / prologue)
    if (fusion && M <= 128 && (fusion->rs_world <= 1 || N % 4 == 0))
        return telb_gemm_skinny_fused(0, x, nullptr, w, nullptr, out, M, N, K, alpha, bias, residual, is_bf16, status, 0, fusion, stream);
    if (fusion) mode = 1;         // otherwise the fused collectives run in the large-M layout
    if (mode == 0 && M <= 128)
        return telb_gemm_skinny(0, x, nullptr, w, nullptr, out, M, N, K, alpha, bias, residual, is_bf16, status, 0, stream);
    const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const bool swapped = mode == 2 || (mode == 0 && M <= 128);
    GemmParams p{};
    apply_fusion(p, fusion);
    p.k = K;
    p.kb_total = (K + kBK - 1) / kBK;
    p.c = out;
    p.bias = bias;
    p.alpha = alpha;
    p.residual = residual;
    p.out_bf16 = is_bf16;
    p.ws = static_cast<float*>(ws);
    p.counters = counters;
    p.status = status;
    CUtensorMap ta, tb;
    int bn;
    if (swapped) {
        bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
        p.rows_a = N;
        p.rows_b = M;
        p.ldc_lane = 1;
        p.ldc_col = N;
        p.feat_on_lane = 1;
        if (make_tmap_2d(&ta, dt, 2, w, N, K, (uint64_t)K * 2, kBM, kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
        if (make_tmap_2d(&tb, dt, 2, x, M, K, (uint64_t)K * 2, bn, kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    } else {
        bn = (N >= 256) ? 256 : (N > 64 ? 128 : 64);
        p.rows_a = M;
        p.rows_b = N;
        p.ldc_lane = N;
        p.ldc_col = 1;
        p.feat_on_lane = 0;
        if (make_tmap_2d(&ta, dt, 2, x, M, K, (uint64_t)K * 2, kBM, kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
        if (make_tmap_2d(&tb, dt, 2, w, N, K, (uint64_t)K * 2, bn, kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
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
    p.splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;   // no empty split
    switch (bn) {
        case 16: return launch_gemm<16, 8>(ta, tb, p, stream);
        case 32: return launch_gemm<32, 8>(ta, tb, p, stream);
        case 64: return launch_gemm<64, 8>(ta, tb, p, stream);
        case 128: return launch_gemm<128, 6>(ta, tb, p, stream);
        default: return launch_gemm<256, 4>(ta, tb, p, stream);
    }
}

extern "C" int telb_gemm_f16(const void* x, const void* w, void* out, int M, int N, int K, const void* bias,
                             const float* alpha, const void* residual, int is_bf16, void* ws, long long ws_bytes,
                             int* counters, int n_counters, int* status, int mode, int force_splits,
                             cudaStream_t stream) {
    return gemm_f16_impl(x, w, out, M, N, K, bias, alpha, residual, is_bf16, ws, ws_bytes, counters, n_counters, status, mode,
                         force_splits, nullptr, stream);
}

// Same GEMM with a tensor-parallel collective fused in (see TelbGemmFusion): reduce-scatter epilogue
// and / or all-gather prologue.  `out` is unused by the reduce-scatter form.
extern "C" int telb_gemm_f16_fused(const void* x, const void* w, void* out, int M, int N, int K, const void* bias,
                                   const float* alpha, int is_bf16, int* status, const TelbGemmFusion* fusion,
                                   cudaStream_t stream) {
    return gemm_f16_impl(x, w, out, M, N, K, bias, alpha, nullptr, is_bf16, nullptr, 0, nullptr, 0, status, 1, 1, fusion, stream);
}

// Grouped form for mixture-of-experts: x [rows_pad, K] is the routed activations in 128-row padded
// expert segments, w [experts * N, K] the stacked expert weights, tile_expert[rows_pad / 128] the
// expert of every row tile (-1 = unused).  out [rows_pad, N].  alpha / bias: [experts * N] or null.
extern "C" int telb_gemm_f16_grouped(const void* x, const void* w, void* out, int rows_pad, int N, int K, int experts,
                                     const int* tile_expert, const float* alpha, const void* bias, int is_bf16, int* status,
                                     cudaStream_t stream) {
    if (rows_pad <= 0) return 0;
    if (K % 8 || rows_pad % kBM || N % 8) return fail("telb_gemm_f16_grouped: K % 8, rows_pad % 128 and N % 8 must be 0");
    const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    GemmParams p{};
    p.k = K;
    p.kb_total = (K + kBK - 1) / kBK;
    p.c = out;
    p.alpha = alpha;
    p.bias = bias;
    p.out_bf16 = is_bf16;
    p.status = status;
    p.rows_a = rows_pad;
    p.rows_b = N;
    p.ldc_lane = N;
    p.ldc_col = 1;
    p.tile_expert = tile_expert;
    p.group_rows_b = N;
    const int bn = N >= 256 && N % 256 == 0 ? 256 : 128;
    if (N % bn) return fail("telb_gemm_f16_grouped: N must be a multiple of 128");
    CUtensorMap ta, tb;
    if (make_tmap_2d(&ta, dt, 2, x, rows_pad, K, (uint64_t)K * 2, kBM, kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    if (make_tmap_2d(&tb, dt, 2, w, (uint64_t)experts * N, K, (uint64_t)K * 2, bn, kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    p.tiles_a = rows_pad / kBM;
    p.tiles_b = N / bn;
    p.splits = 1;
    p.kb_per_split = p.kb_total;
    return bn == 256 ? launch_gemm<256, 4>(ta, tb, p, stream) : launch_gemm<128, 6>(ta, tb, p, stream);
}
