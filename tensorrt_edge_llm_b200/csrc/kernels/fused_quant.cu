// Producers that hand their result to an NVFP4 GEMM without a 16-bit round trip through HBM:
//   * (residual add +) RMSNorm → E2M1 codes + UE4M3 block scales in the tensor-core atom layout
//   * SwiGLU (silu(gate) * up) → the same
// Both keep the reference numerics of the unfused chain: the normalised / activated value is
// rounded to the 16-bit activation type first and quantised from that rounded value, exactly as
// if the 16-bit tensor had been written and re-read.
//
// Reference counterparts: CuTe-DSL rmsnorm + cpp/kernels/moe/fp4SupportKernels/fp4Quantize.cu run
// as separate launches; the dual-GEMM variants with FP4 output
// (kernelSrcs/gemm_cutedsl/gemm_blackwell_nvfp4_ws.py `dual_gemm_blackwell_nvfp4_output`) fuse the
// SwiGLU side into the GEMM instead.
#include "host_utils.h"
#include "nvfp4_common.cuh"

namespace telb {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One CTA per row; thread t owns the 16-element blocks t, t + blockDim, ... (kUnits per thread).
template <typename T, int kUnits>
__global__ void rmsnorm_quant_kernel(const T* __restrict__ x, const T* __restrict__ residual, const T* __restrict__ w,
                                     T* __restrict__ res_out, T* __restrict__ y_out, uint8_t* __restrict__ xq,
                                     uint8_t* __restrict__ sf, const float* __restrict__ global_scale, int hidden,
                                     int k64_pad, float eps) {
    pdl_prologue();
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const int nunits = hidden / 16;
    float v[kUnits][16];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < kUnits; ++u) {
        const int idx = threadIdx.x + u * blockDim.x;
        if (idx < nunits) {
            const T* src = x + row * hidden + idx * 16;
            uint4 a0 = reinterpret_cast<const uint4*>(src)[0], a1 = reinterpret_cast<const uint4*>(src)[1];
            const T* e0 = reinterpret_cast<const T*>(&a0);
            const T* e1 = reinterpret_cast<const T*>(&a1);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[u][i] = Cvt<T>::to_f(e0[i]);
                v[u][8 + i] = Cvt<T>::to_f(e1[i]);
            }
            if (residual) {
                const T* rs = residual + row * hidden + idx * 16;
                uint4 r0 = reinterpret_cast<const uint4*>(rs)[0], r1 = reinterpret_cast<const uint4*>(rs)[1];
                const T* f0 = reinterpret_cast<const T*>(&r0);
                const T* f1 = reinterpret_cast<const T*>(&r1);
                T o[16];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    o[i] = Cvt<T>::from_f(v[u][i] + Cvt<T>::to_f(f0[i]));
                    o[8 + i] = Cvt<T>::from_f(v[u][8 + i] + Cvt<T>::to_f(f1[i]));
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) v[u][i] = Cvt<T>::to_f(o[i]);
                if (res_out) {
                    reinterpret_cast<uint4*>(res_out + row * hidden + idx * 16)[0] = *reinterpret_cast<uint4*>(&o[0]);
                    reinterpret_cast<uint4*>(res_out + row * hidden + idx * 16)[1] = *reinterpret_cast<uint4*>(&o[8]);
                }
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) ss += v[u][i] * v[u][i];
        }
    }
    ss = warp_sum_f(ss);
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) red[wid] = ss;
    __syncthreads();
    float tot = lane < nw ? red[lane] : 0.f;
    tot = warp_sum_f(tot);
    const float inv = rsqrtf(tot / hidden + eps);
    const float gs = *global_scale;
    const float inv_gs = 1.f / gs;
#pragma unroll
    for (int u = 0; u < kUnits; ++u) {
        const int idx = threadIdx.x + u * blockDim.x;
        if (idx < nunits) {
            const T* wp = w + idx * 16;
            uint4 w0 = reinterpret_cast<const uint4*>(wp)[0], w1 = reinterpret_cast<const uint4*>(wp)[1];
            const T* g0 = reinterpret_cast<const T*>(&w0);
            const T* g1 = reinterpret_cast<const T*>(&w1);
            float y[16];
            T yo[16];
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float n = Cvt<T>::to_f(Cvt<T>::from_f(v[u][i] * inv));
                yo[i] = Cvt<T>::from_f(n * Cvt<T>::to_f(i < 8 ? g0[i] : g1[i - 8]));
                y[i] = Cvt<T>::to_f(yo[i]);
                amax = fmaxf(amax, fabsf(y[i]));
            }
            if (y_out) {
                reinterpret_cast<uint4*>(y_out + row * hidden + idx * 16)[0] = *reinterpret_cast<uint4*>(&yo[0]);
                reinterpret_cast<uint4*>(y_out + row * hidden + idx * 16)[1] = *reinterpret_cast<uint4*>(&yo[8]);
            }
            uint8_t s8;
            const uint2 packed = nvfp4_quantize_block16(y, amax, gs, inv_gs, s8);
            *reinterpret_cast<uint2*>(xq + row * (hidden / 2) + idx * 8) = packed;
            sf[sf_atom_offset((long long)row, idx, k64_pad)] = s8;
        }
    }
}

// in [rows, 2*inter] (gate | up) → quantised silu(gate)*up [rows, inter]; one thread per 16 outputs.
template <typename T>
__global__ void swiglu_quant_kernel(const T* __restrict__ in, uint8_t* __restrict__ xq, uint8_t* __restrict__ sf,
                                    const float* __restrict__ global_scale, long long rows, int inter, int k64_pad, int interleaved,
                                    const int* __restrict__ tile_rows) {
    pdl_prologue();
    const int units = inter / 16;
    const long long total = rows * units;
    const float gs = *global_scale;
    const float inv_gs = 1.f / gs;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long r = idx / units;
        const int u = (int)(idx - r * units);
        if (tile_rows && (int)(r & 127) >= tile_rows[r >> 7]) continue;       // padding row of a grouped (MoE) buffer
        // plain layout: [gate(inter) | up(inter)]; interleaved: blocks of 64 gate features followed by their 64 up features
        const T* gp = interleaved ? in + r * 2 * inter + (u >> 2) * 128 + (u & 3) * 16 : in + r * 2 * inter + u * 16;
        const T* up = interleaved ? gp + 64 : gp + inter;
        uint4 g0 = reinterpret_cast<const uint4*>(gp)[0], g1 = reinterpret_cast<const uint4*>(gp)[1];
        uint4 u0 = reinterpret_cast<const uint4*>(up)[0], u1 = reinterpret_cast<const uint4*>(up)[1];
        const T* ge0 = reinterpret_cast<const T*>(&g0);
        const T* ge1 = reinterpret_cast<const T*>(&g1);
        const T* ue0 = reinterpret_cast<const T*>(&u0);
        const T* ue1 = reinterpret_cast<const T*>(&u1);
        float y[16];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float g = Cvt<T>::to_f(i < 8 ? ge0[i] : ge1[i - 8]);
            const float uu = Cvt<T>::to_f(i < 8 ? ue0[i] : ue1[i - 8]);
            y[i] = Cvt<T>::to_f(Cvt<T>::from_f(g / (1.f + __expf(-g)) * uu));
            amax = fmaxf(amax, fabsf(y[i]));
        }
        uint8_t s8;
        const uint2 packed = nvfp4_quantize_block16(y, amax, gs, inv_gs, s8);
        *reinterpret_cast<uint2*>(xq + r * (inter / 2) + u * 8) = packed;
        sf[sf_atom_offset(r, u, k64_pad)] = s8;
    }
}

}  // namespace telb

using namespace telb;

extern "C" int telb_nvfp4_k64_pad(int k);

// y_out / res_out / residual may be null.  The scale buffer must be pre-zeroed when rows % 128 or
// hidden % 256 leave padding.
extern "C" int telb_rmsnorm_quant(const void* x, const void* residual, const void* w, void* res_out, void* y_out, void* xq,
                                  void* sf, const float* global_scale, long long rows, int hidden, float eps, int is_bf16,
                                  cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden % 16) return fail("telb_rmsnorm_quant: hidden must be a multiple of 16");
    const int units = hidden / 16;
    int threads = units >= 256 ? 256 : ((units + 31) / 32) * 32;
    const int per = (units + threads - 1) / threads;
    if (per > 4) return fail("telb_rmsnorm_quant: hidden too large (max 16384)");
    const int k64 = telb_nvfp4_k64_pad(hidden);
#define TELB_RQ(T_, U_)                                                                                            \
    TELB_LAUNCH("rmsnorm_quant_kernel", (rmsnorm_quant_kernel<T_, U_>), dim3((unsigned)rows), dim3(threads), 0, stream, \
                (const T_*)x, (const T_*)residual, (const T_*)w, (T_*)res_out, (T_*)y_out, (uint8_t*)xq, (uint8_t*)sf, \
                global_scale, hidden, k64, eps)
    if (is_bf16) {
        if (per <= 1) TELB_RQ(__nv_bfloat16, 1); else if (per <= 2) TELB_RQ(__nv_bfloat16, 2); else TELB_RQ(__nv_bfloat16, 4);
    } else {
        if (per <= 1) TELB_RQ(__half, 1); else if (per <= 2) TELB_RQ(__half, 2); else TELB_RQ(__half, 4);
    }
#undef TELB_RQ
    TELB_CHECK_LAUNCH("rmsnorm_quant_kernel");
    return 0;
}

extern "C" int telb_swiglu_quant_il(const void* in, void* xq, void* sf, const float* global_scale, long long rows, int inter,
                                    int is_bf16, int interleaved, cudaStream_t stream);
extern "C" int telb_swiglu_quant_rows(const void* in, void* xq, void* sf, const float* global_scale, long long rows, int inter,
                                      int is_bf16, int interleaved, const int* tile_rows, cudaStream_t stream);

extern "C" int telb_swiglu_quant(const void* in, void* xq, void* sf, const float* global_scale, long long rows, int inter,
                                 int is_bf16, cudaStream_t stream) {
    return telb_swiglu_quant_il(in, xq, sf, global_scale, rows, inter, is_bf16, 0, stream);
}

extern "C" int telb_swiglu_quant_il(const void* in, void* xq, void* sf, const float* global_scale, long long rows, int inter,
                                    int is_bf16, int interleaved, cudaStream_t stream) {
    return telb_swiglu_quant_rows(in, xq, sf, global_scale, rows, inter, is_bf16, interleaved, nullptr, stream);
}

// `tile_rows` (optional): rows in use per 128-row tile of a grouped buffer; the other rows are skipped.
extern "C" int telb_swiglu_quant_rows(const void* in, void* xq, void* sf, const float* global_scale, long long rows, int inter,
                                      int is_bf16, int interleaved, const int* tile_rows, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (inter % 16) return fail("telb_swiglu_quant: intermediate size must be a multiple of 16");
    if (interleaved && inter % 64) return fail("telb_swiglu_quant: the interleaved layout needs an intermediate size that is a multiple of 64");
    const long long total = rows * (inter / 16);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    const int k64 = telb_nvfp4_k64_pad(inter);
    if (is_bf16)
        TELB_LAUNCH("swiglu_quant_kernel", (swiglu_quant_kernel<__nv_bfloat16>), dim3((int)blocks), dim3(256), 0, stream, (const __nv_bfloat16*)in, (uint8_t*)xq, (uint8_t*)sf, global_scale, rows, inter, k64, interleaved, tile_rows);
    else
        TELB_LAUNCH("swiglu_quant_kernel", (swiglu_quant_kernel<__half>), dim3((int)blocks), dim3(256), 0, stream, (const __half*)in, (uint8_t*)xq, (uint8_t*)sf, global_scale, rows, inter, k64, interleaved, tile_rows);
    TELB_CHECK_LAUNCH("swiglu_quant_kernel");
    return 0;
}
