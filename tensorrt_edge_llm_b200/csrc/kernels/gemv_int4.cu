// W4A16 GEMV for one to four token rows: out[M, N] = x[M, K] · dequant(wq, scales)[N, K]ᵀ (+ bias, + residual).
//
// With so few rows a tensor-core tile is almost empty and the expansion of the 4-bit tile into a 16-bit operand tile
// (gemm_skinny_tc5.cu, KIND 2) costs more than the multiply; here one warp owns a pair of output rows (one byte row of the
// ModelOpt-prepacked layout [N / 2, K]: low nibble = row 2r, high nibble = row 2r + 1, codes offset by 8) and streams it once
// with 16-byte loads.  A code becomes the float (q − 8) without an integer-to-float conversion: OR-ed into the mantissa of
// 2^23 it is the number 8388608 + q exactly, and one subtraction of 8388616 leaves q − 8.  The group scale (one per row and
// `group` input columns) multiplies the partial sum of a 16-column piece, which never straddles a group.  x rows live in
// shared memory as 16-bit values; sums are fp32, reduced across the warp with shuffles.
//
// Reference counterpart: cpp/kernels/int4GroupwiseGemmKernels/int4WoqGemmCuda.cu (the GEMV path, :98-124).
#include "host_utils.h"
#include "tc5_common.cuh"

namespace telb {

template <typename T, int M>
__global__ void __launch_bounds__(256)
int4_gemv_kernel(const T* __restrict__ x, const uint4* __restrict__ wq, const T* __restrict__ scales, T* __restrict__ out,
                 const T* __restrict__ bias, const T* __restrict__ residual, int n, int k, int group) {
    extern __shared__ uint4 s_x4[];
    T* s_x = reinterpret_cast<T*>(s_x4);
    pdl_prologue();
    for (int i = threadIdx.x; i < M * k / 8; i += blockDim.x) s_x4[i] = reinterpret_cast<const uint4*>(x)[i];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rp = blockIdx.x * (blockDim.x >> 5) + warp;           // byte row = output rows 2 rp and 2 rp + 1
    if (rp * 2 >= n) return;
    const int gpr = k / group;
    const T* sc0 = scales + (size_t)(2 * rp) * gpr;
    const T* sc1 = sc0 + gpr;
    const uint4* wrow = wq + (size_t)rp * (k / 16);
    float acc0[M], acc1[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc0[m] = acc1[m] = 0.f;
    for (int c = lane; c < k / 16; c += 32) {
        const uint4 wv = __ldg(&wrow[c]);
        const int g = (c * 16) / group;
        const float s0 = Cvt<T>::to_f(sc0[g]), s1 = Cvt<T>::to_f(sc1[g]);
        const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
        float lo[16], hi[16];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                lo[j * 4 + b] = __uint_as_float(((w[j] >> (8 * b)) & 0xFu) | 0x4B000000u) - 8388616.f;
                hi[j * 4 + b] = __uint_as_float(((w[j] >> (8 * b + 4)) & 0xFu) | 0x4B000000u) - 8388616.f;
            }
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint4 xa = *reinterpret_cast<const uint4*>(s_x + (size_t)m * k + c * 16);
            const uint4 xb = *reinterpret_cast<const uint4*>(s_x + (size_t)m * k + c * 16 + 8);
            const T* pa = reinterpret_cast<const T*>(&xa);
            const T* pb = reinterpret_cast<const T*>(&xb);
            float d0 = 0.f, d1 = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float xv = Cvt<T>::to_f(pa[i]), xw = Cvt<T>::to_f(pb[i]);
                d0 = fmaf(lo[i], xv, d0);
                d1 = fmaf(hi[i], xv, d1);
                d0 = fmaf(lo[8 + i], xw, d0);
                d1 = fmaf(hi[8 + i], xw, d1);
            }
            acc0[m] = fmaf(s0, d0, acc0[m]);
            acc1[m] = fmaf(s1, d1, acc1[m]);
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            acc0[m] += __shfl_xor_sync(0xffffffffu, acc0[m], o);
            acc1[m] += __shfl_xor_sync(0xffffffffu, acc1[m], o);
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float y0 = acc0[m], y1 = acc1[m];
            const size_t o = (size_t)m * n + 2 * rp;
            if (bias) {
                y0 += Cvt<T>::to_f(bias[2 * rp]);
                y1 += Cvt<T>::to_f(bias[2 * rp + 1]);
            }
            if (residual) {
                y0 += Cvt<T>::to_f(residual[o]);
                y1 += Cvt<T>::to_f(residual[o + 1]);
            }
            out[o] = Cvt<T>::from_f(y0);
            out[o + 1] = Cvt<T>::from_f(y1);
        }
    }
}

template <typename T, int M>
static int launch_int4_gemv(const void* x, const void* wq, const void* scales, void* out, const void* bias, const void* residual, int n,
                            int k, int group, cudaStream_t stream) {
    const int smem = M * k * 2;
    static int configured = 0;
    if (smem > 48 * 1024 && configured < smem) {
        cudaError_t e = cudaFuncSetAttribute(int4_gemv_kernel<T, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail("cudaFuncSetAttribute(int4_gemv)", e);
        configured = smem;
    }
    const int pairs = n / 2;
    TELB_LAUNCH("int4_gemv_kernel", (int4_gemv_kernel<T, M>), dim3((pairs + 7) / 8), dim3(256), smem, stream, (const T*)x, (const uint4*)wq,
                (const T*)scales, (T*)out, (const T*)bias, (const T*)residual, n, k, group);
    TELB_CHECK_LAUNCH("int4_gemv_kernel");
    return 0;
}

}  // namespace telb

using namespace telb;

// x [M, K] (M = 1..4), wq [N / 2, K] packed INT4, scales [N, K / group] in the activation type; K % 16 == 0, group % 16 == 0.
extern "C" int telb_gemv_int4(const void* x, const void* wq, const void* scales, void* out, int M, int N, int K, int group, const void* bias,
                              const void* residual, int is_bf16, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 4) return fail("telb_gemv_int4: at most four rows");
    if (N % 2 || K % 16 || group <= 0 || group % 16 || K % group) return fail("telb_gemv_int4: even N, K % 16 == 0 and a group (multiple of 16) that divides K are required");
    if ((long long)M * K * 2 > 200 * 1024) return fail("telb_gemv_int4: the input rows do not fit shared memory");
#define TELB_GEMV(T_)                                                                                        \
    switch (M) {                                                                                             \
        case 1: return launch_int4_gemv<T_, 1>(x, wq, scales, out, bias, residual, N, K, group, stream);    \
        case 2: return launch_int4_gemv<T_, 2>(x, wq, scales, out, bias, residual, N, K, group, stream);    \
        case 3: return launch_int4_gemv<T_, 3>(x, wq, scales, out, bias, residual, N, K, group, stream);    \
        default: return launch_int4_gemv<T_, 4>(x, wq, scales, out, bias, residual, N, K, group, stream);   \
    }
    if (is_bf16) {
        TELB_GEMV(__nv_bfloat16)
    } else {
        TELB_GEMV(__half)
    }
#undef TELB_GEMV
}
