// FP8 (E4M3) KV-cache storage: the paged pool holds one byte per element with one dequantisation scale per layer for K and
// one for V (value = fp8 * scale, scale = amax / 448 from calibration, 1.0 by default); the attention kernels of this library
// read 16-bit tiles, so a layer's attention works on a 16-bit staging copy of the pages it touches:
//
//   kv_fp8_load    for every sequence of the step, expand the pages that hold its cached tokens [0, past) from the FP8 pool
//                  into the staging layer (same page indices, same [2, Hkv, P, D] layout);
//   (RoPE + KV write puts the step's new rows into the staging layer, 16-bit, as for an unquantised cache)
//   kv_fp8_store   quantise those new rows into the FP8 pool and write the rounded values back into the staging layer, so
//                  the step attends to exactly what later steps will read.
//
// The saving is capacity (half the bytes per cached token); bandwidth per step is not reduced on this path.
// Reference counterparts: FP8 KV write in cpp/kernels/posEncoding/applyRopeWriteKV.cu:286-297 and the dequantise-before-
// attention fallback described in docs/source/user_guide/features/FP8KV.md ("Other GPUs dequantize K/V to FP16").
#include <cuda_fp8.h>

#include "host_utils.h"
#include "tc5_common.cuh"

namespace telb {

template <typename T>
__device__ __forceinline__ void fp8x16_to_t(const uint4& in, float scale, uint4& lo, uint4& hi) {
    const __nv_fp8_storage_t* b = reinterpret_cast<const __nv_fp8_storage_t*>(&in);
    T out[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) out[i] = Cvt<T>::from_f(__half2float(__half(__nv_cvt_fp8_to_halfraw(b[i], __NV_E4M3))) * scale);
    lo = *reinterpret_cast<const uint4*>(&out[0]);
    hi = *reinterpret_cast<const uint4*>(&out[8]);
}

// grid (max logical pages, sequences); a CTA expands one page (K and V slabs of all heads).
template <typename T>
__global__ void __launch_bounds__(256)
kv_fp8_load_kernel(const uint4* __restrict__ pool, uint4* __restrict__ stage, const int* __restrict__ past_len,
                   const int* __restrict__ page_table, const float* __restrict__ scales, int max_pages, int page_size, int hkv, int d,
                   int window) {
    pdl_prologue();
    const int seq = blockIdx.y, lp = blockIdx.x;
    const int past = past_len[seq];
    if (lp * page_size >= past) return;                              // holds no cached token of this sequence
    if (window > 0 && (lp + 1) * page_size + 2 * 128 <= past - window) return;      // wholly outside every kernel's window tiles
    const int page = page_table[(size_t)seq * max_pages + lp];
    if (page < 0) return;
    const int vec_per_slab = hkv * page_size * d / 16;               // 16 FP8 elements per 16-byte vector
    const uint4* src = pool + (size_t)page * 2 * vec_per_slab;
    uint4* dst = stage + (size_t)page * 2 * vec_per_slab * 2;        // two 16-byte vectors of 16-bit values per source vector
    const float ks = scales[0], vs = scales[1];
    for (int i = threadIdx.x; i < 2 * vec_per_slab; i += blockDim.x) {
        uint4 lo, hi;
        fp8x16_to_t<T>(src[i], i < vec_per_slab ? ks : vs, lo, hi);
        dst[2 * i] = lo;
        dst[2 * i + 1] = hi;
    }
}

// One CTA per token: its 2 * Hkv cache rows (and, when given, its Hq query rows, cast to E4M3 with saturation and scale 1 for the
// attention kernel that reads FP8 pages in place) are walked in pieces of eight elements.
template <typename T>
__global__ void __launch_bounds__(256)
kv_fp8_store_kernel(uint8_t* __restrict__ pool, T* __restrict__ stage, const int* __restrict__ seq_ids,
                    const int* __restrict__ q_start, const int* __restrict__ past_len, const int* __restrict__ page_table,
                    const int* __restrict__ kv_offsets, const float* __restrict__ scales, int max_pages, int page_size,
                    int hkv, int d, const T* __restrict__ q, uint8_t* __restrict__ q8, int hq) {
    pdl_prologue();
    const int t = blockIdx.x;
    const int s = seq_ids[t];
    const int off = kv_offsets ? kv_offsets[t] : (t - q_start[s]);
    const int slot = past_len[s] + off;
    const int page = page_table[(size_t)s * max_pages + slot / page_size];
    const int per_row = d / 8;
    const int kv_pieces = page >= 0 ? 2 * hkv * per_row : 0;
    for (int i = threadIdx.x; i < kv_pieces; i += blockDim.x) {
        const int rowi = i / per_row, e0 = (i - rowi * per_row) * 8;
        const int kv = rowi / hkv, head = rowi - kv * hkv;
        const size_t row = ((((size_t)page * 2 + kv) * hkv + head) * page_size + slot % page_size) * d;
        const float scale = scales[kv];
        const float inv = scale > 0.f ? 1.f / scale : 0.f;
        uint4 v = *reinterpret_cast<const uint4*>(stage + row + e0);
        T* x = reinterpret_cast<T*>(&v);
        uint2 packed;
        uint8_t* pb = reinterpret_cast<uint8_t*>(&packed);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const __nv_fp8_storage_t qv = __nv_cvt_float_to_fp8(Cvt<T>::to_f(x[j]) * inv, __NV_SATFINITE, __NV_E4M3);
            pb[j] = qv;
            x[j] = Cvt<T>::from_f(__half2float(__half(__nv_cvt_fp8_to_halfraw(qv, __NV_E4M3))) * scale);
        }
        *reinterpret_cast<uint2*>(pool + row + e0) = packed;
        *reinterpret_cast<uint4*>(stage + row + e0) = v;
    }
    if (q != nullptr) {
        const int q_pieces = hq * per_row;
        const size_t base = (size_t)t * hq * d;
        for (int i = threadIdx.x; i < q_pieces; i += blockDim.x) {
            const uint4 v = *reinterpret_cast<const uint4*>(q + base + (size_t)i * 8);
            const T* x = reinterpret_cast<const T*>(&v);
            uint2 packed;
            uint8_t* pb = reinterpret_cast<uint8_t*>(&packed);
#pragma unroll
            for (int j = 0; j < 8; ++j) pb[j] = __nv_cvt_float_to_fp8(Cvt<T>::to_f(x[j]), __NV_SATFINITE, __NV_E4M3);
            *reinterpret_cast<uint2*>(q8 + base + (size_t)i * 8) = packed;
        }
    }
}

}  // namespace telb

using namespace telb;

// pool: FP8 [pages, 2, Hkv, P, D] of one layer; stage: 16-bit tensor of the same shape; scales: fp32 [2] (K, V).
extern "C" int telb_kv_fp8_load(const void* pool, void* stage, const int* past_len, const int* page_table, const float* scales, int num_seqs,
                                int max_pages, int page_size, int hkv, int d, int window, int is_bf16, cudaStream_t stream) {
    if (num_seqs <= 0) return 0;
    if ((hkv * page_size * d) % 16) return fail("telb_kv_fp8_load: a K / V slab must be a multiple of 16 elements");
    const dim3 grid(max_pages, num_seqs), blk(256);
    if (is_bf16)
        TELB_LAUNCH("kv_fp8_load_kernel", (kv_fp8_load_kernel<__nv_bfloat16>), grid, blk, 0, stream, (const uint4*)pool, (uint4*)stage, past_len,
                    page_table, scales, max_pages, page_size, hkv, d, window);
    else
        TELB_LAUNCH("kv_fp8_load_kernel", (kv_fp8_load_kernel<__half>), grid, blk, 0, stream, (const uint4*)pool, (uint4*)stage, past_len,
                    page_table, scales, max_pages, page_size, hkv, d, window);
    return 0;
}

// `q` / `q8` (both or neither): the step's query rows [tokens, hq, d] and their E4M3 copy, cast in the same launch.
extern "C" int telb_kv_fp8_store(void* pool, void* stage, const int* seq_ids, const int* q_start, const int* past_len, const int* page_table,
                                 const int* kv_offsets, const float* scales, int tokens, int max_pages, int page_size, int hkv, int d,
                                 int is_bf16, const void* q, void* q8, int hq, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (d % 8 || d > 1024) return fail("telb_kv_fp8_store: head_dim must be a multiple of 8 (at most 1024)");
    if ((q == nullptr) != (q8 == nullptr)) return fail("telb_kv_fp8_store: pass the query rows together with their E4M3 destination");
    const dim3 grid(tokens), blk(256);
    if (is_bf16)
        TELB_LAUNCH("kv_fp8_store_kernel", (kv_fp8_store_kernel<__nv_bfloat16>), grid, blk, 0, stream, (uint8_t*)pool, (__nv_bfloat16*)stage,
                    seq_ids, q_start, past_len, page_table, kv_offsets, scales, max_pages, page_size, hkv, d, (const __nv_bfloat16*)q,
                    (uint8_t*)q8, hq);
    else
        TELB_LAUNCH("kv_fp8_store_kernel", (kv_fp8_store_kernel<__half>), grid, blk, 0, stream, (uint8_t*)pool, (__half*)stage, seq_ids,
                    q_start, past_len, page_table, kv_offsets, scales, max_pages, page_size, hkv, d, (const __half*)q, (uint8_t*)q8, hq);
    return 0;
}
