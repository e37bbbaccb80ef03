// Mixture-of-experts routing and token movement around the grouped expert GEMMs.
//
//   moe_route          softmax over E router logits → top-k (ties → lower index) → optional renormalise
//                      (sigmoid + group-limited top-k for DeepSeek/Nemotron-style routers)
//   moe_align          per-expert counts → 128-row padded segment offsets → destination row of every
//                      (token, k) slot → expert id of every 128-row tile (-1 = unused tile)
//   moe_gather_quant   copy each routed token row to its destination row, quantising to NVFP4 on the way
//                      (or plain 16-bit copy for 16-bit experts)
//   moe_combine        out[t] = Σ_k w[t,k] · y[dst_row[t,k]]
// The expert GEMMs themselves are the persistent tcgen05 kernels (gemm_tc5.cu / gemm_nvfp4_tc5.cu)
// run over the padded row space with a per-tile expert table selecting the weight block, so one
// launch covers every expert and each expert's weights are streamed exactly once.
//
// Reference counterparts: cpp/kernels/moe/moeTopkSoftmaxKernels.cu, moeSigmoidGroupTopkKernels.cu,
// moeAlignSumKernels.cu, fp4SupportKernels/{buildLayout,fp4Quantize}.cu (routed variant) and the
// scatter-reduce epilogue of the CuTe-DSL FC2 kernel (kernelSrcs/nvfp4_moe_cutedsl/).
#include "host_utils.h"
#include "nvfp4_common.cuh"

namespace telb {

constexpr int kMaxTopK = 16;

// One warp per token.  E <= 1024.
template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ logits, float* __restrict__ topk_w, int* __restrict__ topk_idx,
                                 const float* __restrict__ bias, int tokens, int experts, int top_k, int renorm, int sigmoid,
                                 int n_group, int topk_group, float scaling) {
    pdl_prologue();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    const int t = blockIdx.x * wpb + warp;
    if (t >= tokens) return;
    float* score = smem + (size_t)warp * 2 * experts;     // selection score
    float* prob = score + experts;                        // weight source
    const T* row = logits + (size_t)t * experts;
    float mx = -INFINITY;
    for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, Cvt<T>::to_f(row[e]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int e = lane; e < experts; e += 32) {
        const float x = Cvt<T>::to_f(row[e]);
        float p;
        if (sigmoid) p = 1.f / (1.f + __expf(-x));
        else { p = __expf(x - mx); sum += p; }
        prob[e] = p;
    }
    if (!sigmoid) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float inv = 1.f / sum;
        for (int e = lane; e < experts; e += 32) prob[e] *= inv;
    }
    __syncwarp();
    for (int e = lane; e < experts; e += 32) score[e] = prob[e] + (bias ? bias[e] : 0.f);
    __syncwarp();
    if (n_group > 1) {
        // group-limited routing: keep the `topk_group` groups with the largest (top-2 sum) score
        const int gs = experts / n_group;
        float gscore = -INFINITY;
        if (lane < n_group) {
            float a = -INFINITY, b = -INFINITY;
            for (int i = 0; i < gs; ++i) {
                const float v = score[lane * gs + i];
                if (v > a) { b = a; a = v; } else if (v > b) b = v;
            }
            gscore = gs > 1 ? a + b : a;
        }
        unsigned keep = 0;
        for (int r = 0; r < topk_group; ++r) {
            float best = gscore;
            int bi = lane;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
            }
            keep |= 1u << bi;
            if (lane == bi) gscore = -INFINITY;
        }
        for (int e = lane; e < experts; e += 32)
            if (!((keep >> (e / gs)) & 1u)) score[e] = -INFINITY;
        __syncwarp();
    }
    float wsum = 0.f;
    float my_w[kMaxTopK];
    int my_i[kMaxTopK];
    for (int r = 0; r < top_k; ++r) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float v = score[e];
            if (v > best || (v == best && e < bi)) { best = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        const float w = prob[bi];
        my_w[r] = w;
        my_i[r] = bi;
        wsum += w;
        __syncwarp();
        if (lane == 0) score[bi] = -INFINITY;
        __syncwarp();
    }
    if (lane == 0) {
        const float inv = renorm ? 1.f / (wsum + (sigmoid ? 1e-20f : 0.f)) : 1.f;
        for (int r = 0; r < top_k; ++r) {
            topk_w[(size_t)t * top_k + r] = my_w[r] * inv * scaling;
            topk_idx[(size_t)t * top_k + r] = my_i[r];
        }
    }
}

// `tile_expert` has 2 * max_tiles entries: the expert of every 128-row tile (-1 = unused), then the number of rows in use in
// every tile (the grouped GEMM stores, and the activation kernel between the two GEMMs processes, only those rows).
// Single CTA.  counts → padded offsets → dst rows (stable within an expert by slot order is not
// required: the combine reads back through dst_row).  `expert_lo/hi`: experts owned by this rank
// (expert parallelism); slots routed elsewhere get dst_row = -1.
__global__ void moe_align_kernel(const int* __restrict__ topk_idx, int* __restrict__ dst_row, int* __restrict__ tile_expert,
                                 int* __restrict__ counts_out, int slots, int experts, int expert_lo, int expert_hi,
                                 int max_tiles) {
    pdl_prologue();
    extern __shared__ int sm[];
    int* count = sm;                  // [experts]
    int* offset = sm + experts;       // [experts] first tile of the expert's segment
    int* cursor = offset + experts;   // [experts]
    __shared__ int total_tiles;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < slots; i += blockDim.x) {
        const int e = topk_idx[i];
        if (e >= expert_lo && e < expert_hi) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    // exclusive prefix sum of the per-expert tile counts: warp 0 walks the experts 32 at a time
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        int carry = 0;
        for (int e0 = 0; e0 < experts; e0 += 32) {
            const int e = e0 + lane;
            const int tiles = e < experts ? (count[e] + 127) / 128 : 0;
            int incl = tiles;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            if (e < experts) {
                offset[e] = carry + incl - tiles;
                cursor[e] = 0;
            }
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) {
            total_tiles = carry;
            counts_out[0] = carry * 128;      // padded rows in use
        }
    }
    __syncthreads();
    // every expert fills in its own tiles; the tiles past the last segment are marked unused
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        const int tiles = (count[e] + 127) / 128;
        for (int t = 0; t < tiles; ++t) {
            const int tile = offset[e] + t;
            if (tile < max_tiles) {
                tile_expert[tile] = e - expert_lo;
                tile_expert[max_tiles + tile] = min(128, count[e] - t * 128);     // rows in use in this tile
            }
        }
    }
    for (int t = total_tiles + threadIdx.x; t < max_tiles; t += blockDim.x) {
        tile_expert[t] = -1;
        tile_expert[max_tiles + t] = 0;
    }
    for (int i = threadIdx.x; i < slots; i += blockDim.x) {
        const int e = topk_idx[i];
        if (e >= expert_lo && e < expert_hi) dst_row[i] = offset[e] * 128 + atomicAdd(&cursor[e], 1);
        else dst_row[i] = -1;
    }
}

// grid.x = routed slots (token*top_k + k); one CTA copies / quantises one row of `hidden` features.
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ dst_row, T* __restrict__ out16,
                                  uint8_t* __restrict__ xq, uint8_t* __restrict__ sf, const float* __restrict__ global_scale,
                                  int top_k, int hidden, int k64_pad) {
    pdl_prologue();
    const int slot = blockIdx.x;
    const int row = dst_row[slot];
    if (row < 0) return;
    const T* src = x + (size_t)(slot / top_k) * hidden;
    if (out16) {
        for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x)
            reinterpret_cast<uint4*>(out16 + (size_t)row * hidden)[i] = reinterpret_cast<const uint4*>(src)[i];
        return;
    }
    const float gs = *global_scale;
    const float inv_gs = 1.f / gs;
    for (int u = threadIdx.x; u < hidden / 16; u += blockDim.x) {
        const uint4 a0 = reinterpret_cast<const uint4*>(src + u * 16)[0], a1 = reinterpret_cast<const uint4*>(src + u * 16)[1];
        const T* e0 = reinterpret_cast<const T*>(&a0);
        const T* e1 = reinterpret_cast<const T*>(&a1);
        float v[16];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = Cvt<T>::to_f(e0[i]);
            v[8 + i] = Cvt<T>::to_f(e1[i]);
            amax = fmaxf(amax, fmaxf(fabsf(v[i]), fabsf(v[8 + i])));
        }
        uint8_t s8;
        const uint2 packed = nvfp4_quantize_block16(v, amax, gs, inv_gs, s8);
        *reinterpret_cast<uint2*>(xq + (size_t)row * (hidden / 2) + u * 8) = packed;
        sf[sf_atom_offset(row, u, k64_pad)] = s8;
    }
}

// out[t, :] = Σ_k w[t,k] * y[dst_row[t,k], :]   (slots routed to other ranks contribute nothing)
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ dst_row, const float* __restrict__ topk_w,
                                   T* __restrict__ out, int top_k, int hidden) {
    pdl_prologue();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int k = 0; k < top_k; ++k) {
            const int row = dst_row[(size_t)t * top_k + k];
            if (row < 0) continue;
            const float w = topk_w[(size_t)t * top_k + k];
            const uint4 u = reinterpret_cast<const uint4*>(y + (size_t)row * hidden)[i];
            const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += w * Cvt<T>::to_f(e[j]);
        }
        uint4 o;
        o.x = Cvt<T>::pack2(acc[0], acc[1]);
        o.y = Cvt<T>::pack2(acc[2], acc[3]);
        o.z = Cvt<T>::pack2(acc[4], acc[5]);
        o.w = Cvt<T>::pack2(acc[6], acc[7]);
        reinterpret_cast<uint4*>(out + (size_t)t * hidden)[i] = o;
    }
}

}  // namespace telb

using namespace telb;

extern "C" int telb_nvfp4_k64_pad(int k);

extern "C" int telb_moe_route(const void* logits, float* topk_w, int* topk_idx, const float* bias, int tokens, int experts,
                              int top_k, int renorm, int sigmoid, int n_group, int topk_group, float scaling, int dtype,
                              cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (top_k > kMaxTopK || experts > 1024 || n_group > 32) return fail("telb_moe_route: top_k <= 16, experts <= 1024, groups <= 32");
    const int wpb = 4;
    const size_t smem = (size_t)wpb * 2 * experts * sizeof(float);
    const dim3 grid((tokens + wpb - 1) / wpb), block(wpb * 32);
    if (dtype == 2)
        TELB_LAUNCH("moe_route_kernel", (moe_route_kernel<float>), grid, block, smem, stream, (const float*)logits, topk_w, topk_idx, bias,
                    tokens, experts, top_k, renorm, sigmoid, n_group, topk_group, scaling);
    else if (dtype == 1)
        TELB_LAUNCH("moe_route_kernel", (moe_route_kernel<__nv_bfloat16>), grid, block, smem, stream, (const __nv_bfloat16*)logits, topk_w,
                    topk_idx, bias, tokens, experts, top_k, renorm, sigmoid, n_group, topk_group, scaling);
    else
        TELB_LAUNCH("moe_route_kernel", (moe_route_kernel<__half>), grid, block, smem, stream, (const __half*)logits, topk_w, topk_idx, bias,
                    tokens, experts, top_k, renorm, sigmoid, n_group, topk_group, scaling);
    return 0;
}

extern "C" int telb_moe_align(const int* topk_idx, int* dst_row, int* tile_expert, int* counts_out, int slots, int experts,
                              int expert_lo, int expert_hi, int max_tiles, cudaStream_t stream) {
    if (experts > 4096) return fail("telb_moe_align: too many experts");
    TELB_LAUNCH("moe_align_kernel", moe_align_kernel, dim3(1), dim3(1024), (size_t)3 * experts * sizeof(int), stream, topk_idx, dst_row,
                tile_expert, counts_out, slots, experts, expert_lo, expert_hi, max_tiles);
    return 0;
}

// out16 != null → 16-bit copy; else NVFP4 (xq, sf with the atom layout over the padded row space).
extern "C" int telb_moe_gather(const void* x, const int* dst_row, void* out16, void* xq, void* sf, const float* global_scale,
                               int slots, int top_k, int hidden, int is_bf16, cudaStream_t stream) {
    if (slots <= 0) return 0;
    if (hidden % 16) return fail("telb_moe_gather: hidden must be a multiple of 16");
    const int k64 = telb_nvfp4_k64_pad(hidden);
    if (is_bf16)
        TELB_LAUNCH("moe_gather_kernel", (moe_gather_kernel<__nv_bfloat16>), dim3(slots), dim3(128), 0, stream, (const __nv_bfloat16*)x,
                    dst_row, (__nv_bfloat16*)out16, (uint8_t*)xq, (uint8_t*)sf, global_scale, top_k, hidden, k64);
    else
        TELB_LAUNCH("moe_gather_kernel", (moe_gather_kernel<__half>), dim3(slots), dim3(128), 0, stream, (const __half*)x, dst_row,
                    (__half*)out16, (uint8_t*)xq, (uint8_t*)sf, global_scale, top_k, hidden, k64);
    return 0;
}

extern "C" int telb_moe_combine(const void* y, const int* dst_row, const float* topk_w, void* out, int tokens, int top_k,
                                int hidden, int is_bf16, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (hidden % 8) return fail("telb_moe_combine: hidden must be a multiple of 8");
    if (is_bf16)
        TELB_LAUNCH("moe_combine_kernel", (moe_combine_kernel<__nv_bfloat16>), dim3(tokens), dim3(256), 0, stream, (const __nv_bfloat16*)y,
                    dst_row, topk_w, (__nv_bfloat16*)out, top_k, hidden);
    else
        TELB_LAUNCH("moe_combine_kernel", (moe_combine_kernel<__half>), dim3(tokens), dim3(256), 0, stream, (const __half*)y, dst_row, topk_w,
                    (__half*)out, top_k, hidden);
    return 0;
}
