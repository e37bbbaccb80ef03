// Bandwidth-bound operators around the GEMMs: RMSNorm (+residual add, +gated group form),
// SwiGLU / ReLU², embedding gather, RoPE + q/k-norm + paged KV write, arg-max.  All are plain
// SIMT kernels with 128-bit global accesses; launch grids scale with rows so decode-size calls
// are a single wave.
//
// Reference counterparts: CuTe-DSL rmsnorm (kernelSrcs/rmsnorm_cutedsl/rmsnorm.py),
// cpp/kernels/posEncoding/applyRopeWriteKV.cu, cpp/kernels/embeddingKernels/embeddingKernels.cu,
// cpp/kernels/common/argmaxKernel.cu, cpp/kernels/moe/moeActivationKernels.cu.
#include <cuda_fp8.h>

#include "host_utils.h"
#include "tc5_common.cuh"

namespace telb {

template <typename T> struct Vec8 {
    uint4 u;
    __device__ __forceinline__ void load(const T* p) { u = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void store(T* p) const { *reinterpret_cast<uint4*>(p) = u; }
    __device__ __forceinline__ float get(int i) const { return Cvt<T>::to_f(reinterpret_cast<const T*>(&u)[i]); }
    __device__ __forceinline__ void set(int i, float v) { reinterpret_cast<T*>(&u)[i] = Cvt<T>::from_f(v); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    if (l == 0) red[w] = v;
    __syncthreads();
    float t = l < nw ? red[l] : 0.f;
    t = warp_sum(t);
    __syncthreads();
    return t;
}

// y = rmsnorm(x [+ residual]) * w ; optionally writes the summed residual stream.
// One CTA per row; each thread owns up to kMaxVec 8-element vectors kept in registers.
template <typename T, int kMaxVec>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ residual, const T* __restrict__ w,
                               T* __restrict__ y, T* __restrict__ res_out, int hidden, float eps) {
    pdl_prologue();
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const int nvec = hidden / 8;
    Vec8<T> v[kMaxVec];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx < nvec) {
            v[i].load(x + row * hidden + idx * 8);
            if (residual) {
                Vec8<T> r;
                r.load(residual + row * hidden + idx * 8);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i].set(j, v[i].get(j) + r.get(j));
                if (res_out) v[i].store(res_out + row * hidden + idx * 8);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float f = v[i].get(j);
                ss += f * f;
            }
        }
    }
    const float tot = block_sum(ss, red);
    const float inv = rsqrtf(tot / hidden + eps);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx < nvec) {
            Vec8<T> wv, o;
            wv.load(w + idx * 8);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float n = Cvt<T>::to_f(Cvt<T>::from_f(v[i].get(j) * inv));   // cast before the weight multiply
                o.set(j, n * wv.get(j));
            }
            o.store(y + row * hidden + idx * 8);
        }
    }
}

// LayerNorm: y = (x - mean) / sqrt(var + eps) * w (+ b).  One CTA per row, two passes over registers.
template <typename T, int kMaxVec>
__global__ void layernorm_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b, T* __restrict__ y,
                                 int hidden, float eps) {
    pdl_prologue();
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const int nvec = hidden / 8;
    Vec8<T> v[kMaxVec];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx < nvec) {
            v[i].load(x + row * hidden + idx * 8);
#pragma unroll
            for (int j = 0; j < 8; ++j) sum += v[i].get(j);
        }
    }
    const float mean = block_sum(sum, red) / hidden;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx < nvec) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float d = v[i].get(j) - mean;
                ss += d * d;
            }
        }
    }
    const float inv = rsqrtf(block_sum(ss, red) / hidden + eps);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx < nvec) {
            Vec8<T> wv, bv, o;
            wv.load(w + idx * 8);
            if (b) bv.load(b + idx * 8);
#pragma unroll
            for (int j = 0; j < 8; ++j) o.set(j, (v[i].get(j) - mean) * inv * wv.get(j) + (b ? bv.get(j) : 0.f));
            o.store(y + row * hidden + idx * 8);
        }
    }
}

// Mamba2 output norm: g = x * silu(z); RMS-normalise each group of `gsize` features; scale.
// One CTA per (row, group).
template <typename T>
__global__ void gated_group_rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ z, const T* __restrict__ w,
                                           T* __restrict__ y, int hidden, int gsize, float eps) {
    pdl_prologue();
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const int g = blockIdx.y;
    const T* xp = x + row * hidden + g * gsize;
    const T* zp = z + row * hidden + g * gsize;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gsize; i += blockDim.x) {
        const float zz = Cvt<T>::to_f(zp[i]);
        const float gv = Cvt<T>::to_f(xp[i]) * (zz / (1.f + __expf(-zz)));
        ss += gv * gv;
    }
    const float inv = rsqrtf(block_sum(ss, red) / gsize + eps);
    for (int i = threadIdx.x; i < gsize; i += blockDim.x) {
        const float zz = Cvt<T>::to_f(zp[i]);
        const float gv = Cvt<T>::to_f(xp[i]) * (zz / (1.f + __expf(-zz)));
        const float n = Cvt<T>::to_f(Cvt<T>::from_f(gv * inv));
        y[row * hidden + g * gsize + i] = Cvt<T>::from_f(n * Cvt<T>::to_f(w[g * gsize + i]));
    }
}

// out[t, i] = silu(in[t, i]) * in[t, inter + i]
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ in, T* __restrict__ out, long long rows, int inter) {
    pdl_prologue();
    const long long nvec = rows * (inter / 8);
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < nvec;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long r = idx / (inter / 8);
        const int c = (int)(idx % (inter / 8)) * 8;
        Vec8<T> g, u, o;
        g.load(in + r * 2 * inter + c);
        u.load(in + r * 2 * inter + inter + c);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float gf = g.get(j);
            o.set(j, gf / (1.f + __expf(-gf)) * u.get(j));
        }
        o.store(out + r * inter + c);
    }
}

// out[t, i] = gelu(in[t, i]) * in[t, inter + i]   (tanh form or exact erf form)
template <typename T>
__global__ void geglu_kernel(const T* __restrict__ in, T* __restrict__ out, long long rows, int inter, int tanh_approx) {
    pdl_prologue();
    const long long nvec = rows * (inter / 8);
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < nvec;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long r = idx / (inter / 8);
        const int c = (int)(idx % (inter / 8)) * 8;
        Vec8<T> g, u, o;
        g.load(in + r * 2 * inter + c);
        u.load(in + r * 2 * inter + inter + c);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float x = g.get(j);
            const float act = tanh_approx ? 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)))
                                          : 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
            o.set(j, act * u.get(j));
        }
        o.store(out + r * inter + c);
    }
}

template <typename T>
__global__ void relu2_kernel(const T* __restrict__ in, T* __restrict__ out, long long n) {
    pdl_prologue();
    for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 8; i < n;
         i += (long long)gridDim.x * blockDim.x * 8) {
        Vec8<T> v, o;
        v.load(in + i);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float f = fmaxf(v.get(j), 0.f);
            o.set(j, f * f);
        }
        o.store(out + i);
    }
}

// GELU, exact (erf) or tanh approximation, elementwise over n values (n % 8 == 0).
template <typename T>
__global__ void gelu_kernel(const T* __restrict__ in, T* __restrict__ out, long long n, int tanh_approx) {
    pdl_prologue();
    for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 8; i < n;
         i += (long long)gridDim.x * blockDim.x * 8) {
        Vec8<T> v, o;
        v.load(in + i);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float x = v.get(j);
            const float y = tanh_approx ? 0.5f * x * (1.f + tanhf(0.7978845608f * (x + 0.044715f * x * x * x)))
                                        : 0.5f * x * (1.f + erff(x * 0.70710678f));
            o.set(j, y);
        }
        o.store(out + i);
    }
}

template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table, T* __restrict__ out,
                                 int hidden, int vocab) {
    pdl_prologue();
    const size_t row = blockIdx.x;
    int id = ids[row];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * hidden);
    uint4* dst = reinterpret_cast<uint4*>(out + row * hidden);
    for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
}

// Embedding rows stored in FP8 (E4M3 bytes with one fp32 scale per row) or NVFP4 (two E2M1 codes per byte, low nibble first, one
// E4M3 scale per 16 values, one fp32 scale for the table) and expanded while they are gathered.  One CTA per looked-up row.
// FMT 0: FP8, FMT 1: NVFP4.  `scale` is fp32 [vocab] (FP8) or E4M3 bytes [vocab, hidden / 16] (NVFP4).
template <typename T, int FMT>
__global__ void embedding_quant_kernel(const int* __restrict__ ids, const uint8_t* __restrict__ data, const void* __restrict__ scale,
                                       const float* __restrict__ global_scale, T* __restrict__ out, int hidden, int vocab) {
    pdl_prologue();
    const size_t row = blockIdx.x;
    int id = ids[row];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    T* dst = out + row * hidden;
    if constexpr (FMT == 0) {
        const float s = reinterpret_cast<const float*>(scale)[id];
        const uint8_t* src = data + (size_t)id * hidden;
        for (int i = threadIdx.x * 2; i < hidden; i += blockDim.x * 2) {
            const float a = __half2float(__half(__nv_cvt_fp8_to_halfraw(src[i], __NV_E4M3))) * s;
            const float b = __half2float(__half(__nv_cvt_fp8_to_halfraw(src[i + 1], __NV_E4M3))) * s;
            *reinterpret_cast<uint32_t*>(dst + i) = Cvt<T>::pack2(a, b);
        }
    } else {
        const float gs = *global_scale;
        const uint8_t* src = data + (size_t)id * (hidden / 2);
        const uint8_t* sf = reinterpret_cast<const uint8_t*>(scale) + (size_t)id * (hidden / 16);
        for (int i = threadIdx.x; i < hidden / 2; i += blockDim.x) {
            const uint8_t byte = src[i];
            const float bs = __half2float(__half(__nv_cvt_fp8_to_halfraw(sf[i >> 3], __NV_E4M3))) * gs;
            float v[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int code = (byte >> (4 * h)) & 0xF;
                const int m = code & 7;
                const float mag = m < 2 ? 0.5f * m : (m < 4 ? 0.5f * m : (m == 4 ? 2.f : (m == 5 ? 3.f : (m == 6 ? 4.f : 6.f))));
                v[h] = (code & 8) ? -mag : mag;
            }
            *reinterpret_cast<uint32_t*>(dst + 2 * i) = Cvt<T>::pack2(v[0] * bs, v[1] * bs);
        }
    }
}

// RoPE table: out[p, i] = att * cos(p * inv[i]), out[p, half + i] = att * sin(p * inv[i]); angles in double (positions reach
// 10^5 and more, where an fp32 product has lost the fraction).  One thread per (position, pair).
__global__ void rope_table_kernel(const double* __restrict__ inv, float att, float* __restrict__ out, int max_pos, int half) {
    pdl_prologue();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)max_pos * half) return;
    const int p = (int)(idx / half), i = (int)(idx - (long long)p * half);
    double s, c;
    sincos((double)p * inv[i], &s, &c);
    out[(size_t)p * 2 * half + i] = (float)(c * att);
    out[(size_t)p * 2 * half + half + i] = (float)(s * att);
}

// Multimodal RoPE rows: pair i of row t looks its angle up at the temporal, height or width position of the row, according to
// the section the pair belongs to (sec0 pairs temporal, then sec1 height, the rest width).  cos_sin [P, 2 half], pos3 [3, T].
__global__ void mrope_rows_kernel(const float* __restrict__ cos_sin, const int* __restrict__ pos3, float* __restrict__ out, int tokens,
                                  int half, int table_rows, int sec0, int sec1) {
    pdl_prologue();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)tokens * half) return;
    const int t = (int)(idx / half), i = (int)(idx - (long long)t * half);
    const int comp = i < sec0 ? 0 : (i < sec0 + sec1 ? 1 : 2);
    int p = pos3[(size_t)comp * tokens + t];
    p = min(max(p, 0), table_rows - 1);
    out[(size_t)t * 2 * half + i] = cos_sin[(size_t)p * 2 * half + i];
    out[(size_t)t * 2 * half + half + i] = cos_sin[(size_t)p * 2 * half + half + i];
}

// RoPE + optional per-head RMSNorm on q and k + paged KV write.
// One warp per (token, head); lane l owns E = D/64 consecutive features of each half of the head
// (rotate-half pairs are (i, i + D/2)), so every access is a contiguous E*2-byte vector and the
// head-wide sum of squares is a warp shuffle.  Requires rot_dim == D (full rotary) and D in
// {64, 128, 256}; other shapes use the generic kernel below.
// qkv is token-major packed [T, (Hq + 2 Hkv) * D]; q_out is [T, Hq, D]; cache layer [pages, 2, Hkv, P, D].
template <typename T, int E>
__global__ void rope_kv_write_warp_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ kv_layer,
                                          const float* __restrict__ cos_sin, const int* __restrict__ positions,
                                          const int* __restrict__ seq_ids, const int* __restrict__ q_start,
                                          const int* __restrict__ past_len, const int* __restrict__ page_table,
                                          const int* __restrict__ kv_offsets, const T* __restrict__ q_norm_w,
                                          const T* __restrict__ k_norm_w, int tokens, int hq, int hkv, int page_size,
                                          int max_pages, float eps) {
    pdl_prologue();
    constexpr int D = E * 64;
    constexpr int half = D / 2;
    const int heads = hq + 2 * hkv;
    const long long wid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)tokens * heads) return;
    const int t = (int)(wid / heads);
    const int h = (int)(wid - (long long)t * heads);
    const T* src = qkv + ((size_t)t * heads + h) * D;
    float a[E], b[E];
    {
        T va[E], vb[E];
        if constexpr (E == 2) {
            *reinterpret_cast<uint32_t*>(va) = *reinterpret_cast<const uint32_t*>(src + lane * E);
            *reinterpret_cast<uint32_t*>(vb) = *reinterpret_cast<const uint32_t*>(src + half + lane * E);
        } else if constexpr (E == 4) {
            *reinterpret_cast<uint2*>(va) = *reinterpret_cast<const uint2*>(src + lane * E);
            *reinterpret_cast<uint2*>(vb) = *reinterpret_cast<const uint2*>(src + half + lane * E);
        } else {
            va[0] = src[lane];
            vb[0] = src[half + lane];
        }
#pragma unroll
        for (int i = 0; i < E; ++i) {
            a[i] = Cvt<T>::to_f(va[i]);
            b[i] = Cvt<T>::to_f(vb[i]);
        }
    }
    const bool is_q = h < hq;
    const bool is_k = !is_q && h < hq + hkv;
    const T* nw = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
    if (nw) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < E; ++i) ss += a[i] * a[i] + b[i] * b[i];
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / D + eps);
#pragma unroll
        for (int i = 0; i < E; ++i) {
            a[i] = Cvt<T>::to_f(Cvt<T>::from_f(Cvt<T>::to_f(Cvt<T>::from_f(a[i] * inv)) * Cvt<T>::to_f(nw[lane * E + i])));
            b[i] = Cvt<T>::to_f(Cvt<T>::from_f(Cvt<T>::to_f(Cvt<T>::from_f(b[i] * inv)) * Cvt<T>::to_f(nw[half + lane * E + i])));
        }
    }
    if (is_q || is_k) {
        const float* cs = cos_sin + (size_t)positions[t] * D;
#pragma unroll
        for (int i = 0; i < E; ++i) {
            const float c = cs[lane * E + i], sn = cs[half + lane * E + i];
            const float ra = a[i] * c - b[i] * sn;
            const float rb = b[i] * c + a[i] * sn;
            a[i] = ra;
            b[i] = rb;
        }
    }
    T* dst;
    if (is_q) {
        dst = q_out + ((size_t)t * hq + h) * D;
    } else {
        const int s = seq_ids[t];
        const int off = kv_offsets ? kv_offsets[t] : (t - q_start[s]);
        const int slot = past_len[s] + off;
        const int page = page_table[(size_t)s * max_pages + slot / page_size];
        if (page < 0) return;      // unreserved page: skip instead of writing out of bounds
        const int kvh = is_k ? h - hq : h - hq - hkv;
        dst = kv_layer + ((((size_t)page * 2 + (is_k ? 0 : 1)) * hkv + kvh) * page_size + slot % page_size) * D;
    }
    T oa[E], ob[E];
#pragma unroll
    for (int i = 0; i < E; ++i) {
        oa[i] = Cvt<T>::from_f(a[i]);
        ob[i] = Cvt<T>::from_f(b[i]);
    }
    if constexpr (E == 2) {
        *reinterpret_cast<uint32_t*>(dst + lane * E) = *reinterpret_cast<uint32_t*>(oa);
        *reinterpret_cast<uint32_t*>(dst + half + lane * E) = *reinterpret_cast<uint32_t*>(ob);
    } else if constexpr (E == 4) {
        *reinterpret_cast<uint2*>(dst + lane * E) = *reinterpret_cast<uint2*>(oa);
        *reinterpret_cast<uint2*>(dst + half + lane * E) = *reinterpret_cast<uint2*>(ob);
    } else {
        dst[lane] = oa[0];
        dst[half + lane] = ob[0];
    }
}

// Prefill form for head_dim 128: one warp per token walks all heads two at a time (half a warp per head, 8-byte
// accesses), so the token's cos / sin row, its norm weights and its page look-up are fetched once instead of once per head.
template <typename T>
__global__ void rope_kv_write_token_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ kv_layer,
                                           const float* __restrict__ cos_sin, const int* __restrict__ positions,
                                           const int* __restrict__ seq_ids, const int* __restrict__ q_start,
                                           const int* __restrict__ past_len, const int* __restrict__ page_table,
                                           const int* __restrict__ kv_offsets, const T* __restrict__ q_norm_w,
                                           const T* __restrict__ k_norm_w, int tokens, int hq, int hkv, int page_size,
                                           int max_pages, float eps) {
    pdl_prologue();
    constexpr int D = 128, half = 64;
    const int t = (int)((blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5);
    if (t >= tokens) return;
    const int lane = threadIdx.x & 31;
    const int sub = lane >> 4, li = lane & 15;           // which head of the pair, and this lane's 4 features li*4 .. li*4+3
    const int heads = hq + 2 * hkv;
    const float* cs = cos_sin + (size_t)positions[t] * D;
    const float4 c4 = *reinterpret_cast<const float4*>(cs + li * 4);
    const float4 s4 = *reinterpret_cast<const float4*>(cs + half + li * 4);
    const float c[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
    float qwa[4], qwb[4], kwa[4], kwb[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        qwa[i] = q_norm_w ? Cvt<T>::to_f(q_norm_w[li * 4 + i]) : 1.f;
        qwb[i] = q_norm_w ? Cvt<T>::to_f(q_norm_w[half + li * 4 + i]) : 1.f;
        kwa[i] = k_norm_w ? Cvt<T>::to_f(k_norm_w[li * 4 + i]) : 1.f;
        kwb[i] = k_norm_w ? Cvt<T>::to_f(k_norm_w[half + li * 4 + i]) : 1.f;
    }
    const int s = seq_ids[t];
    const int off = kv_offsets ? kv_offsets[t] : (t - q_start[s]);
    const int slot = past_len[s] + off;
    const int page = page_table[(size_t)s * max_pages + slot / page_size];
    const T* row = qkv + (size_t)t * heads * D;
#pragma unroll 4
    for (int h0 = 0; h0 < heads; h0 += 2) {
        const int h = h0 + sub;
        const bool live = h < heads;
        const bool is_q = h < hq;
        const bool is_k = !is_q && h < hq + hkv;
        float a[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
        if (live) {
            const uint2 ua = *reinterpret_cast<const uint2*>(row + (size_t)h * D + li * 4);
            const uint2 ub = *reinterpret_cast<const uint2*>(row + (size_t)h * D + half + li * 4);
            const T* ea = reinterpret_cast<const T*>(&ua);
            const T* eb = reinterpret_cast<const T*>(&ub);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a[i] = Cvt<T>::to_f(ea[i]);
                b[i] = Cvt<T>::to_f(eb[i]);
            }
        }
        const bool normed = (is_q && q_norm_w) || (is_k && k_norm_w);
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) ss += a[i] * a[i] + b[i] * b[i];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);      // stays inside the half warp
        if (normed) {
            const float inv = rsqrtf(ss / D + eps);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a[i] = Cvt<T>::to_f(Cvt<T>::from_f(Cvt<T>::to_f(Cvt<T>::from_f(a[i] * inv)) * (is_q ? qwa[i] : kwa[i])));
                b[i] = Cvt<T>::to_f(Cvt<T>::from_f(Cvt<T>::to_f(Cvt<T>::from_f(b[i] * inv)) * (is_q ? qwb[i] : kwb[i])));
            }
        }
        if (is_q || is_k) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float ra = a[i] * c[i] - b[i] * sn[i];
                const float rb = b[i] * c[i] + a[i] * sn[i];
                a[i] = ra;
                b[i] = rb;
            }
        }
        if (!live) continue;
        T* dst;
        if (is_q) {
            dst = q_out + ((size_t)t * hq + h) * D;
        } else {
            if (page < 0) continue;                    // unreserved page: skip instead of writing out of bounds
            const int kvh = is_k ? h - hq : h - hq - hkv;
            dst = kv_layer + ((((size_t)page * 2 + (is_k ? 0 : 1)) * hkv + kvh) * page_size + slot % page_size) * D;
        }
        T oa[4], ob[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            oa[i] = Cvt<T>::from_f(a[i]);
            ob[i] = Cvt<T>::from_f(b[i]);
        }
        *reinterpret_cast<uint2*>(dst + li * 4) = *reinterpret_cast<uint2*>(oa);
        *reinterpret_cast<uint2*>(dst + half + li * 4) = *reinterpret_cast<uint2*>(ob);
    }
}

// Generic form (any even head_dim <= 512, partial rotary): grid (T, Hq + 2*Hkv), block D/2 threads,
// thread i owns features i and i + D/2.
template <typename T>
__global__ void rope_kv_write_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ kv_layer,
                                     const float* __restrict__ cos_sin, const int* __restrict__ positions,
                                     const int* __restrict__ seq_ids, const int* __restrict__ q_start,
                                     const int* __restrict__ past_len, const int* __restrict__ page_table,
                                     const int* __restrict__ kv_offsets, const T* __restrict__ q_norm_w,
                                     const T* __restrict__ k_norm_w, int hq, int hkv, int d, int rot_dim, int page_size,
                                     int max_pages, float eps) {
    pdl_prologue();
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int h = blockIdx.y;
    const int half = d / 2;
    const int i = threadIdx.x;
    const T* src = qkv + (size_t)t * (hq + 2 * hkv) * d + (size_t)h * d;
    float a = Cvt<T>::to_f(src[i]);
    float b = Cvt<T>::to_f(src[i + half]);
    const bool is_q = h < hq;
    const bool is_k = !is_q && h < hq + hkv;
    const T* nw = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
    if (nw) {
        const float tot = block_sum(a * a + b * b, red);
        const float inv = rsqrtf(tot / d + eps);
        a = Cvt<T>::to_f(Cvt<T>::from_f(a * inv)) * Cvt<T>::to_f(nw[i]);
        b = Cvt<T>::to_f(Cvt<T>::from_f(b * inv)) * Cvt<T>::to_f(nw[i + half]);
        a = Cvt<T>::to_f(Cvt<T>::from_f(a));
        b = Cvt<T>::to_f(Cvt<T>::from_f(b));
    }
    if (is_q || is_k) {
        const int rh = rot_dim / 2;
        const int pos = positions[t];
        // rotate-half pairs are (j, j + rot_dim/2) for j < rot_dim/2; with rot_dim == d that is (i, i+half)
        if (rot_dim == d) {
            const float c = cos_sin[(size_t)pos * rot_dim + i];
            const float s = cos_sin[(size_t)pos * rot_dim + rh + i];
            const float ra = a * c - b * s;
            const float rb = b * c + a * s;
            a = ra;
            b = rb;
        } else {
            // partial rotary: stage the head in shared memory and rotate the leading rot_dim features
            __shared__ float stage[512];
            stage[i] = a;
            stage[i + half] = b;
            __syncthreads();
            for (int j = i; j < rh; j += blockDim.x) {
                const float c = cos_sin[(size_t)pos * rot_dim + j];
                const float s = cos_sin[(size_t)pos * rot_dim + rh + j];
                const float x1 = stage[j], x2 = stage[j + rh];
                stage[j] = x1 * c - x2 * s;
                stage[j + rh] = x2 * c + x1 * s;
            }
            __syncthreads();
            a = stage[i];
            b = stage[i + half];
        }
    }
    if (is_q) {
        T* dst = q_out + ((size_t)t * hq + h) * d;
        dst[i] = Cvt<T>::from_f(a);
        dst[i + half] = Cvt<T>::from_f(b);
    } else {
        const int s = seq_ids[t];
        const int off = kv_offsets ? kv_offsets[t] : (t - q_start[s]);
        const int slot = past_len[s] + off;
        const int page = page_table[(size_t)s * max_pages + slot / page_size];
        if (page < 0) return;      // unreserved page: skip instead of writing out of bounds
        const int kvh = is_k ? h - hq : h - hq - hkv;
        T* dst = kv_layer + ((((size_t)page * 2 + (is_k ? 0 : 1)) * hkv + kvh) * page_size + slot % page_size) * d;
        dst[i] = Cvt<T>::from_f(a);
        dst[i + half] = Cvt<T>::from_f(b);
    }
}

// arg-max over the vocabulary, one CTA per row (ties → lowest index).
template <typename T>
__global__ void argmax_kernel(const T* __restrict__ logits, int* __restrict__ out, int vocab, long long stride) {
    pdl_prologue();
    __shared__ float sv[32];
    __shared__ int si[32];
    const T* p = logits + blockIdx.x * stride;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = Cvt<T>::to_f(p[i]);
        if (v > best || (v == best && i < bi)) {
            best = v;
            bi = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) {
            best = ov;
            bi = oi;
        }
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) {
        sv[w] = best;
        si[w] = bi;
    }
    __syncthreads();
    if (w == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        best = l < nw ? sv[l] : -INFINITY;
        bi = l < nw ? si[l] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) {
                best = ov;
                bi = oi;
            }
        }
        if (l == 0) out[blockIdx.x] = bi;
    }
}

}  // namespace telb

using namespace telb;

#define DISPATCH_T(is_bf16, ...)                 \
    if (is_bf16) {                               \
        using T = __nv_bfloat16;                 \
        __VA_ARGS__                              \
    } else {                                     \
        using T = __half;                        \
        __VA_ARGS__                              \
    }

extern "C" int telb_rmsnorm(const void* x, const void* residual, const void* w, void* y, void* res_out, long long rows,
                            int hidden, float eps, int is_bf16, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden % 8) return fail("telb_rmsnorm: hidden must be a multiple of 8");
    const int nvec = hidden / 8;
    int threads = nvec >= 512 ? 512 : ((nvec + 31) / 32) * 32;
    if (threads < 32) threads = 32;
    const int per = (nvec + threads - 1) / threads;
    if (per > 8) return fail("telb_rmsnorm: hidden too large (max 32768)");
    DISPATCH_T(is_bf16, {
        if (per <= 1) TELB_LAUNCH("rmsnorm_kernel", (rmsnorm_kernel<T, 1>), dim3(rows), dim3(threads), 0, stream, (const T*)x, (const T*)residual, (const T*)w, (T*)y, (T*)res_out, hidden, eps);
        else if (per <= 2) TELB_LAUNCH("rmsnorm_kernel", (rmsnorm_kernel<T, 2>), dim3(rows), dim3(threads), 0, stream, (const T*)x, (const T*)residual, (const T*)w, (T*)y, (T*)res_out, hidden, eps);
        else if (per <= 4) TELB_LAUNCH("rmsnorm_kernel", (rmsnorm_kernel<T, 4>), dim3(rows), dim3(threads), 0, stream, (const T*)x, (const T*)residual, (const T*)w, (T*)y, (T*)res_out, hidden, eps);
        else TELB_LAUNCH("rmsnorm_kernel", (rmsnorm_kernel<T, 8>), dim3(rows), dim3(threads), 0, stream, (const T*)x, (const T*)residual, (const T*)w, (T*)y, (T*)res_out, hidden, eps);
    })
    TELB_CHECK_LAUNCH("rmsnorm_kernel");
    return 0;
}

extern "C" int telb_layernorm(const void* x, const void* w, const void* b, void* y, long long rows, int hidden, float eps,
                              int is_bf16, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden % 8) return fail("telb_layernorm: hidden must be a multiple of 8");
    const int nvec = hidden / 8;
    int threads = nvec >= 512 ? 512 : ((nvec + 31) / 32) * 32;
    if (threads < 32) threads = 32;
    const int per = (nvec + threads - 1) / threads;
    if (per > 8) return fail("telb_layernorm: hidden too large (max 32768)");
    DISPATCH_T(is_bf16, {
        if (per <= 1) TELB_LAUNCH("layernorm_kernel", (layernorm_kernel<T, 1>), dim3(rows), dim3(threads), 0, stream, (const T*)x, (const T*)w, (const T*)b, (T*)y, hidden, eps);
        else if (per <= 2) TELB_LAUNCH("layernorm_kernel", (layernorm_kernel<T, 2>), dim3(rows), dim3(threads), 0, stream, (const T*)x, (const T*)w, (const T*)b, (T*)y, hidden, eps);
        else if (per <= 4) TELB_LAUNCH("layernorm_kernel", (layernorm_kernel<T, 4>), dim3(rows), dim3(threads), 0, stream, (const T*)x, (const T*)w, (const T*)b, (T*)y, hidden, eps);
        else TELB_LAUNCH("layernorm_kernel", (layernorm_kernel<T, 8>), dim3(rows), dim3(threads), 0, stream, (const T*)x, (const T*)w, (const T*)b, (T*)y, hidden, eps);
    })
    TELB_CHECK_LAUNCH("layernorm_kernel");
    return 0;
}

extern "C" int telb_gated_group_rmsnorm(const void* x, const void* z, const void* w, void* y, long long rows, int hidden,
                                        int n_groups, float eps, int is_bf16, cudaStream_t stream) {
    if (rows <= 0) return 0;
    dim3 grid((unsigned)rows, n_groups);
    DISPATCH_T(is_bf16, {
        TELB_LAUNCH("gated_group_rmsnorm_kernel", (gated_group_rmsnorm_kernel<T>), dim3(grid), dim3(256), 0, stream, (const T*)x, (const T*)z, (const T*)w, (T*)y, hidden, hidden / n_groups, eps);
    })
    TELB_CHECK_LAUNCH("gated_group_rmsnorm_kernel");
    return 0;
}

extern "C" int telb_swiglu(const void* in, void* out, long long rows, int inter, int is_bf16, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (inter % 8) return fail("telb_swiglu: intermediate size must be a multiple of 8");
    const long long nvec = rows * (inter / 8);
    long long blocks = (nvec + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    DISPATCH_T(is_bf16, { TELB_LAUNCH("swiglu_kernel", (swiglu_kernel<T>), dim3((int)blocks), dim3(256), 0, stream, (const T*)in, (T*)out, rows, inter); })
    TELB_CHECK_LAUNCH("swiglu_kernel");
    return 0;
}

extern "C" int telb_geglu(const void* in, void* out, long long rows, int inter, int tanh_approx, int is_bf16, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (inter % 8) return fail("telb_geglu: intermediate size must be a multiple of 8");
    const long long nvec = rows * (inter / 8);
    long long blocks = (nvec + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    DISPATCH_T(is_bf16, { TELB_LAUNCH("geglu_kernel", (geglu_kernel<T>), dim3((int)blocks), dim3(256), 0, stream, (const T*)in, (T*)out, rows, inter, tanh_approx); })
    TELB_CHECK_LAUNCH("geglu_kernel");
    return 0;
}

extern "C" int telb_relu2(const void* in, void* out, long long n, int is_bf16, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (n % 8) return fail("telb_relu2: element count must be a multiple of 8");
    long long blocks = (n / 8 + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    DISPATCH_T(is_bf16, { TELB_LAUNCH("relu2_kernel", (relu2_kernel<T>), dim3((int)blocks), dim3(256), 0, stream, (const T*)in, (T*)out, n); })
    TELB_CHECK_LAUNCH("relu2_kernel");
    return 0;
}

extern "C" int telb_gelu(const void* in, void* out, long long n, int tanh_approx, int is_bf16, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (n % 8) return fail("telb_gelu: element count must be a multiple of 8");
    long long blocks = (n / 8 + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    DISPATCH_T(is_bf16, { TELB_LAUNCH("gelu_kernel", (gelu_kernel<T>), dim3((int)blocks), dim3(256), 0, stream, (const T*)in, (T*)out, n, tanh_approx); })
    TELB_CHECK_LAUNCH("gelu_kernel");
    return 0;
}

extern "C" int telb_embedding(const int* ids, const void* table, void* out, long long rows, int hidden, int vocab,
                              int is_bf16, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden % 8) return fail("telb_embedding: hidden must be a multiple of 8");
    DISPATCH_T(is_bf16, { TELB_LAUNCH("embedding_kernel", (embedding_kernel<T>), dim3((unsigned)rows), dim3(128), 0, stream, ids, (const T*)table, (T*)out, hidden, vocab); })
    TELB_CHECK_LAUNCH("embedding_kernel");
    return 0;
}

// fmt 0: data [vocab, hidden] E4M3, scale fp32 [vocab]; fmt 1: data [vocab, hidden / 2] packed E2M1, scale E4M3 [vocab, hidden / 16],
// global_scale fp32 [1].  out [rows, hidden] 16-bit.
extern "C" int telb_embedding_quant(const int* ids, const void* data, const void* scale, const float* global_scale, void* out, long long rows,
                                    int hidden, int vocab, int fmt, int is_bf16, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (fmt != 0 && fmt != 1) return fail("telb_embedding_quant: format 0 (fp8) or 1 (nvfp4)");
    if (hidden % 16) return fail("telb_embedding_quant: hidden must be a multiple of 16");
    if (fmt == 1 && global_scale == nullptr) return fail("telb_embedding_quant: NVFP4 tables carry a global scale");
    if (fmt == 0) {
        DISPATCH_T(is_bf16, { TELB_LAUNCH("embedding_quant_kernel", (embedding_quant_kernel<T, 0>), dim3((unsigned)rows), dim3(128), 0, stream, ids, (const uint8_t*)data, scale, global_scale, (T*)out, hidden, vocab); })
    } else {
        DISPATCH_T(is_bf16, { TELB_LAUNCH("embedding_quant_kernel", (embedding_quant_kernel<T, 1>), dim3((unsigned)rows), dim3(128), 0, stream, ids, (const uint8_t*)data, scale, global_scale, (T*)out, hidden, vocab); })
    }
    TELB_CHECK_LAUNCH("embedding_quant_kernel");
    return 0;
}

extern "C" int telb_rope_table(const double* inv_freq, float attention_factor, float* out, int max_pos, int half, cudaStream_t stream) {
    if (max_pos <= 0 || half <= 0) return 0;
    const long long n = (long long)max_pos * half;
    TELB_LAUNCH("rope_table_kernel", rope_table_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, inv_freq, attention_factor, out, max_pos, half);
    TELB_CHECK_LAUNCH("rope_table_kernel");
    return 0;
}

extern "C" int telb_mrope_rows(const float* cos_sin, const int* pos3, float* out, int tokens, int half, int table_rows, int sec0, int sec1,
                               cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (sec0 < 0 || sec1 < 0 || sec0 + sec1 > half) return fail("telb_mrope_rows: sections must fit the rotary pairs");
    const long long n = (long long)tokens * half;
    TELB_LAUNCH("mrope_rows_kernel", mrope_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, cos_sin, pos3, out, tokens, half, table_rows, sec0, sec1);
    TELB_CHECK_LAUNCH("mrope_rows_kernel");
    return 0;
}

extern "C" int telb_rope_kv_write(const void* qkv, void* q_out, void* kv_layer, const float* cos_sin,
                                  const int* positions, const int* seq_ids, const int* q_start, const int* past_len,
                                  const int* page_table, const int* kv_offsets, const void* q_norm_w,
                                  const void* k_norm_w, int tokens, int hq, int hkv, int d, int rot_dim, int page_size,
                                  int max_pages, float eps, int is_bf16, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (d % 2 || d > 512) return fail("telb_rope_kv_write: head_dim must be even and <= 512");
    if (rot_dim == d && d == 128 && tokens >= 1024) {
        const int blocks = (tokens + 3) / 4;             // 4 warps = 4 tokens per block
        DISPATCH_T(is_bf16, {
            TELB_LAUNCH("rope_kv_write_token_kernel", (rope_kv_write_token_kernel<T>), dim3(blocks), dim3(128), 0, stream, (const T*)qkv, (T*)q_out, (T*)kv_layer, cos_sin, positions, seq_ids, q_start, past_len, page_table, kv_offsets, (const T*)q_norm_w, (const T*)k_norm_w, tokens, hq, hkv, page_size, max_pages, eps);
        })
        TELB_CHECK_LAUNCH("rope_kv_write_token_kernel");
        return 0;
    }
    if (rot_dim == d && (d == 64 || d == 128 || d == 256)) {
        const long long warps = (long long)tokens * (hq + 2 * hkv);
        const int blocks = (int)((warps + 7) / 8);
        DISPATCH_T(is_bf16, {
            if (d == 128) TELB_LAUNCH("rope_kv_write_warp_kernel", (rope_kv_write_warp_kernel<T, 2>), dim3(blocks), dim3(256), 0, stream, (const T*)qkv, (T*)q_out, (T*)kv_layer, cos_sin, positions, seq_ids, q_start, past_len, page_table, kv_offsets, (const T*)q_norm_w, (const T*)k_norm_w, tokens, hq, hkv, page_size, max_pages, eps);
            else if (d == 64) TELB_LAUNCH("rope_kv_write_warp_kernel", (rope_kv_write_warp_kernel<T, 1>), dim3(blocks), dim3(256), 0, stream, (const T*)qkv, (T*)q_out, (T*)kv_layer, cos_sin, positions, seq_ids, q_start, past_len, page_table, kv_offsets, (const T*)q_norm_w, (const T*)k_norm_w, tokens, hq, hkv, page_size, max_pages, eps);
            else TELB_LAUNCH("rope_kv_write_warp_kernel", (rope_kv_write_warp_kernel<T, 4>), dim3(blocks), dim3(256), 0, stream, (const T*)qkv, (T*)q_out, (T*)kv_layer, cos_sin, positions, seq_ids, q_start, past_len, page_table, kv_offsets, (const T*)q_norm_w, (const T*)k_norm_w, tokens, hq, hkv, page_size, max_pages, eps);
        })
        TELB_CHECK_LAUNCH("rope_kv_write_warp_kernel");
        return 0;
    }
    dim3 grid(tokens, hq + 2 * hkv);
    DISPATCH_T(is_bf16, {
        TELB_LAUNCH("rope_kv_write_kernel", (rope_kv_write_kernel<T>), dim3(grid), dim3(d / 2), 0, stream, (const T*)qkv, (T*)q_out, (T*)kv_layer, cos_sin, positions, seq_ids, q_start, past_len, page_table, kv_offsets, (const T*)q_norm_w, (const T*)k_norm_w, hq, hkv, d, rot_dim, page_size, max_pages, eps);
    })
    TELB_CHECK_LAUNCH("rope_kv_write_kernel");
    return 0;
}

namespace telb {
__global__ void argmax_f32_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab, long long stride) {
    pdl_prologue();
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* p = logits + blockIdx.x * stride;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = p[i];
        if (v > best || (v == best && i < bi)) {
            best = v;
            bi = i;
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) {
            best = ov;
            bi = oi;
        }
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) {
        sv[w] = best;
        si[w] = bi;
    }
    __syncthreads();
    if (w == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        best = l < nw ? sv[l] : -INFINITY;
        bi = l < nw ? si[l] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) {
                best = ov;
                bi = oi;
            }
        }
        if (l == 0) out[blockIdx.x] = bi;
    }
}
}  // namespace telb

namespace telb {
// Two-level arg-max for decode-size batches: `nblk` CTAs per row each reduce a slice and publish
// a packed (order-preserving value bits, inverted index) key with atomicMax; the CTA that arrives
// last at the row's counter writes the winning index and re-arms the scratch for the next launch.
template <typename T>
__global__ void argmax_split_kernel(const T* __restrict__ logits, int* __restrict__ out, int vocab, long long stride,
                                    unsigned long long* __restrict__ keys, int* __restrict__ counters) {
    pdl_prologue();
    __shared__ unsigned long long sk[32];
    const int row = blockIdx.y;
    const int nblk = gridDim.x;
    const int per = (vocab + nblk - 1) / nblk;
    const int lo = blockIdx.x * per, hi = min(vocab, lo + per);
    const T* p = logits + row * stride;
    unsigned long long best = 0ull;
    auto consider = [&](float v, int i) {
        uint32_t u = __float_as_uint(v);
        u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
        const unsigned long long key = ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)i);
        best = key > best ? key : best;
    };
    if constexpr (sizeof(T) == 2) {
        // 16-byte loads over the aligned middle of the segment (8 values each); the ragged ends go one value at a time
        const bool vec_ok = (reinterpret_cast<uintptr_t>(p) & 15) == 0;
        const int a0 = vec_ok ? min(hi, (lo + 7) & ~7) : hi;
        const int a1 = vec_ok ? max(a0, hi & ~7) : hi;
        for (int i = lo + threadIdx.x; i < a0; i += blockDim.x) consider(Cvt<T>::to_f(p[i]), i);
        for (int c = a0 / 8 + threadIdx.x; c < a1 / 8; c += blockDim.x) {
            const uint4 q = __ldg(reinterpret_cast<const uint4*>(p) + c);
            const T* e = reinterpret_cast<const T*>(&q);
            float bv = Cvt<T>::to_f(e[0]);
            int bi = 0;
#pragma unroll
            for (int j = 1; j < 8; ++j) {
                const float v = Cvt<T>::to_f(e[j]);
                if (v > bv) {               // strict: the first of equal values keeps the lower index
                    bv = v;
                    bi = j;
                }
            }
            bool has_nan = false;
#pragma unroll
            for (int j = 0; j < 8; ++j) has_nan = has_nan || !(Cvt<T>::to_f(e[j]) == Cvt<T>::to_f(e[j]));
            if (has_nan) {
#pragma unroll
                for (int j = 0; j < 8; ++j) consider(Cvt<T>::to_f(e[j]), c * 8 + j);      // keys order NaN like the scalar path does
            } else {
                consider(bv, c * 8 + bi);
            }
        }
        for (int i = a1 + threadIdx.x; i < hi; i += blockDim.x) consider(Cvt<T>::to_f(p[i]), i);
    } else {
        for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) consider((float)p[i], i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) sk[w] = best;
    __syncthreads();
    if (w == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        best = l < nw ? sk[l] : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        if (l == 0) {
            atomicMax(&keys[row], best);
            __threadfence();
            const int prev = atomicAdd(&counters[row], 1);
            if (prev == nblk - 1) {
                __threadfence();
                const unsigned long long k = atomicExch(&keys[row], 0ull);
                counters[row] = 0;
                out[row] = (int)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull));
            }
        }
    }
}
}  // namespace telb

// dtype: 0 = fp16, 1 = bf16, 2 = fp32.  `keys` (rows x u64, zeroed once) and `counters` (rows x int,
// zeroed once) are scratch for the split form used when rows are few; pass null to force one CTA per row.
extern "C" int telb_argmax(const void* logits, int* out, long long rows, int vocab, long long stride, int dtype,
                           void* keys, int* counters, int scratch_rows, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (keys && counters && rows <= scratch_rows && rows * 8 <= 4 * 148 && vocab >= 8192) {
        int nblk = (int)((2 * 148 + rows - 1) / rows);
        if (nblk > 64) nblk = 64;
        dim3 grid(nblk, (unsigned)rows);
        unsigned long long* k = (unsigned long long*)keys;
        if (dtype == 2) TELB_LAUNCH("argmax_split_kernel", (argmax_split_kernel<float>), dim3(grid), dim3(512), 0, stream, (const float*)logits, out, vocab, stride, k, counters);
        else if (dtype == 1) TELB_LAUNCH("argmax_split_kernel", (argmax_split_kernel<__nv_bfloat16>), dim3(grid), dim3(512), 0, stream, (const __nv_bfloat16*)logits, out, vocab, stride, k, counters);
        else TELB_LAUNCH("argmax_split_kernel", (argmax_split_kernel<__half>), dim3(grid), dim3(512), 0, stream, (const __half*)logits, out, vocab, stride, k, counters);
        TELB_CHECK_LAUNCH("argmax_split_kernel");
        return 0;
    }
    if (dtype == 2) TELB_LAUNCH("argmax_f32_kernel", (argmax_f32_kernel), dim3((unsigned)rows), dim3(1024), 0, stream, (const float*)logits, out, vocab, stride);
    else if (dtype == 1) TELB_LAUNCH("argmax_kernel", (argmax_kernel<__nv_bfloat16>), dim3((unsigned)rows), dim3(1024), 0, stream, (const __nv_bfloat16*)logits, out, vocab, stride);
    else TELB_LAUNCH("argmax_kernel", (argmax_kernel<__half>), dim3((unsigned)rows), dim3(1024), 0, stream, (const __half*)logits, out, vocab, stride);
    TELB_CHECK_LAUNCH("argmax_kernel");
    return 0;
}
