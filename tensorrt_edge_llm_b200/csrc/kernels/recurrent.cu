// Recurrent-layer kernels for hybrid models: depthwise causal conv1d with rolling state, the
// Mamba2 selective-state recurrence and the gated delta rule, all on the packed ragged step ABI
// (prefill chunks and decode rows in one launch; state rows addressed by slot id, never moved).
//
// These are the state-carrying SIMT forms: one CTA per (sequence, head) walks the sequence's rows
// in order with the fp32 state held in registers, so a prefill chunk costs O(tokens) sequential
// steps per head (decode is a single step).  State precision is fp32, activations 16-bit.
//
// Reference counterparts: cpp/kernels/mamba/causalConv1d.cu, cpp/kernels/mamba/selectiveStateUpdate.cu
// (decode / multi-token), the CuTe-DSL SSD and GDN prefill kernels (kernelSrcs/ssd_cutedsl,
// kernelSrcs/gdn_cutedsl) and gdn decode; semantics follow the CPU references in
// unittests/cpp/kernels/mamba/*Tests.cu and unittests/cpp/kernels/gdnKernels/gdnCuteDslTests.cu:157-238.
#include "host_utils.h"
#include "tc5_common.cuh"

namespace telb {

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// ---- causal conv1d ---------------------------------------------------------------------------------
// x [T, C] packed rows; weight [C, W]; conv_state [rows, C, W-1] (oldest first) indexed by slot.
// grid (ceil(C/128), T): thread = one (token, channel) output; history comes from earlier rows of the
// same sequence or from the state.  A second launch (grid.y = num_seqs) rolls the state forward.
template <typename T, int W>
__global__ void conv1d_fwd_kernel(const T* __restrict__ x, const T* __restrict__ weight, const T* __restrict__ bias,
                                  const T* __restrict__ conv_state, T* __restrict__ out, const int* __restrict__ seq_ids,
                                  const int* __restrict__ q_start, const int* __restrict__ past_len, const int* __restrict__ slot_ids,
                                  int channels, int activation) {
    pdl_prologue();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = blockIdx.y;
    if (c >= channels) return;
    const int s = seq_ids[t];
    const int i = t - q_start[s];                   // index of this row inside the sequence's chunk
    const bool has_hist = past_len[s] > 0;
    const T* st = conv_state + ((size_t)slot_ids[s] * channels + c) * (W - 1);
    float acc = bias ? Cvt<T>::to_f(bias[c]) : 0.f;
#pragma unroll
    for (int k = 0; k < W; ++k) {
        const int j = i - (W - 1) + k;              // source row relative to the chunk start
        float v;
        if (j >= 0) v = Cvt<T>::to_f(x[(size_t)(t - i + j) * channels + c]);
        else v = has_hist ? Cvt<T>::to_f(st[(W - 1) + j]) : 0.f;
        acc += v * Cvt<T>::to_f(weight[(size_t)c * W + k]);
    }
    out[(size_t)t * channels + c] = Cvt<T>::from_f(activation ? silu_f(acc) : acc);
}

template <typename T, int W>
__global__ void conv1d_state_kernel(const T* __restrict__ x, T* __restrict__ conv_state, const int* __restrict__ q_start,
                                    const int* __restrict__ q_len, const int* __restrict__ past_len,
                                    const int* __restrict__ slot_ids, int channels) {
    pdl_prologue();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int s = blockIdx.y;
    if (c >= channels) return;
    const int ql = q_len[s];
    if (ql <= 0) return;
    T* st = conv_state + ((size_t)slot_ids[s] * channels + c) * (W - 1);
    T nw[W - 1];
#pragma unroll
    for (int k = 0; k < W - 1; ++k) {
        const int j = ql - (W - 1) + k;             // row relative to the chunk start
        if (j >= 0) nw[k] = x[(size_t)(q_start[s] + j) * channels + c];
        else nw[k] = past_len[s] > 0 ? st[(W - 1) + j] : Cvt<T>::from_f(0.f);
    }
#pragma unroll
    for (int k = 0; k < W - 1; ++k) st[k] = nw[k];
}

// ---- Mamba2 selective state ------------------------------------------------------------------------
// One CTA per (sequence, head), HD threads: thread p owns state row h[p][0..N) in registers.
//   dt = softplus(dt + dt_bias) (clamped), dA = exp(A dt), h = h dA + (dt x[p]) B, y[p] = h·C + D x[p], y *= silu(z)
template <typename T, int HD, int N>
__global__ void __launch_bounds__(HD)
ssm_scan_kernel(const T* __restrict__ x, const T* __restrict__ dt, const float* __restrict__ A, const T* __restrict__ B,
                const T* __restrict__ C, const float* __restrict__ D, const float* __restrict__ dt_bias, const T* __restrict__ z,
                float* __restrict__ state, T* __restrict__ y, const int* __restrict__ q_start, const int* __restrict__ q_len,
                const int* __restrict__ past_len, const int* __restrict__ slot_ids, int nheads, int ngroups, int dt_softplus,
                float dt_limit) {
    pdl_prologue();
    __shared__ float sB[N], sC[N];
    const int s = blockIdx.x, h = blockIdx.y, p = threadIdx.x;
    const int ql = q_len[s];
    if (ql <= 0) return;
    const int g = h / (nheads / ngroups);
    float* st = state + (((size_t)slot_ids[s] * nheads + h) * HD + p) * N;
    float hreg[N];
    if (past_len[s] > 0) {
#pragma unroll
        for (int n = 0; n < N; n += 4) {
            const float4 v = *reinterpret_cast<const float4*>(st + n);
            hreg[n] = v.x; hreg[n + 1] = v.y; hreg[n + 2] = v.z; hreg[n + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int n = 0; n < N; ++n) hreg[n] = 0.f;
    }
    const float a = A[h], dd = D[h], db = dt_bias[h];
    for (int i = 0; i < ql; ++i) {
        const size_t t = (size_t)q_start[s] + i;
        __syncthreads();
        for (int n = p; n < N; n += HD) {
            sB[n] = Cvt<T>::to_f(B[(t * ngroups + g) * N + n]);
            sC[n] = Cvt<T>::to_f(C[(t * ngroups + g) * N + n]);
        }
        __syncthreads();
        float d = Cvt<T>::to_f(dt[t * nheads + h]) + db;
        if (dt_softplus) d = softplus_f(d);
        if (dt_limit > 0.f) d = fminf(d, dt_limit);
        const float dA = __expf(a * d);
        const float xv = Cvt<T>::to_f(x[(t * nheads + h) * HD + p]);
        const float dx = d * xv;
        float acc = 0.f;
#pragma unroll
        for (int n = 0; n < N; ++n) {
            hreg[n] = hreg[n] * dA + dx * sB[n];
            acc += hreg[n] * sC[n];
        }
        acc += dd * xv;
        if (z) acc *= silu_f(Cvt<T>::to_f(z[(t * nheads + h) * HD + p]));
        y[(t * nheads + h) * HD + p] = Cvt<T>::from_f(acc);
    }
#pragma unroll
    for (int n = 0; n < N; n += 4) *reinterpret_cast<float4*>(st + n) = make_float4(hreg[n], hreg[n + 1], hreg[n + 2], hreg[n + 3]);
}

// ---- Mamba2 selective state, segmented for long prefill chunks -----------------------------------
// The recurrence h_t = dA_t h_{t-1} + (dt_t x_t) ⊗ B_t is linear in h, so a long chunk is cut into segments of
// `seg_len` tokens that run in parallel (grid.z):
//   pass 1 (MODE 1): every segment starts from zero, and stores its local end state and the product of its dA;
//   carry         : per (sequence, head), h_init[s+1] = h_init[s] * prod_s + local_s, sequentially over segments
//                   (h_init[0] is the pooled state, or zero for a fresh sequence); the end state goes to the pool;
//   pass 2 (MODE 2): every segment reruns from its true initial state and writes y.
// Twice the arithmetic of the sequential walk, but (segments x heads x sequences) CTAs instead of (heads x sequences).
template <typename T, int HD, int N, int MODE>
__global__ void __launch_bounds__(HD)
ssm_scan_seg_kernel(const T* __restrict__ x, const T* __restrict__ dt, const float* __restrict__ A, const T* __restrict__ B,
                    const T* __restrict__ C, const float* __restrict__ D, const float* __restrict__ dt_bias, const T* __restrict__ z,
                    float* __restrict__ seg_state, float* __restrict__ seg_decay, T* __restrict__ y, const int* __restrict__ q_start,
                    const int* __restrict__ q_len, int nheads, int ngroups, int dt_softplus, float dt_limit, int seg_len,
                    int max_segs) {
    pdl_prologue();
    __shared__ float sB[N], sC[N];
    const int s = blockIdx.x, h = blockIdx.y, seg = blockIdx.z, p = threadIdx.x;
    const int ql = q_len[s];
    const int t0 = seg * seg_len;
    if (t0 >= ql) return;
    const int t1 = min(ql, t0 + seg_len);
    const int g = h / (nheads / ngroups);
    float* st = seg_state + ((((size_t)s * nheads + h) * max_segs + seg) * HD + p) * N;
    float hreg[N];
    if (MODE == 2) {
#pragma unroll
        for (int n = 0; n < N; n += 4) {
            const float4 v = *reinterpret_cast<const float4*>(st + n);
            hreg[n] = v.x; hreg[n + 1] = v.y; hreg[n + 2] = v.z; hreg[n + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int n = 0; n < N; ++n) hreg[n] = 0.f;
    }
    const float a = A[h], dd = D[h], db = dt_bias[h];
    float decay = 1.f;
    for (int i = t0; i < t1; ++i) {
        const size_t t = (size_t)q_start[s] + i;
        __syncthreads();
        for (int n = p; n < N; n += HD) {
            sB[n] = Cvt<T>::to_f(B[(t * ngroups + g) * N + n]);
            if (MODE == 2) sC[n] = Cvt<T>::to_f(C[(t * ngroups + g) * N + n]);
        }
        __syncthreads();
        float d = Cvt<T>::to_f(dt[t * nheads + h]) + db;
        if (dt_softplus) d = softplus_f(d);
        if (dt_limit > 0.f) d = fminf(d, dt_limit);
        const float dA = __expf(a * d);
        decay *= dA;
        const float xv = Cvt<T>::to_f(x[(t * nheads + h) * HD + p]);
        const float dx = d * xv;
        float acc = 0.f;
#pragma unroll
        for (int n = 0; n < N; ++n) {
            hreg[n] = hreg[n] * dA + dx * sB[n];
            if (MODE == 2) acc += hreg[n] * sC[n];
        }
        if (MODE == 2) {
            acc += dd * xv;
            if (z) acc *= silu_f(Cvt<T>::to_f(z[(t * nheads + h) * HD + p]));
            y[(t * nheads + h) * HD + p] = Cvt<T>::from_f(acc);
        }
    }
    if (MODE == 1) {
#pragma unroll
        for (int n = 0; n < N; n += 4) *reinterpret_cast<float4*>(st + n) = make_float4(hreg[n], hreg[n + 1], hreg[n + 2], hreg[n + 3]);
        if (p == 0) seg_decay[((size_t)s * nheads + h) * max_segs + seg] = decay;
    }
}

// grid (sequences, heads), HD * N / 4 elements per ... one thread per 4 state elements; walks the segments in order,
// replacing each local end state by the segment's true initial state.
template <int HD, int N>
__global__ void ssm_carry_kernel(float* __restrict__ seg_state, const float* __restrict__ seg_decay, float* __restrict__ state,
                                 const int* __restrict__ q_len, const int* __restrict__ past_len, const int* __restrict__ slot_ids,
                                 int nheads, int seg_len, int max_segs) {
    pdl_prologue();
    const int s = blockIdx.x, h = blockIdx.y;
    const int ql = q_len[s];
    if (ql <= 0) return;
    const int nseg = (ql + seg_len - 1) / seg_len;
    float4* pool = reinterpret_cast<float4*>(state + ((size_t)slot_ids[s] * nheads + h) * HD * N);
    float4* segs = reinterpret_cast<float4*>(seg_state + (((size_t)s * nheads + h) * max_segs) * HD * N);
    const float* dec = seg_decay + ((size_t)s * nheads + h) * max_segs;
    const bool fresh = past_len[s] <= 0;
    for (int e = threadIdx.x; e < HD * N / 4; e += blockDim.x) {
        float4 cur = fresh ? make_float4(0.f, 0.f, 0.f, 0.f) : pool[e];
        for (int k = 0; k < nseg; ++k) {
            float4* slot = segs + (size_t)k * (HD * N / 4) + e;
            const float4 loc = *slot;
            const float d = dec[k];
            *slot = cur;                                   // the segment's initial state
            cur = make_float4(cur.x * d + loc.x, cur.y * d + loc.y, cur.z * d + loc.z, cur.w * d + loc.w);
        }
        pool[e] = cur;
    }
}

// ---- gated delta rule ------------------------------------------------------------------------------
// One CTA per (sequence, value head), V threads: thread v owns state column H[0..K)[v] in registers.
//   q̂ = q/‖q‖/√K, k̂ = k/‖k‖, g = exp(-exp(A_log) softplus(a + dt_bias)), β = σ(b)
//   H = g H;  Δ = β (v - Hᵀk̂);  H += k̂ ⊗ Δ;  o = Hᵀ q̂
template <typename T, int K, int V>
__global__ void __launch_bounds__(V)
gdn_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ a,
           const T* __restrict__ b, const float* __restrict__ A_log, const float* __restrict__ dt_bias, float* __restrict__ state,
           T* __restrict__ out, const int* __restrict__ q_start, const int* __restrict__ q_len, const int* __restrict__ past_len,
           const int* __restrict__ slot_ids, int hk, int hv) {
    pdl_prologue();
    __shared__ float sq[K], sk[K];
    __shared__ float red[8];
    const int s = blockIdx.x, h = blockIdx.y, tv = threadIdx.x;
    const int ql = q_len[s];
    if (ql <= 0) return;
    const int kh = h / (hv / hk);
    float* st = state + ((size_t)slot_ids[s] * hv + h) * K * V;        // [K][V]
    float H[K];
    if (past_len[s] > 0) {
#pragma unroll
        for (int i = 0; i < K; ++i) H[i] = st[(size_t)i * V + tv];
    } else {
#pragma unroll
        for (int i = 0; i < K; ++i) H[i] = 0.f;
    }
    const float neg_exp_a = -__expf(A_log[h]), db = dt_bias[h];
    for (int i = 0; i < ql; ++i) {
        const size_t t = (size_t)q_start[s] + i;
        __syncthreads();
        float qq = 0.f, kk = 0.f;
        for (int j = tv; j < K; j += V) {
            sq[j] = Cvt<T>::to_f(q[(t * hk + kh) * K + j]);
            sk[j] = Cvt<T>::to_f(k[(t * hk + kh) * K + j]);
            qq += sq[j] * sq[j];
            kk += sk[j] * sk[j];
        }
        // block-wide sums of squares (only the first K threads contributed)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            qq += __shfl_xor_sync(0xffffffffu, qq, o);
            kk += __shfl_xor_sync(0xffffffffu, kk, o);
        }
        if ((tv & 31) == 0) { red[(tv >> 5) * 2] = qq; red[(tv >> 5) * 2 + 1] = kk; }
        __syncthreads();
        float tq = 0.f, tk = 0.f;
#pragma unroll
        for (int w = 0; w < V / 32; ++w) { tq += red[w * 2]; tk += red[w * 2 + 1]; }
        const float qn = rsqrtf(tq + 1e-6f) * rsqrtf((float)K);
        const float kn = rsqrtf(tk + 1e-6f);
        const float gdec = __expf(neg_exp_a * softplus_f(Cvt<T>::to_f(a[t * hv + h]) + db));
        const float beta = 1.f / (1.f + __expf(-Cvt<T>::to_f(b[t * hv + h])));
        float pred = 0.f;
#pragma unroll
        for (int j = 0; j < K; ++j) {
            H[j] *= gdec;
            pred += H[j] * (sk[j] * kn);
        }
        const float delta = beta * (Cvt<T>::to_f(v[(t * hv + h) * V + tv]) - pred);
        float o = 0.f;
#pragma unroll
        for (int j = 0; j < K; ++j) {
            H[j] += (sk[j] * kn) * delta;
            o += H[j] * (sq[j] * qn);
        }
        out[(t * hv + h) * V + tv] = Cvt<T>::from_f(o);
    }
#pragma unroll
    for (int i = 0; i < K; ++i) st[(size_t)i * V + tv] = H[i];
}

}  // namespace telb

using namespace telb;

constexpr int kSsmSegLen = 128;     // tokens per parallel segment of a long Mamba2 prefill chunk

extern "C" int telb_causal_conv1d(const void* x, const void* weight, const void* bias, void* conv_state, void* out,
                                  const int* seq_ids, const int* q_start, const int* q_len, const int* past_len,
                                  const int* slot_ids, int tokens, int num_seqs, int channels, int width, int activation,
                                  int is_bf16, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (width < 2 || width > 4) return fail("telb_causal_conv1d: width must be 2, 3 or 4");
    const dim3 g1((channels + 127) / 128, tokens), g2((channels + 127) / 128, num_seqs), blk(128);
#define TELB_CONV(T_, W_)                                                                                                      \
    do {                                                                                                                       \
        TELB_LAUNCH("conv1d_fwd_kernel", (conv1d_fwd_kernel<T_, W_>), g1, blk, 0, stream, (const T_*)x, (const T_*)weight,     \
                    (const T_*)bias, (const T_*)conv_state, (T_*)out, seq_ids, q_start, past_len, slot_ids, channels, activation); \
        TELB_LAUNCH("conv1d_state_kernel", (conv1d_state_kernel<T_, W_>), g2, blk, 0, stream, (const T_*)x, (T_*)conv_state, q_start, \
                    q_len, past_len, slot_ids, channels);                                                                      \
    } while (0)
    if (is_bf16) {
        if (width == 4) TELB_CONV(__nv_bfloat16, 4); else if (width == 3) TELB_CONV(__nv_bfloat16, 3); else TELB_CONV(__nv_bfloat16, 2);
    } else {
        if (width == 4) TELB_CONV(__half, 4); else if (width == 3) TELB_CONV(__half, 3); else TELB_CONV(__half, 2);
    }
#undef TELB_CONV
    return 0;
}

extern "C" int telb_ssm_scan(const void* x, const void* dt, const float* A, const void* B, const void* C, const float* D,
                             const float* dt_bias, const void* z, float* state, void* y, const int* q_start, const int* q_len,
                             const int* past_len, const int* slot_ids, int num_seqs, int nheads, int head_dim, int d_state,
                             int ngroups, int dt_softplus, float dt_limit, int is_bf16, int max_q_len, float* seg_scratch,
                             long long seg_scratch_floats, cudaStream_t stream) {
    if (num_seqs <= 0) return 0;
    if (head_dim != 64 || d_state != 128) return fail("telb_ssm_scan: head_dim 64 and d_state 128 are the compiled shape");
    if (seg_scratch && max_q_len >= 2 * kSsmSegLen) {
        // long prefill chunk: three passes over parallel segments (see ssm_scan_seg_kernel)
        const int max_segs = (max_q_len + kSsmSegLen - 1) / kSsmSegLen;
        const long long need = (long long)num_seqs * nheads * max_segs * (64 * 128 + 1);
        if (need <= seg_scratch_floats) {
            float* seg_state = seg_scratch;
            float* seg_decay = seg_scratch + (size_t)num_seqs * nheads * max_segs * 64 * 128;
            const dim3 g3(num_seqs, nheads, max_segs), g2(num_seqs, nheads);
#define TELB_SEG(T_)                                                                                                              \
    do {                                                                                                                           \
        TELB_LAUNCH("ssm_scan_seg_kernel", (ssm_scan_seg_kernel<T_, 64, 128, 1>), g3, dim3(64), 0, stream, (const T_*)x, (const T_*)dt, A, \
                    (const T_*)B, (const T_*)C, D, dt_bias, (const T_*)z, seg_state, seg_decay, (T_*)y, q_start, q_len, nheads, ngroups,   \
                    dt_softplus, dt_limit, kSsmSegLen, max_segs);                                                                  \
        TELB_LAUNCH("ssm_carry_kernel", (ssm_carry_kernel<64, 128>), g2, dim3(256), 0, stream, seg_state, (const float*)seg_decay, state,  \
                    q_len, past_len, slot_ids, nheads, kSsmSegLen, max_segs);                                                      \
        TELB_LAUNCH("ssm_scan_seg_kernel", (ssm_scan_seg_kernel<T_, 64, 128, 2>), g3, dim3(64), 0, stream, (const T_*)x, (const T_*)dt, A, \
                    (const T_*)B, (const T_*)C, D, dt_bias, (const T_*)z, seg_state, seg_decay, (T_*)y, q_start, q_len, nheads, ngroups,   \
                    dt_softplus, dt_limit, kSsmSegLen, max_segs);                                                                  \
    } while (0)
            if (is_bf16) TELB_SEG(__nv_bfloat16); else TELB_SEG(__half);
#undef TELB_SEG
            return 0;
        }
    }
    const dim3 grid(num_seqs, nheads);
    if (is_bf16)
        TELB_LAUNCH("ssm_scan_kernel", (ssm_scan_kernel<__nv_bfloat16, 64, 128>), grid, dim3(64), 0, stream, (const __nv_bfloat16*)x,
                    (const __nv_bfloat16*)dt, A, (const __nv_bfloat16*)B, (const __nv_bfloat16*)C, D, dt_bias, (const __nv_bfloat16*)z, state,
                    (__nv_bfloat16*)y, q_start, q_len, past_len, slot_ids, nheads, ngroups, dt_softplus, dt_limit);
    else
        TELB_LAUNCH("ssm_scan_kernel", (ssm_scan_kernel<__half, 64, 128>), grid, dim3(64), 0, stream, (const __half*)x, (const __half*)dt, A,
                    (const __half*)B, (const __half*)C, D, dt_bias, (const __half*)z, state, (__half*)y, q_start, q_len, past_len,
                    slot_ids, nheads, ngroups, dt_softplus, dt_limit);
    return 0;
}

extern "C" int telb_gated_delta_rule(const void* q, const void* k, const void* v, const void* a, const void* b,
                                     const float* A_log, const float* dt_bias, float* state, void* out, const int* q_start,
                                     const int* q_len, const int* past_len, const int* slot_ids, int num_seqs, int hk, int hv,
                                     int kdim, int vdim, int is_bf16, cudaStream_t stream) {
    if (num_seqs <= 0) return 0;
    if (kdim != 128 || vdim != 128) return fail("telb_gated_delta_rule: key / value head dims of 128 are the compiled shape");
    const dim3 grid(num_seqs, hv);
    if (is_bf16)
        TELB_LAUNCH("gdn_kernel", (gdn_kernel<__nv_bfloat16, 128, 128>), grid, dim3(128), 0, stream, (const __nv_bfloat16*)q,
                    (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, A_log, dt_bias, state,
                    (__nv_bfloat16*)out, q_start, q_len, past_len, slot_ids, hk, hv);
    else
        TELB_LAUNCH("gdn_kernel", (gdn_kernel<__half, 128, 128>), grid, dim3(128), 0, stream, (const __half*)q, (const __half*)k, (const __half*)v,
                    (const __half*)a, (const __half*)b, A_log, dt_bias, state, (__half*)out, q_start, q_len, past_len, slot_ids, hk, hv);
    return 0;
}
