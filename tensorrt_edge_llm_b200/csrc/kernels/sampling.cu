// Token sampling on the device: per-row temperature / top-k / top-p with a caller-supplied uniform
// per row (so a request's draws never depend on its batch position), plus the token-bitmask and
// logit-bias helpers used by guided decoding.
//
// One CTA per row:  radix-select the k-th largest logit (k = top_k, or 1024 when only top-p is
// set — the same candidate cap as the reference), gather the candidates into shared memory, bitonic
// sort them (value descending, index ascending), softmax with temperature, cut at top-p, sample.
// Rows with temperature < 1e-3 are greedy.  Among logits exactly equal to the k-th largest value the
// ones with the lowest token ids enter the candidate set, so the result never depends on the order in
// which threads arrive: a greedy row returns the lowest index of the maximum (the same answer as the
// arg-max kernel) whatever else is in the batch, and seeded sampling is reproducible.
//
// token_logprobs: the log-probability of each row's chosen token and the k most likely tokens with theirs (one CTA per row:
// an online max / sum-of-exponentials pass, then k ordered arg-max passes over the row, which stays in L2).
//
// Reference counterpart: cpp/sampler/sampling.cu (topKStage1/2, topP kernels, applyTokenBitmask,
// applyLogitBias); semantics cpp/sampler/sampling.h:56-160 (kMaxSamplingTopK 1024).
#include "host_utils.h"
#include "tc5_common.cuh"

namespace telb {

constexpr int kSampleThreads = 1024;
constexpr int kMaxCand = 1024;

__device__ __forceinline__ uint32_t order_key(float v) {
    const uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

template <typename T>
__device__ __forceinline__ float load_logit(const T* p, int i) {
    if constexpr (sizeof(T) == 4) return static_cast<float>(p[i]);
    else return Cvt<T>::to_f(p[i]);
}

template <typename T>
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const T* __restrict__ logits, long long stride, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniforms,
              int* __restrict__ out) {
    pdl_prologue();
    __shared__ unsigned long long cand[kMaxCand];
    __shared__ float scan[kMaxCand];
    __shared__ int hist[256];
    __shared__ int s_misc[4];
    __shared__ float s_wsum[32];
    const int row = blockIdx.x;
    const int tid = threadIdx.x;
    const T* p = logits + (size_t)row * stride;
    const float temp = temperature[row];
    const bool greedy = temp < 1e-3f;
    int k = greedy ? 1 : top_k[row];
    if (k <= 0 || k > kMaxCand) k = kMaxCand;
    if (k > vocab) k = vocab;

    // ---- radix select: key of the k-th largest logit ----
    uint32_t prefix = 0, mask = 0;
    int remaining = k;
    for (int pass = 3; pass >= 0; --pass) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        for (int i = tid; i < vocab; i += kSampleThreads) {
            const uint32_t key = order_key(load_logit(p, i));
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> (8 * pass)) & 0xFF], 1);
        }
        __syncthreads();
        if (tid == 0) {
            int cum = 0, bin = 255;
            for (; bin > 0; --bin) {
                if (cum + hist[bin] >= remaining) break;
                cum += hist[bin];
            }
            s_misc[0] = bin;
            s_misc[1] = remaining - cum;
            s_misc[3] = hist[bin];          // after the last pass: how many logits equal the threshold exactly
        }
        __syncthreads();
        prefix |= static_cast<uint32_t>(s_misc[0]) << (8 * pass);
        mask |= 0xFFu << (8 * pass);
        remaining = s_misc[1];
        __syncthreads();
    }
    const uint32_t thresh = prefix;         // `remaining` of the keys equal to it are wanted
    // ---- gather candidates ----
    const int n_equal = s_misc[3];
    __syncthreads();
    if (tid == 0) s_misc[2] = 0;
    cand[tid] = 0ull;
    __syncthreads();
    const bool all_ties = n_equal <= remaining;     // every logit equal to the threshold is wanted: no choice to make
    for (int i = tid; i < vocab; i += kSampleThreads) {
        const uint32_t key = order_key(load_logit(p, i));
        if (key > thresh || (all_ties && key == thresh)) {
            const int slot = atomicAdd(&s_misc[2], 1);
            if (slot < kMaxCand) cand[slot] = (static_cast<unsigned long long>(key) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(i));
        }
    }
    if (!all_ties) {
        // More ties than places: the `remaining` lowest token ids win.  Each thread owns a contiguous index range, counts
        // its ties, a block-wide exclusive scan turns the counts into ranks in index order, and ranks below `remaining`
        // are taken.  (The slot a candidate lands in is still arbitrary; the sort below orders by value, then index.)
        const int chunk = (vocab + kSampleThreads - 1) / kSampleThreads;
        const int lo = min(vocab, tid * chunk), hi = min(vocab, lo + chunk);
        int cnt = 0;
        for (int i = lo; i < hi; ++i) cnt += order_key(load_logit(p, i)) == thresh ? 1 : 0;
        int inc = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, inc, o);
            if ((tid & 31) >= o) inc += n;
        }
        __syncthreads();                             // hist[] is free again (the radix passes are over)
        if ((tid & 31) == 31) hist[tid >> 5] = inc;
        __syncthreads();
        if (tid < 32) {
            int w = hist[tid];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, w, o);
                if (tid >= o) w += n;
            }
            hist[32 + tid] = w;
        }
        __syncthreads();
        int rank = inc - cnt + ((tid >> 5) > 0 ? hist[32 + (tid >> 5) - 1] : 0);
        if (rank < remaining) {
            for (int i = lo; i < hi && rank < remaining; ++i) {
                if (order_key(load_logit(p, i)) == thresh) {
                    const int slot = atomicAdd(&s_misc[2], 1);
                    if (slot < kMaxCand) cand[slot] = (static_cast<unsigned long long>(thresh) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(i));
                    ++rank;
                }
            }
        }
    }
    __syncthreads();
    // ---- bitonic sort, descending ----
    for (int size = 2; size <= kMaxCand; size <<= 1) {
        for (int strd = size >> 1; strd > 0; strd >>= 1) {
            const int j = tid ^ strd;
            if (j > tid) {
                const unsigned long long a = cand[tid], b = cand[j];
                const bool desc = (tid & size) == 0;
                if (desc ? a < b : a > b) { cand[tid] = b; cand[j] = a; }
            }
            __syncthreads();
        }
    }
    if (greedy) {
        if (tid == 0) out[row] = static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(cand[0] & 0xFFFFFFFFull));
        return;
    }
    // ---- softmax over the candidates, inclusive scan ----
    const float vmax = key_value(static_cast<uint32_t>(cand[0] >> 32));
    float pr = 0.f;
    if (tid < k) pr = __expf((key_value(static_cast<uint32_t>(cand[tid] >> 32)) - vmax) / temp);
    float v = pr;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, v, o);
        if ((tid & 31) >= o) v += n;
    }
    if ((tid & 31) == 31) s_wsum[tid >> 5] = v;
    __syncthreads();
    if (tid < 32) {
        float w = s_wsum[tid];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n = __shfl_up_sync(0xffffffffu, w, o);
            if (tid >= o) w += n;
        }
        s_wsum[tid] = w;
    }
    __syncthreads();
    const float cum = v + ((tid >> 5) > 0 ? s_wsum[(tid >> 5) - 1] : 0.f);
    scan[tid] = cum;
    const float total = s_wsum[31];
    // ---- top-p cut: keep the sorted prefix whose mass before each token is < top_p ----
    const float tp = top_p[row];
    const bool kept = tid < k && (tp >= 1.f || (cum - pr) < tp * total);
    const int n_kept = __syncthreads_count(kept);
    const float kept_total = scan[max(n_kept, 1) - 1];
    const float target = uniforms[row] * kept_total;
    const int below = __syncthreads_count(tid < n_kept && cum <= target);
    if (tid == 0) {
        const int pick = min(below, max(n_kept, 1) - 1);
        out[row] = static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(cand[pick] & 0xFFFFFFFFull));
    }
}

// logits[row, i] = -1e30 where bit i of bitmask[row] is 0 (guided decoding); in place.
template <typename T>
__global__ void token_bitmask_kernel(T* __restrict__ logits, long long stride, int vocab, const int* __restrict__ bitmask, int words) {
    pdl_prologue();
    const int row = blockIdx.y;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) {
        if (!((bitmask[(size_t)row * words + (i >> 5)] >> (i & 31)) & 1)) {
            if constexpr (sizeof(T) == 4) logits[(size_t)row * stride + i] = -1e30f;
            else logits[(size_t)row * stride + i] = Cvt<T>::from_f(-6e4f);      // most negative finite half-range value
        }
    }
}

// logits[row, ids[j]] += bias[j] for the sparse bias list of each row.
template <typename T>
__global__ void logit_bias_kernel(T* __restrict__ logits, long long stride, const int* __restrict__ ids, const float* __restrict__ bias,
                                  const int* __restrict__ row_offsets) {
    pdl_prologue();
    const int row = blockIdx.x;
    for (int j = row_offsets[row] + threadIdx.x; j < row_offsets[row + 1]; j += blockDim.x) {
        T* q = logits + (size_t)row * stride + ids[j];
        if constexpr (sizeof(T) == 4) *q += bias[j];
        else *q = Cvt<T>::from_f(Cvt<T>::to_f(*q) + bias[j]);
    }
}


constexpr int kLogprobThreads = 512;
constexpr int kMaxLogprobs = 32;

// logits [rows, stride]; tokens [rows]; chosen [rows]; top_ids / top_vals [rows, k] ordered by (log-probability descending,
// token id ascending).  Pass j finds the best element that comes after pick j - 1 in that order, so no exclusion list is kept.
template <typename T>
__global__ void __launch_bounds__(kLogprobThreads) token_logprobs_kernel(const T* __restrict__ logits, long long stride, int vocab,
                                                                         const int* __restrict__ tokens, int k, float* __restrict__ chosen,
                                                                         int* __restrict__ top_ids, float* __restrict__ top_vals) {
    pdl_prologue();
    __shared__ float s_m[kLogprobThreads / 32], s_s[kLogprobThreads / 32];
    __shared__ unsigned long long s_key[kLogprobThreads / 32];
    __shared__ float s_lse;
    __shared__ unsigned long long s_prev;
    const int row = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const T* p = logits + (size_t)row * stride;
    float m = -INFINITY, sum = 0.f;
    for (int i = tid; i < vocab; i += kLogprobThreads) {
        const float v = load_logit(p, i);
        if (v > m) {
            sum = sum * __expf(m - v) + 1.f;
            m = v;
        } else if (v > -INFINITY) {
            sum += __expf(v - m);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, sum, o);
        const float mm = fmaxf(m, m2);
        sum = (m == -INFINITY ? 0.f : sum * __expf(m - mm)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mm));
        m = mm;
    }
    if (lane == 0) {
        s_m[warp] = m;
        s_s[warp] = sum;
    }
    __syncthreads();
    if (tid == 0) {
        float mm = -INFINITY, ss = 0.f;
        for (int w = 0; w < kLogprobThreads / 32; ++w) mm = fmaxf(mm, s_m[w]);
        for (int w = 0; w < kLogprobThreads / 32; ++w)
            if (s_m[w] > -INFINITY) ss += s_s[w] * __expf(s_m[w] - mm);
        s_lse = mm + logf(ss);
        const int t = min(max(tokens[row], 0), vocab - 1);
        chosen[row] = load_logit(p, t) - s_lse;
        s_prev = ~0ull;                                   // above every key: the first pass takes the overall best
    }
    __syncthreads();
    const float lse = s_lse;
    for (int j = 0; j < k; ++j) {
        const unsigned long long prev = s_prev;
        unsigned long long best = 0ull;
        for (int i = tid; i < vocab; i += kLogprobThreads) {
            float v = load_logit(p, i);
            if (!(v == v)) v = -INFINITY;
            if (v == 0.f) v = 0.f;
            const unsigned long long key = (static_cast<unsigned long long>(order_key(v)) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(i));
            if (key < prev && key > best) best = key;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        if (lane == 0) s_key[warp] = best;
        __syncthreads();
        if (tid == 0) {
            unsigned long long b = 0ull;
            for (int w = 0; w < kLogprobThreads / 32; ++w) b = s_key[w] > b ? s_key[w] : b;
            s_prev = b;
            if (b != 0ull) {
                top_ids[(size_t)row * k + j] = static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(b & 0xFFFFFFFFull));
                top_vals[(size_t)row * k + j] = key_value(static_cast<uint32_t>(b >> 32)) - lse;
            } else {                                      // fewer than k elements
                top_ids[(size_t)row * k + j] = -1;
                top_vals[(size_t)row * k + j] = -INFINITY;
            }
        }
        __syncthreads();
    }
}

}  // namespace telb

using namespace telb;

// Log-probability of tokens[row] under softmax(logits[row]) and the k (<= 32) most likely tokens with theirs.  dtype as in telb_sample.
extern "C" int telb_token_logprobs(const void* logits, long long stride, int rows, int vocab, const int* tokens, int k, float* chosen,
                                   int* top_ids, float* top_vals, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (k < 0 || k > kMaxLogprobs) return fail("telb_token_logprobs: 0..32 alternatives");
    if (dtype == 2)
        TELB_LAUNCH("token_logprobs_kernel", (token_logprobs_kernel<float>), dim3(rows), dim3(kLogprobThreads), 0, stream, (const float*)logits, stride, vocab, tokens, k, chosen, top_ids, top_vals);
    else if (dtype == 1)
        TELB_LAUNCH("token_logprobs_kernel", (token_logprobs_kernel<__nv_bfloat16>), dim3(rows), dim3(kLogprobThreads), 0, stream, (const __nv_bfloat16*)logits, stride, vocab, tokens, k, chosen, top_ids, top_vals);
    else
        TELB_LAUNCH("token_logprobs_kernel", (token_logprobs_kernel<__half>), dim3(rows), dim3(kLogprobThreads), 0, stream, (const __half*)logits, stride, vocab, tokens, k, chosen, top_ids, top_vals);
    TELB_CHECK_LAUNCH("token_logprobs_kernel");
    return 0;
}

// dtype: 0 = fp16, 1 = bf16, 2 = fp32
extern "C" int telb_sample(const void* logits, long long stride, int rows, int vocab, const float* temperature,
                           const int* top_k, const float* top_p, const float* uniforms, int* out, int dtype,
                           cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (dtype == 2)
        TELB_LAUNCH("sample_kernel", (sample_kernel<float>), dim3(rows), dim3(kSampleThreads), 0, stream, (const float*)logits, stride, vocab,
                    temperature, top_k, top_p, uniforms, out);
    else if (dtype == 1)
        TELB_LAUNCH("sample_kernel", (sample_kernel<__nv_bfloat16>), dim3(rows), dim3(kSampleThreads), 0, stream, (const __nv_bfloat16*)logits,
                    stride, vocab, temperature, top_k, top_p, uniforms, out);
    else
        TELB_LAUNCH("sample_kernel", (sample_kernel<__half>), dim3(rows), dim3(kSampleThreads), 0, stream, (const __half*)logits, stride, vocab,
                    temperature, top_k, top_p, uniforms, out);
    return 0;
}

extern "C" int telb_apply_token_bitmask(void* logits, long long stride, int rows, int vocab, const int* bitmask, int dtype,
                                        cudaStream_t stream) {
    if (rows <= 0) return 0;
    const int words = (vocab + 31) / 32;
    const dim3 grid(64, rows), blk(256);
    if (dtype == 2) TELB_LAUNCH("token_bitmask_kernel", (token_bitmask_kernel<float>), grid, blk, 0, stream, (float*)logits, stride, vocab, bitmask, words);
    else if (dtype == 1) TELB_LAUNCH("token_bitmask_kernel", (token_bitmask_kernel<__nv_bfloat16>), grid, blk, 0, stream, (__nv_bfloat16*)logits, stride, vocab, bitmask, words);
    else TELB_LAUNCH("token_bitmask_kernel", (token_bitmask_kernel<__half>), grid, blk, 0, stream, (__half*)logits, stride, vocab, bitmask, words);
    return 0;
}

extern "C" int telb_apply_logit_bias(void* logits, long long stride, int rows, const int* ids, const float* bias,
                                     const int* row_offsets, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (dtype == 2) TELB_LAUNCH("logit_bias_kernel", (logit_bias_kernel<float>), dim3(rows), dim3(128), 0, stream, (float*)logits, stride, ids, bias, row_offsets);
    else if (dtype == 1) TELB_LAUNCH("logit_bias_kernel", (logit_bias_kernel<__nv_bfloat16>), dim3(rows), dim3(128), 0, stream, (__nv_bfloat16*)logits, stride, ids, bias, row_offsets);
    else TELB_LAUNCH("logit_bias_kernel", (logit_bias_kernel<__half>), dim3(rows), dim3(128), 0, stream, (__half*)logits, stride, ids, bias, row_offsets);
    return 0;
}
