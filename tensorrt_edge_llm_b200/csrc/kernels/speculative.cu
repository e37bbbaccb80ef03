// Speculative-decoding helpers that touch per-sequence trees and the paged KV cache:
//   spec_accept_greedy   walk each sequence's verification tree from the root, following the child whose
//                        token equals the target model's arg-max at the current node; emits the accepted
//                        path, its length and the bonus token.  A forced length per sequence (benchmark
//                        mode, null = off) follows the first child instead of comparing tokens.
//   spec_accept_sampling lossless acceptance for sampled requests: a node's children are tried in order, child c is kept with
//                        the target's (residual) probability of its token, a rejected token leaves the distribution; when no
//                        child is kept the bonus token is drawn from what is left.  One CTA per sequence, no host read.
//   kv_commit_path       compact the accepted path in the paged cache: the entry written at tree slot
//                        past + path[j] moves to past + j, for every layer / K,V / head, in place.
//
//   eagle_tree_meta      from a parent table (parents precede children) build what a tree step needs on the
//                        device: the packed ancestor mask (bit c of row r = "row r may attend new row c"), the
//                        depth of every row and its RoPE position, so no tree shape is read back by the host.
//   eagle_select_verify  pick the `keep` best-scoring nodes of the draft's candidate pool, keep them in pool
//                        order (so parents still precede children), renumber their parents and prepend the
//                        root: tokens, parents and depths of the verification tree.
//
//   dflash2_conv         one side of DFlash 2's per-token dynamic grouped depthwise convolution along a proposal block
//                        (fixed per-channel taps plus per-token, per-group offsets; causal, never across a block edge).
//   dflash2_selector     DFlash 2's chain selector: one CTA per sequence walks the proposal slots, scoring each slot's
//                        candidates against the token chosen for the slot before (bilinear codebook term), greedy or sampled.
//   markov_greedy_step   DSpark's Markov head, one proposal step for the whole batch: logits + W2 · W1[prev] and its arg-max in
//                        one pass over W2 (the winner is an atomic max of packed (value, id) keys, read by the next step).
//   lattice_chain_walk   LiLiCorr's walk over per-slot candidates with a [prev, next] transition table per slot.
//   candidate_rescore    second half of the EAGLE-4 low-rank candidate head: exact fp32 logits of each row's candidate
//                        tokens from their lm_head rows, candidates ordered by (logit descending, id ascending) and
//                        log-softmax over the set.  The first half (two small GEMMs and a top-k) runs as library ops.
//
// Reference counterparts: cpp/plugins/lowRankCandidateHeadPlugin (candidate head),
// cpp/kernels/speculative/dflash2GroupedDynamicConv.cu, dflash2CandidateSelector.cu (chain walk), lilicorrChainWalk.cu, dsparkKernels.cu (fused greedy Markov step),
// cpp/kernels/speculative/speculativeKernels.cu (acceptGreedy, the tree construction
// kernels at :509 and :571, commitSpecTargetKVBatchedKernel :1692), forceAcceptanceKernels.cu.
#include "host_utils.h"
#include "tc5_common.cuh"

namespace telb {

constexpr int kMaxTreeNodes = 128;      // same cap as the reference's tree size limit

// One warp per sequence.  Nodes are ordered so that a parent precedes its children.
__global__ void spec_accept_greedy_kernel(const int* __restrict__ target_tokens, const int* __restrict__ tree_tokens,
                                          const int* __restrict__ parents, int* __restrict__ path, int* __restrict__ path_len,
                                          int* __restrict__ bonus, int nodes, int max_path, const int* __restrict__ force_lens) {
    pdl_prologue();
    const int b = blockIdx.x, lane = threadIdx.x;
    const int* tt = target_tokens + (size_t)b * nodes;
    const int* tr = tree_tokens + (size_t)b * nodes;
    const int* pa = parents + (size_t)b * nodes;
    const int force_len = force_lens ? force_lens[b] : 0;
    int cur = 0, len = 1;
    if (lane == 0) path[(size_t)b * max_path] = 0;
    while (len < max_path) {
        if (force_len > 0 && len >= force_len) break;
        const int want = tt[cur];
        int found = nodes;
        for (int c = cur + 1 + lane; c < nodes; c += 32) {
            if (pa[c] == cur && (force_len > 0 || tr[c] == want)) {
                found = c;
                break;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) found = min(found, __shfl_xor_sync(0xffffffffu, found, o));
        if (found >= nodes) break;
        cur = found;
        if (lane == 0) path[(size_t)b * max_path + len] = cur;
        ++len;
    }
    if (lane == 0) {
        path_len[b] = len;
        bonus[b] = tt[cur];
    }
}

// grid (B, layers * 2 * Hkv); the block first pulls every source row into registers, then stores.
template <int D>
__global__ void __launch_bounds__(256)
kv_commit_path_kernel(uint4* __restrict__ pool, const int* __restrict__ page_table, const int* __restrict__ past_len,
                      const int* __restrict__ path, const int* __restrict__ path_len, int max_path, int max_pages, int num_pages,
                      int hkv, int page_size) {
    pdl_prologue();
    constexpr int kVecPerRow = D * 2 / 16;
    const int b = blockIdx.x;
    const int m = path_len[b] - 1;               // rows to move (path[0] is the root and stays)
    if (m <= 0) return;
    const int lkh = blockIdx.y;                   // (layer * 2 + kv) * hkv + head
    const int head = lkh % hkv;
    const int lk = lkh / hkv;                     // layer * 2 + kv
    const int past = past_len[b];
    const int* pt = page_table + (size_t)b * max_pages;
    auto row_ptr = [&](int slot) -> uint4* {
        const int page = pt[slot / page_size];
        const size_t layer = lk >> 1, kv = lk & 1;
        return pool + ((((layer * num_pages + page) * 2 + kv) * hkv + head) * (size_t)page_size + slot % page_size) * kVecPerRow;
    };
    constexpr int kPer = 4;                       // up to 4 vectors per thread: 1024 vectors = 64 rows of D = 128
    uint4 v[kPer];
    const int total = m * kVecPerRow;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        const int idx = threadIdx.x + i * 256;
        if (idx < total) {
            const int j = idx / kVecPerRow + 1;
            v[i] = row_ptr(past + path[(size_t)b * max_path + j])[idx % kVecPerRow];
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        const int idx = threadIdx.x + i * 256;
        if (idx < total) {
            const int j = idx / kVecPerRow + 1;
            row_ptr(past + j)[idx % kVecPerRow] = v[i];
        }
    }
}

// One thread per tree row: walk to the root setting one bit per ancestor.  `parents` index rows of the same tree (−1 = no
// parent among the new rows).  depth_base is the depth given to parentless rows (1 for draft rows hanging under the root
// that is not part of the step, 0 for a verification tree whose row 0 is the root).
__global__ void eagle_tree_meta_kernel(const int* __restrict__ parents, const int* __restrict__ base_pos, int* __restrict__ mask,
                                       int* __restrict__ depth, int* __restrict__ positions, int rows, int words, int depth_base,
                                       int pos_offset) {
    pdl_prologue();
    const int b = blockIdx.x;
    const int* pa = parents + (size_t)b * rows;
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
        uint32_t w[kMaxTreeNodes / 32];
#pragma unroll
        for (int i = 0; i < kMaxTreeNodes / 32; ++i) w[i] = 0u;
        int cur = r, d = depth_base;
        for (int hops = 0; hops < rows; ++hops) {          // bounded even if the table were cyclic
            w[cur >> 5] |= 1u << (cur & 31);
            const int up = pa[cur];
            if (up < 0 || up >= cur) break;
            cur = up;
            ++d;
        }
        for (int i = 0; i < words; ++i) mask[((size_t)b * rows + r) * words + i] = (int)w[i];
        if (depth) depth[(size_t)b * rows + r] = d;
        if (positions) positions[(size_t)b * rows + r] = base_pos[b] + d + pos_offset;
    }
}

constexpr int kMaxPool = 2048;      // candidate pool per sequence (top-k 16 x depth 8 stays far below)

// One CTA per sequence.  rank(i) = number of candidates that beat i (higher score, or equal score and lower index): the
// stable descending order of the host formulation.  Selected nodes keep their pool order.
__global__ void __launch_bounds__(256)
eagle_select_verify_kernel(const float* __restrict__ p_sc, const int* __restrict__ p_tok, const int* __restrict__ p_par,
                           const int* __restrict__ p_dep, const int* __restrict__ root, int pool, int keep, int* __restrict__ tree_tok,
                           int* __restrict__ tree_par, int* __restrict__ tree_dep) {
    pdl_prologue();
    __shared__ float s_sc[kMaxPool];
    __shared__ short s_slot[kMaxPool];         // output slot (1-based) of a selected candidate, 0 = not selected
    __shared__ int s_warp[8];
    const int b = blockIdx.x;
    const float* sc = p_sc + (size_t)b * pool;
    for (int i = threadIdx.x; i < pool; i += blockDim.x) s_sc[i] = sc[i];
    __syncthreads();
    const int nn = keep + 1;
    // candidates are walked in blocks of 256 consecutive indices so that a block scan yields the pool-order slot
    int base_slot = 0;
    for (int i0 = 0; i0 < pool; i0 += blockDim.x) {
        const int i = i0 + threadIdx.x;
        int sel = 0;
        if (i < pool) {
            const float mine = s_sc[i];
            int rank = 0;
            for (int j = 0; j < pool; ++j) {
                const float o = s_sc[j];
                rank += (o > mine || (o == mine && j < i)) ? 1 : 0;
            }
            sel = rank < keep ? 1 : 0;
        }
        // inclusive scan of `sel` over the block
        int v = sel;
        const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, v, o);
            if (lane >= o) v += t;
        }
        if (lane == 31) s_warp[wid] = v;
        __syncthreads();
        int before = 0;
        for (int w = 0; w < wid; ++w) before += s_warp[w];
        int total = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += s_warp[w];
        if (i < pool) s_slot[i] = sel ? (short)(base_slot + before + v) : (short)0;
        base_slot += total;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        tree_tok[(size_t)b * nn] = root[b];
        tree_par[(size_t)b * nn] = -1;
        tree_dep[(size_t)b * nn] = 0;
    }
    for (int i = threadIdx.x; i < pool; i += blockDim.x) {
        const int slot = s_slot[i];
        if (slot > 0) {
            const int par = p_par[(size_t)b * pool + i];
            // a selected node's parent is selected too whenever scores fall along a path (cumulative log-probabilities);
            // a parent that was not kept re-attaches the node to the root
            tree_tok[(size_t)b * nn + slot] = p_tok[(size_t)b * pool + i];
            tree_par[(size_t)b * nn + slot] = par < 0 ? 0 : (int)s_slot[par];
            tree_dep[(size_t)b * nn + slot] = p_dep[(size_t)b * pool + i];
        }
    }
}


// out[t, c] = sum_{k < K, k <= t % block} (base[k, c] + delta[t, k, c / group]) * hidden[t - k, c]  (+ residual[t, c]).
// One thread per channel pair (group sizes are even, so a pair shares its group); grid (channel pairs / 256, tokens).
template <typename T, int K>
__global__ void __launch_bounds__(256) dflash2_conv_kernel(const T* __restrict__ hidden, const T* __restrict__ delta,
                                                           const T* __restrict__ base, const T* __restrict__ residual,
                                                           T* __restrict__ out, int H, int block, int group_size) {
    pdl_prologue();
    const int t = blockIdx.y;
    const int pc = blockIdx.x * 256 + threadIdx.x;
    if (pc * 2 >= H) return;
    const int c = pc * 2, groups = H / group_size, g = c / group_size, pos = t % block;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
        if (pos >= k) {
            const float dyn = Cvt<T>::to_f(delta[((size_t)t * K + k) * groups + g]);
            const T* b = base + (size_t)k * H + c;
            const T* x = hidden + (size_t)(t - k) * H + c;
            s0 = fmaf(Cvt<T>::to_f(b[0]) + dyn, Cvt<T>::to_f(x[0]), s0);
            s1 = fmaf(Cvt<T>::to_f(b[1]) + dyn, Cvt<T>::to_f(x[1]), s1);
        }
    }
    if (residual != nullptr) {
        s0 += Cvt<T>::to_f(residual[(size_t)t * H + c]);
        s1 += Cvt<T>::to_f(residual[(size_t)t * H + c + 1]);
    }
    *reinterpret_cast<uint32_t*>(out + (size_t)t * H + c) = Cvt<T>::pack2(s0, s1);
}

constexpr int kSelMaxTopK = 32;
constexpr int kSelMaxRank = 1024;

// One CTA of topk warps per sequence; the slots are walked in order because slot s depends on the token chosen for s - 1.
template <typename T>
__global__ void __launch_bounds__(1024) dflash2_selector_kernel(const int* __restrict__ cand, const float* __restrict__ unary,
                                                               const T* __restrict__ projected, const int* __restrict__ anchor,
                                                               const T* __restrict__ pred_cb, const T* __restrict__ succ_cb,
                                                               const float* __restrict__ temperatures, const float* __restrict__ uniforms,
                                                               int* __restrict__ tokens, float* __restrict__ probs, int steps, int topk,
                                                               int rank, int vocab) {
    pdl_prologue();
    __shared__ float s_query[kSelMaxRank];
    __shared__ float s_score[kSelMaxTopK];
    __shared__ float s_prob[kSelMaxTopK];
    __shared__ int s_prev;
    const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) s_prev = anchor[b];
    __syncthreads();
    const bool greedy = temperatures == nullptr || temperatures[b] < 1e-3f;
    for (int step = 0; step < steps; ++step) {
        const size_t row = (size_t)b * steps + step;
        const int prev = s_prev;
        const bool prev_ok = prev >= 0 && prev < vocab;
        for (int r = threadIdx.x; r < rank; r += blockDim.x)
            s_query[r] = prev_ok ? Cvt<T>::to_f(pred_cb[(size_t)prev * rank + r]) * Cvt<T>::to_f(projected[row * rank + r]) : 0.f;
        __syncthreads();
        if (warp < topk) {
            const int c = cand[row * topk + warp];
            float dot = 0.f;
            if (c >= 0 && c < vocab) {
                const T* q = succ_cb + (size_t)c * rank;
                for (int r = lane; r < rank; r += 32) dot = fmaf(s_query[r], Cvt<T>::to_f(q[r]), dot);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            if (lane == 0) s_score[warp] = unary[row * topk + warp] + dot;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int sel = 0;
            if (greedy) {
                float best = -INFINITY;
                int best_tok = 0x7fffffff;
                for (int k = 0; k < topk; ++k) {
                    const int tok = cand[row * topk + k];
                    if (s_score[k] > best || (s_score[k] == best && tok < best_tok)) {
                        best = s_score[k];
                        best_tok = tok;
                        sel = k;
                    }
                }
                for (int k = 0; k < topk; ++k) s_prob[k] = k == sel ? 1.f : 0.f;
            } else {
                const float inv_t = 1.f / temperatures[b];
                float mx = -INFINITY;
                for (int k = 0; k < topk; ++k) mx = fmaxf(mx, s_score[k] * inv_t);
                float sum = 0.f;
                for (int k = 0; k < topk; ++k) {
                    s_prob[k] = expf(s_score[k] * inv_t - mx);
                    sum += s_prob[k];
                }
                const float u = fminf(fmaxf(uniforms[row], 0.f), 0.99999994f);
                float cum = 0.f;
                sel = topk - 1;
                bool found = false;
                for (int k = 0; k < topk; ++k) {
                    s_prob[k] /= sum;
                    cum += s_prob[k];
                    if (!found && u < cum) {
                        sel = k;
                        found = true;
                    }
                }
            }
            s_prev = cand[row * topk + sel];
            tokens[row] = s_prev;
        }
        __syncthreads();
        if (threadIdx.x < topk) probs[row * topk + threadIdx.x] = s_prob[threadIdx.x];
        __syncthreads();
    }
}

__device__ __forceinline__ unsigned long long pack_greedy_key(float v, int idx) {
    if (!(v == v)) v = -INFINITY;                       // NaN never wins
    if (v == 0.f) v = 0.f;                              // -0 and +0 are one value
    uint32_t bits = __float_as_uint(v);
    bits = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
    return (static_cast<unsigned long long>(bits) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(idx));   // ties: the lowest id
}

constexpr int kMarkovMaxRank = 512;
constexpr int kMarkovWarps = 8;

// One proposal step of the Markov head for every sequence.  logits [B, P, V] fp32; w1 [V1, R], w2 [V, R] 16-bit; slots [B, P] u64,
// zeroed before step 0.  A CTA owns `rows_per_cta` vocabulary rows: it reads each W2 row once and scores it for all B sequences.
// Dynamic shared memory: B * R floats (the queries W1[prev_b]) then B u64 (the CTA's best key per sequence).
template <typename T>
__global__ void __launch_bounds__(kMarkovWarps * 32) markov_greedy_step_kernel(const float* __restrict__ logits, const T* __restrict__ w1,
                                                                               const T* __restrict__ w2, const int* __restrict__ first_prev,
                                                                               unsigned long long* __restrict__ slots, int step, int P,
                                                                               int V, int V1, int R, int B, int rows_per_cta) {
    pdl_prologue();
    extern __shared__ __align__(8) unsigned char mk_smem[];
    float* s_q = reinterpret_cast<float*>(mk_smem);
    unsigned long long* s_best = reinterpret_cast<unsigned long long*>(s_q + (((size_t)B * R + 1) & ~size_t(1)));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < B * R; i += blockDim.x) {
        const int b = i / R, r = i - b * R;
        int prev = step == 0 ? first_prev[b] : static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(slots[(size_t)b * P + step - 1] & 0xFFFFFFFFull));
        prev = min(max(prev, 0), V1 - 1);
        s_q[i] = Cvt<T>::to_f(w1[(size_t)prev * R + r]);
    }
    for (int b = threadIdx.x; b < B; b += blockDim.x) s_best[b] = 0ull;
    __syncthreads();
    const int row0 = blockIdx.x * rows_per_cta;
    const int row1 = min(V, row0 + rows_per_cta);
    constexpr int kPerLane = kMarkovMaxRank / 32;
    for (int row = row0 + warp; row < row1; row += kMarkovWarps) {
        float w[kPerLane];
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
            const int r = lane + 32 * i;
            w[i] = r < R ? Cvt<T>::to_f(w2[(size_t)row * R + r]) : 0.f;
        }
        for (int b = 0; b < B; ++b) {
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < kPerLane; ++i) {
                const int r = lane + 32 * i;
                if (r < R) dot = fmaf(w[i], s_q[(size_t)b * R + r], dot);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            if (lane == 0) atomicMax(&s_best[b], pack_greedy_key(logits[((size_t)b * P + step) * V + row] + dot, row));
        }
    }
    __syncthreads();
    for (int b = threadIdx.x; b < B; b += blockDim.x)
        if (s_best[b] != 0ull) atomicMax(&slots[(size_t)b * P + step], s_best[b]);
}

__global__ void markov_unpack_kernel(const unsigned long long* __restrict__ slots, int* __restrict__ tokens, int n) {
    pdl_prologue();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) tokens[i] = static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(slots[i] & 0xFFFFFFFFull));
}

// One warp per sequence; lane k owns candidate k (topk <= 32).  transition [B, S, K, K] fp32.
__global__ void __launch_bounds__(32) lattice_chain_walk_kernel(const int* __restrict__ cand, const float* __restrict__ transition,
                                                                const float* __restrict__ temperatures, const float* __restrict__ uniforms,
                                                                int* __restrict__ tokens, float* __restrict__ probs, int steps, int topk) {
    pdl_prologue();
    const int b = blockIdx.x, lane = threadIdx.x;
    const bool greedy = temperatures == nullptr || temperatures[b] < 1e-3f;
    const float inv_t = greedy ? 1.f : 1.f / temperatures[b];
    int prev = 0;
    for (int step = 0; step < steps; ++step) {
        const size_t row = (size_t)b * steps + step;
        const float sc = lane < topk ? transition[(row * topk + prev) * topk + lane] * inv_t : -INFINITY;
        float mx = sc;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        int sel;
        float p;
        if (greedy) {
            const unsigned best = __ballot_sync(0xffffffffu, lane < topk && sc == mx);
            sel = best ? __ffs(best) - 1 : 0;                       // lowest index among the maxima (0 if every score is NaN)
            p = lane == sel ? 1.f : 0.f;
        } else {
            const float e = lane < topk ? expf(sc - mx) : 0.f;
            float sum = e;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            p = e / sum;
            float cum = p;                                          // inclusive prefix sum over lanes
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float v = __shfl_up_sync(0xffffffffu, cum, o);
                if (lane >= o) cum += v;
            }
            const float u = fminf(fmaxf(uniforms[row], 0.f), 0.99999994f);
            const unsigned hit = __ballot_sync(0xffffffffu, lane < topk && u < cum);
            sel = hit ? __ffs(hit) - 1 : topk - 1;
        }
        if (lane < topk) probs[row * topk + lane] = p;
        if (lane == 0) tokens[row] = cand[row * topk + sel];
        prev = sel;
    }
}

constexpr int kAcceptThreads = 256;
constexpr int kAcceptMaxRejected = 64;

// probs [B, N, V] fp32 (each row a distribution), tree_tokens / parents [B, N], uniforms [B, max_path, kw] (kw - 1 sibling trials and
// one bonus draw per depth) -> path [B, max_path], path_len [B], bonus [B].  Sums run in double, like the host restatement.
__global__ void __launch_bounds__(kAcceptThreads) spec_accept_sampling_kernel(const float* __restrict__ probs, const int* __restrict__ tree_tokens,
                                                                              const int* __restrict__ parents, const float* __restrict__ uniforms,
                                                                              int* __restrict__ path, int* __restrict__ path_len,
                                                                              int* __restrict__ bonus, int N, int V, int max_path, int kw) {
    pdl_prologue();
    __shared__ double s_part[kAcceptThreads];
    __shared__ int s_rej[kAcceptMaxRejected];
    __shared__ int s_nrej, s_next, s_seg;
    __shared__ double s_total, s_rejmass, s_before;
    const int b = blockIdx.x, tid = threadIdx.x;
    const int* tok = tree_tokens + (size_t)b * N;
    const int* par = parents + (size_t)b * N;
    const float* u = uniforms + (size_t)b * max_path * kw;
    const int seg = (V + kAcceptThreads - 1) / kAcceptThreads;           // contiguous vocabulary segment per thread
    const int lo = min(V, tid * seg), hi = min(V, lo + seg);
    int cur = 0, ln = 1;
    if (tid == 0) path[(size_t)b * max_path] = 0;
    for (;;) {
        const float* p = probs + ((size_t)b * N + cur) * V;
        const int depth = ln - 1;
        double part = 0.0;
        for (int i = lo; i < hi; ++i) part += (double)p[i];
        s_part[tid] = part;
        __syncthreads();
        if (tid == 0) {
            double total = 0.0;
            for (int i = 0; i < kAcceptThreads; ++i) total += s_part[i];
            int nrej = 0, nxt = -1;
            double rejmass = 0.0;
            if (ln < max_path) {
                int trial = 0;
                for (int c = cur + 1; c < N; ++c) {
                    if (par[c] != cur) continue;
                    const int t = min(max(tok[c], 0), V - 1);
                    bool gone = false;
                    for (int j = 0; j < nrej; ++j) gone = gone || s_rej[j] == t;
                    const double mass = total - rejmass;
                    const double pc = (mass > 0.0 && !gone) ? (double)p[t] / mass : 0.0;
                    if ((double)u[depth * kw + min(trial, kw - 2)] < pc) {
                        nxt = c;
                        break;
                    }
                    if (!gone && nrej < kAcceptMaxRejected) {
                        s_rej[nrej++] = t;
                        rejmass += (double)p[t];
                    }
                    ++trial;
                }
            }
            if (nxt < 0 && total - rejmass <= 0.0) {       // every token with mass was a rejected candidate: fall back to the full row
                nrej = 0;
                rejmass = 0.0;
            }
            s_total = total;
            s_rejmass = rejmass;
            s_nrej = nrej;
            s_next = nxt;
        }
        __syncthreads();
        if (s_next >= 0) {
            cur = s_next;
            if (tid == 0) path[(size_t)b * max_path + ln] = cur;
            ++ln;
            __syncthreads();
            continue;
        }
        // bonus draw: first index whose cumulative residual mass reaches u * mass
        const int nrej = s_nrej;
        if (nrej > 0) {                                     // segment sums without the rejected tokens
            for (int j = 0; j < nrej; ++j) {
                const int t = s_rej[j];
                if (t >= lo && t < hi) part -= (double)p[t];
            }
        }
        __syncthreads();
        s_part[tid] = part;
        __syncthreads();
        if (tid == 0) {
            const double target = (double)u[depth * kw + kw - 1] * (s_total - s_rejmass);
            double cum = 0.0;
            int sg = kAcceptThreads - 1;
            for (int i = 0; i < kAcceptThreads; ++i) {
                if (cum + s_part[i] >= target && s_part[i] > 0.0) {
                    sg = i;
                    break;
                }
                cum += s_part[i];
            }
            if (sg == kAcceptThreads - 1 && !(cum + s_part[sg] >= target)) {
                // rounding left the target just above the total: the last segment that holds mass
                cum = 0.0;
                int last = 0;
                for (int i = 0; i < kAcceptThreads; ++i)
                    if (s_part[i] > 0.0) last = i;
                for (int i = 0; i < last; ++i) cum += s_part[i];
                sg = last;
            }
            s_seg = sg;
            s_before = cum;
        }
        __syncthreads();
        if (tid == s_seg) {
            const double target = (double)u[depth * kw + kw - 1] * (s_total - s_rejmass);
            double cum = s_before;
            int pick = -1, last_mass = -1;
            for (int i = lo; i < hi; ++i) {
                double v = (double)p[i];
                for (int j = 0; j < nrej; ++j)
                    if (s_rej[j] == i) v = 0.0;
                if (v > 0.0) last_mass = i;
                cum += v;
                if (cum >= target && v > 0.0) {
                    pick = i;
                    break;
                }
            }
            if (pick < 0) pick = last_mass >= 0 ? last_mass : min(V - 1, max(lo, 0));
            bonus[b] = pick;
            path_len[b] = ln;
        }
        return;
    }
}

// One CTA per row.  hidden [R, H] and lm_head [V, H] 16-bit, cand [R, kc] int32 (distinct ids per row).
// Shared memory: H floats (the row), kc floats (logits), kc ints (ids).
template <typename T>
__global__ void __launch_bounds__(256) candidate_rescore_kernel(const T* __restrict__ hidden, const T* __restrict__ lm_head,
                                                                const int* __restrict__ cand, int* __restrict__ out_ids,
                                                                float* __restrict__ out_lp, int H, int kc, int vocab) {
    pdl_prologue();
    extern __shared__ float cr_smem[];
    float* s_h = cr_smem;
    float* s_l = s_h + H;
    int* s_id = reinterpret_cast<int*>(s_l + kc);
    __shared__ float s_red[8];
    const int r = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < H; i += 256) s_h[i] = Cvt<T>::to_f(hidden[(size_t)r * H + i]);
    __syncthreads();
    for (int c = warp; c < kc; c += 8) {
        int id = cand[(size_t)r * kc + c];
        id = min(max(id, 0), vocab - 1);
        const uint4* row = reinterpret_cast<const uint4*>(lm_head + (size_t)id * H);
        float acc = 0.f;
        for (int i = lane; i < H / 8; i += 32) {
            const uint4 u = __ldg(row + i);
            const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
            for (int q = 0; q < 8; ++q) acc += Cvt<T>::to_f(e[q]) * s_h[i * 8 + q];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) {
            const bool finite = (acc - acc) == 0.f;                 // false for inf and NaN
            s_l[c] = finite ? acc : -INFINITY;
            s_id[c] = id;
        }
    }
    __syncthreads();
    // the maximum, then the log of the sum of exponentials
    float mx = -INFINITY;
    for (int c = tid; c < kc; c += 256) mx = fmaxf(mx, s_l[c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) s_red[warp] = mx;
    __syncthreads();
    mx = s_red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, s_red[w]);
    __syncthreads();
    float sum = 0.f;
    for (int c = tid; c < kc; c += 256) sum += (s_l[c] == -INFINITY) ? 0.f : expf(s_l[c] - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) s_red[warp] = sum;
    __syncthreads();
    sum = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) sum += s_red[w];
    const float lse = sum > 0.f ? mx + logf(sum) : -INFINITY;
    // rank of every candidate = how many candidates come before it
    for (int c = tid; c < kc; c += 256) {
        const float l = s_l[c];
        const int id = s_id[c];
        int rank = 0;
        for (int j = 0; j < kc; ++j) {
            const float lj = s_l[j];
            rank += (lj > l || (lj == l && s_id[j] < id)) ? 1 : 0;
        }
        out_ids[(size_t)r * kc + rank] = id;
        out_lp[(size_t)r * kc + rank] = (l == -INFINITY) ? -INFINITY : l - lse;
    }
}

}  // namespace telb

using namespace telb;

// parents [batch, rows] → mask [batch * rows, words], depth [batch, rows] (may be null), positions [batch * rows] (may be null;
// = base_pos[b] + depth + pos_offset).
extern "C" int telb_eagle_tree_meta(const int* parents, const int* base_pos, int* mask, int* depth, int* positions, int batch, int rows,
                                    int words, int depth_base, int pos_offset, cudaStream_t stream) {
    if (batch <= 0 || rows <= 0) return 0;
    if (rows > kMaxTreeNodes) return fail("telb_eagle_tree_meta: at most 128 rows per tree");
    if (words * 32 < rows) return fail("telb_eagle_tree_meta: mask words do not cover the rows");
    if (positions && !base_pos) return fail("telb_eagle_tree_meta: positions need base_pos");
    TELB_LAUNCH("eagle_tree_meta_kernel", eagle_tree_meta_kernel, dim3(batch), dim3(128), 0, stream, parents, base_pos, mask, depth, positions,
                rows, words, depth_base, pos_offset);
    return 0;
}

// Pool arrays are [batch, pool]; outputs [batch, keep + 1] with the root in slot 0.
extern "C" int telb_eagle_select_verify(const float* p_sc, const int* p_tok, const int* p_par, const int* p_dep, const int* root, int batch,
                                        int pool, int keep, int* tree_tok, int* tree_par, int* tree_dep, cudaStream_t stream) {
    if (batch <= 0) return 0;
    if (pool < 1 || pool > kMaxPool) return fail("telb_eagle_select_verify: candidate pool must hold 1..2048 nodes");
    if (keep < 0 || keep > pool || keep + 1 > kMaxTreeNodes) return fail("telb_eagle_select_verify: keep must be 0..min(pool, 127)");
    TELB_LAUNCH("eagle_select_verify_kernel", eagle_select_verify_kernel, dim3(batch), dim3(256), 0, stream, p_sc, p_tok, p_par, p_dep, root,
                pool, keep, tree_tok, tree_par, tree_dep);
    return 0;
}

extern "C" int telb_spec_accept_greedy(const int* target_tokens, const int* tree_tokens, const int* parents, int* path,
                                       int* path_len, int* bonus, int batch, int nodes, int max_path, const int* force_lens,
                                       cudaStream_t stream) {
    if (batch <= 0) return 0;
    if (nodes < 1 || nodes > kMaxTreeNodes) return fail("telb_spec_accept_greedy: tree size must be 1..128");
    if (max_path < 1) return fail("telb_spec_accept_greedy: max_path must be positive");
    TELB_LAUNCH("spec_accept_greedy_kernel", spec_accept_greedy_kernel, dim3(batch), dim3(32), 0, stream, target_tokens, tree_tokens,
                parents, path, path_len, bonus, nodes, max_path, force_lens);
    return 0;
}

// pool: 16-bit [layers, num_pages, 2, hkv, page_size, d]
extern "C" int telb_kv_commit_path(void* pool, const int* page_table, const int* past_len, const int* path, const int* path_len,
                                   int batch, int max_path, int max_pages, int layers, int num_pages, int hkv, int page_size, int d,
                                   cudaStream_t stream) {
    if (batch <= 0 || layers <= 0) return 0;
    if (d != 64 && d != 128 && d != 256) return fail("telb_kv_commit_path: head_dim must be 64, 128 or 256");
    if ((max_path - 1) * (d * 2 / 16) > 1024) return fail("telb_kv_commit_path: accepted path too long for one block");
    const dim3 grid(batch, layers * 2 * hkv), blk(256);
    if (d == 128)
        TELB_LAUNCH("kv_commit_path_kernel", (kv_commit_path_kernel<128>), grid, blk, 0, stream, (uint4*)pool, page_table, past_len, path,
                    path_len, max_path, max_pages, num_pages, hkv, page_size);
    else if (d == 64)
        TELB_LAUNCH("kv_commit_path_kernel", (kv_commit_path_kernel<64>), grid, blk, 0, stream, (uint4*)pool, page_table, past_len, path,
                    path_len, max_path, max_pages, num_pages, hkv, page_size);
    else
        TELB_LAUNCH("kv_commit_path_kernel", (kv_commit_path_kernel<256>), grid, blk, 0, stream, (uint4*)pool, page_table, past_len, path,
                    path_len, max_path, max_pages, num_pages, hkv, page_size);
    return 0;
}

// hidden [rows, H], lm_head [vocab, H] (both fp16 or both bf16), cand [rows, kc] int32 with distinct ids per row →
// out_ids [rows, kc] int32, out_lp [rows, kc] fp32.
extern "C" int telb_candidate_rescore(const void* hidden, const void* lm_head, const int* cand, int* out_ids, float* out_lp, int rows,
                                      int H, int kc, int vocab, int is_bf16, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H % 8 || H > 8192) return fail("telb_candidate_rescore: hidden size must be a multiple of 8, at most 8192");
    if (kc < 1 || kc > 1024) return fail("telb_candidate_rescore: 1..1024 candidates");
    const int smem = (H + 2 * kc) * 4;
    if (is_bf16) TELB_LAUNCH("candidate_rescore_kernel", (candidate_rescore_kernel<__nv_bfloat16>), dim3(rows), dim3(256), smem, stream, (const __nv_bfloat16*)hidden, (const __nv_bfloat16*)lm_head, cand, out_ids, out_lp, H, kc, vocab);
    else TELB_LAUNCH("candidate_rescore_kernel", (candidate_rescore_kernel<__half>), dim3(rows), dim3(256), smem, stream, (const __half*)hidden, (const __half*)lm_head, cand, out_ids, out_lp, H, kc, vocab);
    TELB_CHECK_LAUNCH("candidate_rescore_kernel");
    return 0;
}

// hidden [tokens, H] holds whole blocks of `block` rows; delta [tokens, K, H / group_size]; base [K, H]; residual [tokens, H] or
// null; out [tokens, H].  One 16-bit type throughout; 1 to 4 taps.
extern "C" int telb_dflash2_conv(const void* hidden, const void* delta, const void* base, const void* residual, void* out, int tokens,
                                 int H, int block, int taps, int group_size, int is_bf16, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (taps < 1 || taps > 4) return fail("telb_dflash2_conv: 1 to 4 taps");
    if (block < 1 || tokens % block) return fail("telb_dflash2_conv: rows must be whole blocks");
    if (group_size < 2 || (group_size & 1) || H % group_size) return fail("telb_dflash2_conv: an even group size that divides the hidden size");
    const dim3 grid((H / 2 + 255) / 256, tokens), blk(256);
#define TELB_CONV(TT, KK)                                                                                                           \
    TELB_LAUNCH("dflash2_conv_kernel", (dflash2_conv_kernel<TT, KK>), grid, blk, 0, stream, (const TT*)hidden, (const TT*)delta,    \
                (const TT*)base, (const TT*)residual, (TT*)out, H, block, group_size)
#define TELB_CONV_T(TT)                      \
    do {                                     \
        if (taps == 1) TELB_CONV(TT, 1);     \
        else if (taps == 2) TELB_CONV(TT, 2); \
        else if (taps == 3) TELB_CONV(TT, 3); \
        else TELB_CONV(TT, 4);               \
    } while (0)
    if (is_bf16) TELB_CONV_T(__nv_bfloat16);
    else TELB_CONV_T(__half);
#undef TELB_CONV_T
#undef TELB_CONV
    TELB_CHECK_LAUNCH("dflash2_conv_kernel");
    return 0;
}

// cand / unary [batch, steps, topk], projected [batch, steps, rank], anchor [batch], codebooks [vocab, rank]; temperatures [batch]
// and uniforms [batch, steps] may be null (greedy) → tokens [batch, steps] int32, probs [batch, steps, topk] fp32.
extern "C" int telb_dflash2_selector(const int* cand, const float* unary, const void* projected, const int* anchor, const void* pred_cb,
                                     const void* succ_cb, const float* temperatures, const float* uniforms, int* tokens, float* probs,
                                     int batch, int steps, int topk, int rank, int vocab, int is_bf16, cudaStream_t stream) {
    if (batch <= 0 || steps <= 0) return 0;
    if (topk < 1 || topk > kSelMaxTopK) return fail("telb_dflash2_selector: 1..32 candidates per slot");
    if (rank < 1 || rank > kSelMaxRank) return fail("telb_dflash2_selector: selector rank 1..1024");
    if (temperatures != nullptr && uniforms == nullptr) return fail("telb_dflash2_selector: sampled rows need uniforms");
    const dim3 grid(batch), blk(32 * topk);
    if (is_bf16) TELB_LAUNCH("dflash2_selector_kernel", (dflash2_selector_kernel<__nv_bfloat16>), grid, blk, 0, stream, cand, unary, (const __nv_bfloat16*)projected, anchor, (const __nv_bfloat16*)pred_cb, (const __nv_bfloat16*)succ_cb, temperatures, uniforms, tokens, probs, steps, topk, rank, vocab);
    else TELB_LAUNCH("dflash2_selector_kernel", (dflash2_selector_kernel<__half>), grid, blk, 0, stream, cand, unary, (const __half*)projected, anchor, (const __half*)pred_cb, (const __half*)succ_cb, temperatures, uniforms, tokens, probs, steps, topk, rank, vocab);
    TELB_CHECK_LAUNCH("dflash2_selector_kernel");
    return 0;
}

// cand [batch, steps, topk] int32, transition [batch, steps, topk, topk] fp32; temperatures [batch] and uniforms [batch, steps] may be
// null (greedy) → tokens [batch, steps] int32, probs [batch, steps, topk] fp32.
extern "C" int telb_lattice_chain_walk(const int* cand, const float* transition, const float* temperatures, const float* uniforms,
                                       int* tokens, float* probs, int batch, int steps, int topk, cudaStream_t stream) {
    if (batch <= 0 || steps <= 0) return 0;
    if (topk < 1 || topk > 32) return fail("telb_lattice_chain_walk: 1..32 candidates per slot");
    if (temperatures != nullptr && uniforms == nullptr) return fail("telb_lattice_chain_walk: sampled rows need uniforms");
    TELB_LAUNCH("lattice_chain_walk_kernel", lattice_chain_walk_kernel, dim3(batch), dim3(32), 0, stream, cand, transition, temperatures,
                uniforms, tokens, probs, steps, topk);
    TELB_CHECK_LAUNCH("lattice_chain_walk_kernel");
    return 0;
}

// The whole greedy Markov chain: `steps` launches over logits [batch, steps, vocab] (fp32), then the winners unpacked into
// tokens [batch, steps].  slots is caller-provided scratch of batch * steps u64.  w1 [vocab1, rank], w2 [vocab, rank], 16-bit.
extern "C" int telb_markov_greedy_chain(const float* logits, const void* w1, const void* w2, const int* first_prev,
                                        unsigned long long* slots, int* tokens, int batch, int steps, int vocab, int vocab1, int rank,
                                        int is_bf16, cudaStream_t stream) {
    if (batch <= 0 || steps <= 0) return 0;
    if (rank < 1 || rank > kMarkovMaxRank) return fail("telb_markov_greedy_chain: Markov rank 1..512");
    const size_t smem = (((size_t)batch * rank + 1) & ~size_t(1)) * 4 + (size_t)batch * 8;
    if (smem > 200 * 1024) return fail("telb_markov_greedy_chain: batch * rank too large for one CTA's shared memory");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(markov_greedy_step_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(markov_greedy_step_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return fail("cudaFuncSetAttribute(markov_greedy_step)", e);
        configured = true;
    }
    cudaError_t e = cudaMemsetAsync(slots, 0, (size_t)batch * steps * 8, stream);
    if (e != cudaSuccess) return fail("telb_markov_greedy_chain: memset", e);
    const int rows_per_cta = 256;
    const dim3 grid((vocab + rows_per_cta - 1) / rows_per_cta), blk(kMarkovWarps * 32);
    for (int step = 0; step < steps; ++step) {
        if (is_bf16) TELB_LAUNCH("markov_greedy_step_kernel", (markov_greedy_step_kernel<__nv_bfloat16>), grid, blk, smem, stream, logits, (const __nv_bfloat16*)w1, (const __nv_bfloat16*)w2, first_prev, slots, step, steps, vocab, vocab1, rank, batch, rows_per_cta);
        else TELB_LAUNCH("markov_greedy_step_kernel", (markov_greedy_step_kernel<__half>), grid, blk, smem, stream, logits, (const __half*)w1, (const __half*)w2, first_prev, slots, step, steps, vocab, vocab1, rank, batch, rows_per_cta);
        TELB_CHECK_LAUNCH("markov_greedy_step_kernel");
    }
    TELB_LAUNCH("markov_unpack_kernel", markov_unpack_kernel, dim3((batch * steps + 127) / 128), dim3(128), 0, stream, slots, tokens, batch * steps);
    TELB_CHECK_LAUNCH("markov_unpack_kernel");
    return 0;
}

// Lossless tree acceptance for sampled requests.  probs [batch, nodes, vocab] fp32 rows of the target distribution at every tree
// node; uniforms [batch, max_path, kw] with kw >= 2.
extern "C" int telb_spec_accept_sampling(const float* probs, const int* tree_tokens, const int* parents, const float* uniforms, int* path,
                                         int* path_len, int* bonus, int batch, int nodes, int vocab, int max_path, int kw,
                                         cudaStream_t stream) {
    if (batch <= 0) return 0;
    if (nodes < 1 || max_path < 1 || kw < 2) return fail("telb_spec_accept_sampling: needs a tree, a path bound and at least two uniforms per depth");
    cudaError_t e = cudaMemsetAsync(path, 0, (size_t)batch * max_path * sizeof(int), stream);
    if (e != cudaSuccess) return fail("telb_spec_accept_sampling: memset", e);
    TELB_LAUNCH("spec_accept_sampling_kernel", spec_accept_sampling_kernel, dim3(batch), dim3(kAcceptThreads), 0, stream, probs, tree_tokens,
                parents, uniforms, path, path_len, bonus, nodes, vocab, max_path, kw);
    TELB_CHECK_LAUNCH("spec_accept_sampling_kernel");
    return 0;
}
