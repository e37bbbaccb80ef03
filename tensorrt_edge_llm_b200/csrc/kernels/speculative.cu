// Speculative-decoding helpers that touch per-sequence trees and the paged KV cache:
//   spec_accept_greedy   walk each sequence's verification tree from the root, following the child whose
//                        token equals the target model's arg-max at the current node; emits the accepted
//                        path, its length and the bonus token.  A forced length per sequence (benchmark
//                        mode, null = off) follows the first child instead of comparing tokens.
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
// Reference counterparts: cpp/kernels/speculative/speculativeKernels.cu (acceptGreedy, the tree construction
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
