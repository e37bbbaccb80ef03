// Speculative-decoding helpers that touch per-sequence trees and the paged KV cache:
//   spec_accept_greedy   walk each sequence's verification tree from the root, following the child whose
//                        token equals the target model's arg-max at the current node; emits the accepted
//                        path, its length and the bonus token.  A forced length per sequence (benchmark
//                        mode, null = off) follows the first child instead of comparing tokens.
//   kv_commit_path       compact the accepted path in the paged cache: the entry written at tree slot
//                        past + path[j] moves to past + j, for every layer / K,V / head, in place.
//
// Reference counterparts: cpp/kernels/speculative/speculativeKernels.cu (acceptGreedy,
// commitSpecTargetKVBatchedKernel :1692), forceAcceptanceKernels.cu.
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

}  // namespace telb

using namespace telb;

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
