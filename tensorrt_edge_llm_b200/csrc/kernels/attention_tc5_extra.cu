// The paged tile attention kernel with its optional parts: attention sinks, the skip-softmax tile vote and 256-wide heads.
// The plain head_dim 64 / 128 kernel is attention_tc5.cu; this translation unit expands the same kernel body
// (attention_tc5_kernel.inc) with the extras compiled in and owns the public entry points, which forward to the dense path
// whenever a step needs none of them.  Also here: the split merge for 256-wide heads and the merge that writes NVFP4.
//
// Reference counterparts: attention sinks and sliding windows of the GPT-OSS style families, the Gemma 256-wide heads
// (kernelSrcs/fmha_cutedsl_blackwell/fmha.py head_dim variants) and skip-softmax attention.
#include <type_traits>

#include "host_utils.h"
#include "nvfp4_common.cuh"
#include "tc5_common.cuh"

namespace telb {

struct AttnParams {
    void* out;                 // [T, Hq, D] 16-bit
    float* ws_o;               // [splits, T, Hq, D] fp32 (splits > 1)
    float* ws_lse;             // [splits, T, Hq]    log2-domain log-sum-exp
    const int* q_start;        // [N+1]
    const int* q_len;          // [N]
    const int* past_len;       // [N]
    const int* page_table;     // [N, max_pages]
    const int* tree_mask;      // [T, mask_words] or null
    int mask_words;
    int max_pages, page_size;
    int hq, hkv, group;        // group = hq / hkv
    int tq;                    // query tokens per tile = 128 / group
    int splits;
    int total_tokens;
    int window;                // sliding window, 0 = none, -1 = no causal mask (every row sees every cached and new token)
    float scale_log2;          // softmax scale * log2(e)
    const float* sinks;        // [Hq] fp32 per-head sink logits (natural-log units) joining every row's softmax denominator, or null
    // Skip-softmax (BLASST tile vote): skip_thr[seq] = log2(lambda) of the sequence (lambda = S / length, -inf = dense), or null.
    // A KV tile whose largest score lies more than that below the running maximum for every query row of a warp is not
    // exponentiated (its P rows are zeros); when all four warps vote so, the tile's P·V products are not issued either.
    const float* skip_thr;
    int* skip_stats;           // optional [2]: tiles processed, tiles whose P·V was skipped (diagnostics / tests), or null
    int out_bf16;
    int* status;
};

constexpr int kAttnThreads = 192;
constexpr int kKvTile = 64;
constexpr float kRescaleThreshold = 8.0f;   // log2 units

__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// KVS: depth of the K and V tile rings; MINB: CTAs resident per SM (as in the dense kernel).
#define TELB_ATTN_EXTRA 1
#define TELB_ATTN_KERNEL attn_tc5_extra_kernel
#include "attention_tc5_kernel.inc"
#undef TELB_ATTN_KERNEL
#undef TELB_ATTN_EXTRA

// Merge split partials: out = Σ_s 2^(lse_s - max) O_s / Σ_s 2^(lse_s - max).
// One CTA of D threads per (token, head); splits (<= 32) are weighted by lanes of warp 0 first so
// the D-wide accumulation issues all of its loads independently.
template <int D, typename T>
__global__ void attn_combine_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_lse, T* __restrict__ out,
                                    int total_rows /* T*Hq */, int splits) {
    pdl_prologue();
    __shared__ float w[32];
    const int row = blockIdx.x;
    const int d = threadIdx.x;
    if (threadIdx.x < 32) {
        const float l = threadIdx.x < splits ? ws_lse[(size_t)threadIdx.x * total_rows + row] : -INFINITY;
        float mx = l;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float e = (l == -INFINITY) ? 0.f : exp2f(l - mx);
        float den = e;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        w[threadIdx.x] = den > 0.f ? e / den : 0.f;
    }
    __syncthreads();
    float acc = 0.f;
#pragma unroll 8
    for (int s = 0; s < splits; ++s) acc += w[s] * __ldcg(&ws_o[((size_t)s * total_rows + row) * D + d]);
    out[(size_t)row * D + d] = Cvt<T>::from_f(acc);
}

// The same merge with the result written as NVFP4 (input of the output projection): thread d of row (token, head) holds
// output dim d, so a 16-element block is 16 consecutive lanes.
template <int D, typename T>
__global__ void attn_combine_quant_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_lse, uint8_t* __restrict__ oq,
                                          uint8_t* __restrict__ osf, const float* __restrict__ ogs, int total_rows /* T*Hq */, int hq,
                                          int splits, int k64) {
    pdl_prologue();
    __shared__ float w[32];
    const int row = blockIdx.x;
    const int d = threadIdx.x;
    if (threadIdx.x < 32) {
        const float l = threadIdx.x < splits ? ws_lse[(size_t)threadIdx.x * total_rows + row] : -INFINITY;
        float mx = l;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float e = (l == -INFINITY) ? 0.f : exp2f(l - mx);
        float den = e;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        w[threadIdx.x] = den > 0.f ? e / den : 0.f;
    }
    __syncthreads();
    float acc = 0.f;
#pragma unroll 8
    for (int s = 0; s < splits; ++s) acc += w[s] * __ldcg(&ws_o[((size_t)s * total_rows + row) * D + d]);
    const float gs = *ogs;
    uint8_t s8;
    const uint32_t w4 = nvfp4_quantize_lane16(Cvt<T>::to_f(Cvt<T>::from_f(acc)), gs, 1.f / gs, s8);
    const int tok = row / hq, head = row - tok * hq;
    const int col = head * D + d;
    if ((d & 7) == 0) *reinterpret_cast<uint32_t*>(oq + (size_t)tok * (hq * D / 2) + col / 2) = w4;
    if ((d & 15) == 0) osf[sf_atom_offset((long long)tok, col >> 4, k64)] = s8;
}

template <int D, typename T, int KVS, int MINB>
static int launch_attn_extra(const CUtensorMap& tq, const CUtensorMap& tkv, const AttnParams& p, int qtiles, int nseq, cudaStream_t stream) {
    constexpr int smem = 128 * D * 2 + 2 * KVS * kKvTile * D * 2 + 2 * 128 * kKvTile * 2 + 1024 + 512;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc5_extra_kernel<D, T, KVS, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail("cudaFuncSetAttribute(attn_tc5_extra)", e);
        configured = true;
    }
    dim3 grid(qtiles, p.hkv, nseq * p.splits);
    TELB_LAUNCH("attn_tc5_extra_kernel", (attn_tc5_extra_kernel<D, T, KVS, MINB>), dim3(grid), dim3(kAttnThreads), smem, stream, tq, tkv, p);
    TELB_CHECK_LAUNCH("attn_tc5_extra_kernel");
    if (p.splits > 1) {
        const int rows = p.total_tokens * p.hq;
        TELB_LAUNCH("attn_combine_kernel", (attn_combine_kernel<D, T>), dim3(rows), dim3(D), 0, stream, p.ws_o, p.ws_lse, reinterpret_cast<T*>(p.out), rows, p.splits);
        TELB_CHECK_LAUNCH("attn_combine_kernel");
    }
    return 0;
}

template <int D, typename T>
static int launch_attn(const CUtensorMap& tq, const CUtensorMap& tkv, const AttnParams& p, int qtiles, int nseq, cudaStream_t stream) {
    // 256-wide heads (Gemma family): the Q tile alone is 64 KB and O takes 256 TMEM columns, so one CTA per SM with
    // single-stage K / V rings is the only shape that fits; narrower heads run two CTAs per SM
    if constexpr (D > 128) return launch_attn_extra<D, T, 1, 1>(tq, tkv, p, qtiles, nseq, stream);
    return launch_attn_extra<D, T, 1, 2>(tq, tkv, p, qtiles, nseq, stream);
}

}  // namespace telb

using namespace telb;

extern "C" int telb_attn_combine_dense(const float* ws_o, const float* ws_lse, void* out, int rows, int splits, int d, int is_bf16,
                                       cudaStream_t stream);
extern "C" int telb_paged_attention_dense(const void* q, const void* kv_layer, void* out, const int* q_start, const int* q_len,
                                          const int* past_len, const int* page_table, const int* tree_mask, int mask_words,
                                          int num_seqs, int total_tokens, int max_q_len, int num_pages, int max_pages, int page_size,
                                          int hq, int hkv, int d, float scale, int window, int splits, float* ws, long long ws_floats,
                                          int is_bf16, int* status, cudaStream_t stream);

// Merge `splits` partial results (ws_o [splits, rows, d] fp32, ws_lse [splits, rows]) into out [rows, d].
extern "C" int telb_attn_combine(const float* ws_o, const float* ws_lse, void* out, int rows, int splits, int d, int is_bf16,
                                 cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (d != 256) return telb_attn_combine_dense(ws_o, ws_lse, out, rows, splits, d, is_bf16, stream);
    if (is_bf16) TELB_LAUNCH("attn_combine_kernel", (attn_combine_kernel<256, __nv_bfloat16>), dim3(rows), dim3(256), 0, stream, ws_o, ws_lse, (__nv_bfloat16*)out, rows, splits);
    else TELB_LAUNCH("attn_combine_kernel", (attn_combine_kernel<256, __half>), dim3(rows), dim3(256), 0, stream, ws_o, ws_lse, (__half*)out, rows, splits);
    TELB_CHECK_LAUNCH("attn_combine_kernel");
    return 0;
}

extern "C" int telb_nvfp4_k64_pad(int k);

// The merge with an NVFP4 result: packed codes oq [tokens, hq * d / 2] and atom-layout scales osf over hq * d columns.
extern "C" int telb_attn_combine_quant(const float* ws_o, const float* ws_lse, void* oq, void* osf, const float* ogs, int tokens, int hq,
                                       int splits, int d, int is_bf16, cudaStream_t stream) {
    const int rows = tokens * hq;
    if (rows <= 0) return 0;
    if (d != 128) return fail("telb_attn_combine_quant: head_dim must be 128");
    if (splits > 32) return fail("telb_attn_combine_quant: at most 32 splits");
    const int k64 = telb_nvfp4_k64_pad(hq * d);
    if (is_bf16) TELB_LAUNCH("attn_combine_quant_kernel", (attn_combine_quant_kernel<128, __nv_bfloat16>), dim3(rows), dim3(128), 0, stream, ws_o, ws_lse, (uint8_t*)oq, (uint8_t*)osf, ogs, rows, hq, splits, k64);
    else TELB_LAUNCH("attn_combine_quant_kernel", (attn_combine_quant_kernel<128, __half>), dim3(rows), dim3(128), 0, stream, ws_o, ws_lse, (uint8_t*)oq, (uint8_t*)osf, ogs, rows, hq, splits, k64);
    TELB_CHECK_LAUNCH("attn_combine_quant_kernel");
    return 0;
}

// q [T,Hq,D], kv_layer [pages,2,Hkv,P,D], out [T,Hq,D]; metadata as in the ragged step ABI.
// ws must hold splits*T*Hq*(D+1) floats when splits > 1 (pass splits = 1 to avoid scratch).
extern "C" int telb_paged_attention(const void* q, const void* kv_layer, void* out, const int* q_start,
                                    const int* q_len, const int* past_len, const int* page_table,
                                    const int* tree_mask, int mask_words, int num_seqs, int total_tokens,
                                    int max_q_len, int num_pages, int max_pages, int page_size, int hq, int hkv, int d,
                                    float scale, int window, int splits, float* ws, long long ws_floats, int is_bf16,
                                    int* status, const float* sinks, const float* skip_thr, int* skip_stats, cudaStream_t stream) {
    if (num_seqs <= 0 || total_tokens <= 0) return 0;
    if (sinks == nullptr && skip_thr == nullptr && d != 256)
        return telb_paged_attention_dense(q, kv_layer, out, q_start, q_len, past_len, page_table, tree_mask, mask_words, num_seqs,
                                          total_tokens, max_q_len, num_pages, max_pages, page_size, hq, hkv, d, scale, window, splits,
                                          ws, ws_floats, is_bf16, status, stream);
    if (d != 64 && d != 128 && d != 256) return fail("telb_paged_attention: head_dim must be 64, 128 or 256");
    if (page_size != 64 && page_size != 128) return fail("telb_paged_attention: page size must be 64 or 128");
    if (hq % hkv) return fail("telb_paged_attention: Hq must be a multiple of Hkv");
    const int group = hq / hkv;
    if (group > 128 || (128 % group)) return fail("telb_paged_attention: GQA ratio must divide 128");
    AttnParams p{};
    p.out = out;
    p.q_start = q_start;
    p.q_len = q_len;
    p.past_len = past_len;
    p.page_table = page_table;
    p.tree_mask = tree_mask;
    p.mask_words = mask_words;
    p.max_pages = max_pages;
    p.page_size = page_size;
    p.hq = hq;
    p.hkv = hkv;
    p.group = group;
    p.tq = 128 / group;
    p.total_tokens = total_tokens;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.out_bf16 = is_bf16;
    p.sinks = sinks;
    p.skip_thr = skip_thr;
    p.skip_stats = skip_stats;
    p.status = status;
    if (splits < 1) splits = 1;
    while (splits > 1 && (long long)splits * total_tokens * hq * (d + 1) > ws_floats) --splits;
    p.splits = splits;
    p.ws_o = ws;
    p.ws_lse = ws ? ws + (size_t)splits * total_tokens * hq * d : nullptr;
    const int qtiles = (max_q_len + p.tq - 1) / p.tq;
    const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap tq, tkv;
    {
        const uint64_t dims[3] = {(uint64_t)d, (uint64_t)hq, (uint64_t)total_tokens};
        const uint64_t strides[2] = {(uint64_t)d * 2, (uint64_t)hq * d * 2};
        const uint32_t box[3] = {64, (uint32_t)group, (uint32_t)p.tq};
        if (make_tmap_nd(&tq, dt, 3, q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    }
    {
        const uint64_t rows = (uint64_t)num_pages * 2 * hkv * page_size;
        if (make_tmap_2d(&tkv, dt, 2, kv_layer, rows, d, (uint64_t)d * 2, kKvTile, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    }
    if (d == 128) {
        if (is_bf16) return launch_attn<128, __nv_bfloat16>(tq, tkv, p, qtiles, num_seqs, stream);
        return launch_attn<128, __half>(tq, tkv, p, qtiles, num_seqs, stream);
    }
    if (d == 256) {
        if (is_bf16) return launch_attn<256, __nv_bfloat16>(tq, tkv, p, qtiles, num_seqs, stream);
        return launch_attn<256, __half>(tq, tkv, p, qtiles, num_seqs, stream);
    }
    if (is_bf16) return launch_attn<64, __nv_bfloat16>(tq, tkv, p, qtiles, num_seqs, stream);
    return launch_attn<64, __half>(tq, tkv, p, qtiles, num_seqs, stream);
}
