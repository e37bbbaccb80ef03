// Pieces shared by the tcgen05 GEMM kernels (16-bit and NVFP4): launch parameters, the persistent
// tile order, and the epilogue that turns an fp32 accumulator row into 16-bit output with the
// optional per-feature scale, bias and residual.
#pragma once

#include "host_utils.h"
#include "nvfp4_common.cuh"
#include "tc5_common.cuh"

namespace telb {

struct GemmParams {
    int rows_a, rows_b, k;
    int splits, kb_per_split, kb_total;
    int tiles_a, tiles_b;
    void* c;
    long long ldc_lane, ldc_col;
    const void* bias;
    const float* alpha;
    const void* residual;
    int feat_on_lane;
    int out_bf16;
    float* ws;
    int* counters;
    int* status;
    // Grouped (mixture-of-experts) mode: 128-row A tile `ta` multiplies the weight block of expert
    // tile_expert[ta] (rows [e * group_rows_b, (e+1) * group_rows_b) of the B tensor); -1 = unused tile.
    // tile_expert[tiles_a + ta] = rows of tile ta that hold routed tokens (the rest is padding and is not stored).
    const int* tile_expert;
    int group_rows_b;
    // Tensor-parallel fusion (both optional, large-M layout only).
    //  reduce-scatter epilogue: output row r belongs to rank d = r / rs_rows_per_rank and is stored into
    //  that rank's partial buffer rs_out[d] (a peer mapping) at row rs_rank * rs_rows_per_rank + (r - d * rpr).
    void* rs_out[8];
    int rs_world, rs_rank, rs_rows_per_rank;
    //  all-gather prologue: rows [o * ag_rows_per_rank, ...) of the A operand were pushed into this GPU's
    //  memory by rank o; the producer waits for ag_flags[o] to reach *ag_epoch before loading them.
    const int* ag_flags;
    const int* ag_epoch;
    int ag_world, ag_rows_per_rank;
    // SwiGLU + NVFP4 output (large-M layout, 128-wide tiles over weights whose gate / up rows alternate in blocks of
    // 64): the epilogue computes silu(gate) * up for the tile's 64 features and stores them quantised — packed codes
    // into sw_xq [rows, sw_ld bytes] and block scales into the atom-layout buffer sw_sf — instead of 16-bit values.
    uint8_t* sw_xq;
    uint8_t* sw_sf;
    const float* sw_gs;
    int sw_ld, sw_k64_pad;
};

// Fusion request as the host passes it (same fields, plain C layout).
struct TelbGemmFusion {
    void* rs_out[8];
    int rs_world, rs_rank, rs_rows_per_rank, pad0;
    const int* ag_flags;
    const int* ag_epoch;
    int ag_world, ag_rows_per_rank;
};

inline void apply_fusion(GemmParams& p, const TelbGemmFusion* f) {
    if (!f) return;
    for (int i = 0; i < 8; ++i) p.rs_out[i] = f->rs_out[i];
    p.rs_world = f->rs_world;
    p.rs_rank = f->rs_rank;
    p.rs_rows_per_rank = f->rs_rows_per_rank;
    p.ag_flags = f->ag_flags;
    p.ag_epoch = f->ag_epoch;
    p.ag_world = f->ag_world;
    p.ag_rows_per_rank = f->ag_rows_per_rank;
}

__device__ __forceinline__ int ld_acquire_sys_s32(const int* ptr) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
    return v;
}

constexpr int kBM = 128;
constexpr int kBK = 64;                       // 64 x 2 B = one 128-byte swizzle atom
constexpr int kATileBytes = kBM * kBK * 2;    // 16 KiB
constexpr int kGemmThreads = 192;
constexpr int kRasterGroup = 8;

// Producer side of the all-gather prologue: block until every rank that owns a row of the tile
// [a0, a0 + 128) has published epoch `e` (bounded; false = gave up, status recorded).  Peers wrote the
// rows with ordinary stores, the tile is read by TMA: the proxy fence orders the two.
__device__ __forceinline__ bool ag_wait_rows(const GemmParams& p, int a0, int e, volatile uint32_t* abort_flag) {
    const int last_row = min(a0 + kBM, p.rows_a) - 1;
    const int o0 = a0 / p.ag_rows_per_rank, o1 = min(last_row / p.ag_rows_per_rank, p.ag_world - 1);
    for (int o = o0; o <= o1; ++o) {
        const uint64_t t0 = global_timer_ns();
        uint32_t it = 0;
        while (ld_acquire_sys_s32(p.ag_flags + o) - e < 0) {
            if ((++it & 63u) == 0) {
                if (*abort_flag) return false;
                if (global_timer_ns() - t0 > kWaitLimitNs) {
                    *abort_flag = 1;
                    if (p.status) atomicCAS(p.status, kStatusOk, kStatusPeerTimeout);
                    return false;
                }
            }
        }
    }
    asm volatile("fence.proxy.async;" ::: "memory");
    return true;
}


struct TileCoord {
    int a0, b0, kb0, kb1, tile, split;
    int brow;      // first row of the B tensor for this tile
    bool skip;     // grouped mode: tile beyond the rows in use
};

__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, int t) {
    TileCoord c;
    c.split = t % p.splits;
    const int tt = t / p.splits;
    const int per_group = kRasterGroup * p.tiles_b;
    const int group = tt / per_group;
    const int within = tt - group * per_group;
    const int gfirst = group * kRasterGroup;
    const int gsize = min(kRasterGroup, p.tiles_a - gfirst);
    const int ta = gfirst + within % gsize;
    const int tb = within / gsize;
    c.tile = tb * p.tiles_a + ta;
    c.a0 = ta * kBM;
    c.kb0 = c.split * p.kb_per_split;
    c.kb1 = min(p.kb_total, c.kb0 + p.kb_per_split);
    c.b0 = tb;   // multiplied by BN by the caller
    c.brow = -1;
    c.skip = false;
    if (p.tile_expert) {
        const int e = p.tile_expert[ta];
        c.skip = e < 0;
        c.brow = e * p.group_rows_b;     // caller adds tb * BN
    }
    return c;
}

// One accumulator row chunk (32 fp32 values of row `row`, columns col0..col0+31) → 16-bit output.
// All register arrays are indexed with compile-time constants only; the common case (a full,
// 16-byte aligned chunk of a row-major output) moves everything with 128-bit accesses.
template <typename T>
__device__ __forceinline__ void epilogue_store(const GemmParams& p, const float (&v)[32], int row, int col0,
                                               int ncols_valid) {
    T* cptr = reinterpret_cast<T*>(p.c);
    const T* rptr = reinterpret_cast<const T*>(p.residual);
    const T* bptr = reinterpret_cast<const T*>(p.bias);
    if (p.ldc_col == 1) {
        T* dst = cptr + row * p.ldc_lane + col0;
        const bool fast = (ncols_valid == 32) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) && ((col0 & 7) == 0);
        if (fast) {
            float o[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = v[j];
            if (p.alpha) {
                const float4* ap = reinterpret_cast<const float4*>(p.alpha + col0);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const float4 a = ap[q];
                    o[4 * q] *= a.x;
                    o[4 * q + 1] *= a.y;
                    o[4 * q + 2] *= a.z;
                    o[4 * q + 3] *= a.w;
                }
            }
            if (bptr) {
                const uint4* bp = reinterpret_cast<const uint4*>(bptr + col0);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint4 b = __ldg(&bp[q]);
                    const T* e = reinterpret_cast<const T*>(&b);
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[8 * q + i] += Cvt<T>::to_f(e[i]);
                }
            }
            if (rptr) {
                const uint4* rp = reinterpret_cast<const uint4*>(rptr + row * p.ldc_lane + col0);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint4 b = rp[q];
                    const T* e = reinterpret_cast<const T*>(&b);
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[8 * q + i] += Cvt<T>::to_f(e[i]);
                }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint4 u;
                u.x = Cvt<T>::pack2(o[q * 8 + 0], o[q * 8 + 1]);
                u.y = Cvt<T>::pack2(o[q * 8 + 2], o[q * 8 + 3]);
                u.z = Cvt<T>::pack2(o[q * 8 + 4], o[q * 8 + 5]);
                u.w = Cvt<T>::pack2(o[q * 8 + 6], o[q * 8 + 7]);
                reinterpret_cast<uint4*>(dst)[q] = u;
            }
            return;
        }
    }
    // general path: per-element, fully unrolled and predicated (no runtime-indexed arrays)
    const float a_lane = (p.alpha && p.feat_on_lane) ? __ldg(&p.alpha[row]) : 1.f;
    const float b_lane = (bptr && p.feat_on_lane) ? Cvt<T>::to_f(bptr[row]) : 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        if (j < ncols_valid) {
            float x = v[j];
            if (p.feat_on_lane) {
                x = x * a_lane + b_lane;
            } else {
                if (p.alpha) x *= p.alpha[col0 + j];
                if (bptr) x += Cvt<T>::to_f(bptr[col0 + j]);
            }
            const long long o = row * p.ldc_lane + (long long)(col0 + j) * p.ldc_col;
            if (rptr) x += Cvt<T>::to_f(rptr[o]);
            cptr[o] = Cvt<T>::from_f(x);
        }
    }
}

// A full 32-column chunk of one accumulator row → 64 bytes of 16-bit output, with the per-column
// scale and bias applied (no residual).  Requires col0 % 8 == 0 and all 32 columns valid.
template <typename T>
__device__ __forceinline__ void pack_chunk(const GemmParams& p, const float (&v)[32], int col0, uint4 (&u)[4]) {
    float o[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) o[j] = v[j];
    if (p.alpha) {
        const float4* ap = reinterpret_cast<const float4*>(p.alpha + col0);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 a = ap[q];
            o[4 * q] *= a.x;
            o[4 * q + 1] *= a.y;
            o[4 * q + 2] *= a.z;
            o[4 * q + 3] *= a.w;
        }
    }
    if (p.bias) {
        const uint4* bp = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.bias) + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 b = __ldg(&bp[q]);
            const T* e = reinterpret_cast<const T*>(&b);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[8 * q + i] += Cvt<T>::to_f(e[i]);
        }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        u[q].x = Cvt<T>::pack2(o[q * 8 + 0], o[q * 8 + 1]);
        u[q].y = Cvt<T>::pack2(o[q * 8 + 2], o[q * 8 + 3]);
        u[q].z = Cvt<T>::pack2(o[q * 8 + 4], o[q * 8 + 5]);
        u[q].w = Cvt<T>::pack2(o[q * 8 + 6], o[q * 8 + 7]);
    }
}

constexpr int kRsStageRowBytes = 144;                        // 64 columns x 2 B + 16 B pad (conflict-free 16 B accesses)
constexpr int kRsStageBytes = 4 * 32 * kRsStageRowBytes;     // one 32-row slab per epilogue warp
constexpr int kAlphaStageBytes = 2 * 256 * 4;                // per-column scales of the current and the next tile

// The epilogue role (warps 2-5, 128 threads): drains finished accumulators from TMEM.  Without
// split-K each thread converts and stores its row.  With split-K it parks the fp32 partial row in
// the workspace; the CTA that arrives last at the tile's counter sums all partials and stores.
template <int BN>
__device__ __forceinline__ void gemm_epilogue_role(const GemmParams& p, uint32_t tmem_base, uint64_t* tfull_bar,
                                                   uint64_t* tempty_bar, volatile uint32_t* abort_flag,
                                                   volatile uint32_t* last_flag, int total_tiles, int acc_stride,
                                                   uint8_t* rs_stage = nullptr, float* s_alpha = nullptr) {
    constexpr int kChunks = (BN + 31) / 32;
    int tile_iter = 0;
    const int kAccStride = acc_stride;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int quad = warp & 3;
    const int lrow = quad * 32 + lane;     // row inside the 128-row tile == TMEM lane
    const int etid = (warp - 2) * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        const TileCoord tc = decode_tile(p, t);
        if (tc.skip) continue;
        const int b0 = tc.b0 * BN;
        GemmParams pt = p;                  // grouped mode: per-expert scale / bias vectors
        if (p.tile_expert && tc.brow > 0) {
            if (p.alpha) pt.alpha = p.alpha + tc.brow;
            if (p.bias) pt.bias = reinterpret_cast<const uint16_t*>(p.bias) + tc.brow;
        }
        if (s_alpha != nullptr && pt.alpha != nullptr && !p.feat_on_lane && p.tile_expert != nullptr) {
            // Grouped (mixture-of-experts) tiles have short K loops, so the epilogue is on the critical path.  The
            // per-column scales of a tile are the same for every row: fetch them once, while the tile's MMAs are still
            // running, instead of as dependent global loads inside every chunk after the accumulator is ready
            // (decode-size expert GEMM with K = 768: 51.7 -> 36.6 us).  Dense GEMMs hide their epilogue behind long K
            // loops and keep the direct loads.
            float* buf = s_alpha + (tile_iter & 1) * 256;
            for (int i = etid; i < BN; i += 128) buf[i] = b0 + i < p.rows_b ? __ldg(&pt.alpha[b0 + i]) : 0.f;
            named_barrier_sync(2, 128);
            pt.alpha = buf - b0;
        }
        ++tile_iter;
        if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, kStatusEpilogueTimeout)) break;
        tc_fence_after_sync();
        const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kAccStride;
        const int row = tc.a0 + lrow;
        bool row_ok = row < p.rows_a;
        // grouped mode: rows past the expert's own rows in this tile are padding, their results are never read
        if (p.tile_expert) row_ok = row_ok && lrow < p.tile_expert[p.tiles_a + tc.a0 / kBM];
        int out_row = row;
        if (p.rs_world > 1 && row_ok) {     // reduce-scatter: this row's partial goes to its owner's buffer
            const int d = row / p.rs_rows_per_rank;
            pt.c = p.rs_out[d];
            out_row = p.rs_rank * p.rs_rows_per_rank + (row - d * p.rs_rows_per_rank);
        }
        if (p.splits == 1 && p.rs_world > 1 && rs_stage != nullptr && BN >= 64) {
            // Reduce-scatter epilogue.  A lane owns a row, but 64-byte pieces of 32 different rows per store
            // make poor use of NVLink: two 32-column chunks are transposed through a per-warp slab of shared
            // memory and leave as whole 128-byte lines, four rows per store instruction.
            uint8_t* slab = rs_stage + quad * (32 * kRsStageRowBytes);
            const int seg = lane & 7, rsub = lane >> 3;
            if constexpr (BN >= 64) {
#pragma unroll 1
                for (int c = 0; c < kChunks; c += 2) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint32_t r[32];
                        tmem_ld_x32(t_addr + (c + h) * 32, r);
                        tmem_ld_wait();
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                        uint4 u[4];
                        const int col0 = min(b0 + (c + h) * 32, max(p.rows_b - 32, 0));   // clamp: columns past N are not stored
                        if (p.out_bf16) pack_chunk<__nv_bfloat16>(pt, v, col0, u);
                        else pack_chunk<__half>(pt, v, col0, u);
                        uint4* dst = reinterpret_cast<uint4*>(slab + lane * kRsStageRowBytes + h * 64);
#pragma unroll
                        for (int q = 0; q < 4; ++q) dst[q] = u[q];
                    }
                    __syncwarp();
                    const int colseg = b0 + c * 32 + seg * 8;           // first of this lane's 8 columns
#pragma unroll
                    for (int rr = 0; rr < 32; rr += 4) {
                        const int lr = rr + rsub;
                        const int grow = tc.a0 + quad * 32 + lr;
                        if (grow < p.rows_a && colseg + 8 <= p.rows_b) {
                            const int d = grow / p.rs_rows_per_rank;
                            const size_t orow = (size_t)p.rs_rank * p.rs_rows_per_rank + (grow - d * p.rs_rows_per_rank);
                            const uint4 val = *reinterpret_cast<const uint4*>(slab + lr * kRsStageRowBytes + seg * 16);
                            uint16_t* base = reinterpret_cast<uint16_t*>(p.rs_out[d]);
                            *reinterpret_cast<uint4*>(base + orow * (size_t)p.ldc_lane + colseg) = val;
                        }
                    }
                    __syncwarp();
                }
            }
            tc_fence_before_sync();
            mbar_arrive(&tempty_bar[acc]);
            // the peer stores of this tile are performed system-wide before the thread moves on, so the
            // "GEMM finished" flag that a later kernel publishes can never overtake them
            __threadfence_system();
        } else if (BN == 128 && p.sw_xq != nullptr && p.splits == 1) {
            if constexpr (BN == 128) {
                // columns [0, 64) of the tile are gate features f0 .. f0+63, columns [64, 128) the matching up features
                const float gs = *p.sw_gs;
                const float inv_gs = 1.f / gs;
                const int f0 = tc.b0 * 64;
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {
                    uint32_t rg[32], ru[32];
                    tmem_ld_x32(t_addr + c * 32, rg);
                    tmem_ld_x32(t_addr + 64 + c * 32, ru);
                    tmem_ld_wait();
                    if (row_ok) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            float y[16];
                            float amax = 0.f;
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const int j = h * 16 + i;
                                float g = __uint_as_float(rg[j]), u = __uint_as_float(ru[j]);
                                if (pt.alpha) {
                                    g *= pt.alpha[b0 + c * 32 + j];
                                    u *= pt.alpha[b0 + 64 + c * 32 + j];
                                }
                                // the same roundings as the unfused chain: 16-bit GEMM output, 16-bit activation, then quantise
                                if (p.out_bf16) {
                                    g = Cvt<__nv_bfloat16>::to_f(Cvt<__nv_bfloat16>::from_f(g));
                                    u = Cvt<__nv_bfloat16>::to_f(Cvt<__nv_bfloat16>::from_f(u));
                                    y[i] = Cvt<__nv_bfloat16>::to_f(Cvt<__nv_bfloat16>::from_f(g / (1.f + __expf(-g)) * u));
                                } else {
                                    g = Cvt<__half>::to_f(Cvt<__half>::from_f(g));
                                    u = Cvt<__half>::to_f(Cvt<__half>::from_f(u));
                                    y[i] = Cvt<__half>::to_f(Cvt<__half>::from_f(g / (1.f + __expf(-g)) * u));
                                }
                                amax = fmaxf(amax, fabsf(y[i]));
                            }
                            uint8_t s8;
                            const uint2 packed = nvfp4_quantize_block16(y, amax, gs, inv_gs, s8);
                            const int blk = (f0 + c * 32 + h * 16) >> 4;
                            *reinterpret_cast<uint2*>(p.sw_xq + (size_t)row * p.sw_ld + blk * 8) = packed;
                            p.sw_sf[sf_atom_offset((long long)row, blk, p.sw_k64_pad)] = s8;
                        }
                    }
                }
            }
            tc_fence_before_sync();
            mbar_arrive(&tempty_bar[acc]);
        } else if (p.splits == 1) {
#pragma unroll 1
            for (int c = 0; c < kChunks; ++c) {
                float v[32];
                if constexpr (BN >= 32) {
                    uint32_t r[32];
                    tmem_ld_x32(t_addr + c * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                } else {
                    uint32_t r[16];
                    tmem_ld_x16(t_addr, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = j < 16 ? __uint_as_float(r[j & 15]) : 0.f;
                }
                const int col0 = b0 + c * 32;
                int nvalid = min(min(32, BN - c * 32), p.rows_b - col0);
                if (row_ok && nvalid > 0) {
                    if (p.out_bf16) epilogue_store<__nv_bfloat16>(pt, v, out_row, col0, nvalid);
                    else epilogue_store<__half>(pt, v, out_row, col0, nvalid);
                }
            }
            tc_fence_before_sync();
            mbar_arrive(&tempty_bar[acc]);
        } else {
            // split-K: park the fp32 partial tile, the last split to arrive reduces all of them
            float* wtile = p.ws + (static_cast<size_t>(tc.tile) * p.splits + tc.split) * (size_t)(BN * kBM);
            float4* wrow = reinterpret_cast<float4*>(wtile + (size_t)lrow * BN);
#pragma unroll 1
            for (int c = 0; c < kChunks; ++c) {
                if constexpr (BN >= 32) {
                    uint32_t r[32];
                    tmem_ld_x32(t_addr + c * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        __stcg(&wrow[c * 8 + j], make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                             __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
                } else {
                    uint32_t r[16];
                    tmem_ld_x16(t_addr, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        __stcg(&wrow[j], make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                     __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
                }
            }
            tc_fence_before_sync();
            mbar_arrive(&tempty_bar[acc]);     // TMEM buffer is free again
            __threadfence();
            named_barrier_sync(1, 128);
            if (etid == 0) {
                const int prev = atomicAdd(&p.counters[tc.tile], 1);
                const bool last = prev == p.splits - 1;
                if (last) p.counters[tc.tile] = 0;     // ready for the next launch / graph replay
                *last_flag = last ? 1u : 0u;
            }
            named_barrier_sync(1, 128);
            const bool is_last = *last_flag != 0;
            if (is_last) {
                __threadfence();
                const float* wbase = p.ws + static_cast<size_t>(tc.tile) * p.splits * (size_t)(BN * kBM);
#pragma unroll 1
                for (int c = 0; c < kChunks; ++c) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0.f;
                    const int ncol = min(32, BN - c * 32);
                    for (int s = 0; s < p.splits; ++s) {
                        const float4* wt = reinterpret_cast<const float4*>(wbase + static_cast<size_t>(s) * (BN * kBM) +
                                                                            (size_t)lrow * BN + c * 32);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            if (j * 4 < ncol) {
                                const float4 f = __ldcg(&wt[j]);
                                v[4 * j] += f.x;
                                v[4 * j + 1] += f.y;
                                v[4 * j + 2] += f.z;
                                v[4 * j + 3] += f.w;
                            }
                        }
                    }
                    const int col0 = b0 + c * 32;
                    int nvalid = min(ncol, p.rows_b - col0);
                    if (row_ok && nvalid > 0) {
                        if (p.out_bf16) epilogue_store<__nv_bfloat16>(pt, v, row, col0, nvalid);
                        else epilogue_store<__half>(pt, v, row, col0, nvalid);
                    }
                }
            }
            named_barrier_sync(1, 128);    // last_flag may be rewritten only after everyone read it
        }
        if (++acc == 2) {
            acc = 0;
            acc_phase ^= 1;
        }
    }
}

// Split counts are chosen so the work-item total fills whole waves of SMs; each extra split costs
// a little in the partial-tile reduction, hence the small penalty.
inline int choose_splits(int tiles, int kb_total, int force_splits) {
    if (force_splits > 0) return force_splits < kb_total ? force_splits : kb_total;
    const int sms = sm_count();
    const int max_s = kb_total / 2 < 16 ? (kb_total / 2 > 0 ? kb_total / 2 : 1) : 16;
    float best = -1.f;
    int splits = 1;
    for (int s = 1; s <= max_s; ++s) {
        const int items = tiles * s;
        const int waves = (items + sms - 1) / sms;
        const float score = (float)items / (float)(waves * sms) - 0.015f * s - 0.01f * waves;
        if (score > best) {
            best = score;
            splits = s;
        }
    }
    return splits;
}

}  // namespace telb
