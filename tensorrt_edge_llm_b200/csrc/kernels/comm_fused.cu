// Tensor-parallel collectives fused with the work that follows them, over peer memory
// (NVLink / NVSwitch).  Buffers live in symmetric memory: every rank allocates the same layout
// and maps all peers' copies, so a kernel can store to or load from any rank with plain
// pointers.  No TMA and no cluster multicast is used on peer memory here.
//
//   ar_add_rmsnorm   one-shot all-reduce of the row-parallel GEMM output, fused with the residual
//                    add, RMSNorm and (optionally) NVFP4 quantisation of the next GEMM's input.
//                    Decode-size messages (rows <= 256): latency-bound, every rank reads the
//                    partial rows of all peers directly.
//
// Synchronisation is per row: a CTA publishes its partial row into its own symmetric buffer,
// then stores an epoch value into the flag slot it owns on every peer (st.release.sys) and polls
// its local slots (ld.acquire.sys) until all peers have published the same epoch.  Epochs are kept
// in device memory per row, so the kernel can be replayed from a CUDA graph.  Two partial buffers
// alternate with the epoch parity; a rank can only be two calls ahead after every peer has entered
// the call in between, so a buffer is never overwritten while a peer still reads it.  Every spin
// is bounded: on expiry the CTA records kStatusPeerTimeout and finishes the row with what it has.
//
// Reference counterpart: AllReducePlugin → ncclAllReduce followed by a separate norm
// (cpp/plugins/allReducePlugin/allReducePlugin.cpp:96-110); nothing in the reference fuses them.
#include "host_utils.h"
#include "nvfp4_common.cuh"

namespace telb {

constexpr int kMaxRanks = 8;
constexpr int kMaxHidden = 16384;       // 4 units x 256 threads x 16 elements

struct ArParams {
    const void* x;                       // this rank's partial [rows, hidden] (local)
    void* sym_partial[kMaxRanks];        // symmetric partial buffers of every rank: [2][max_rows][hidden]
    int* sym_flags[kMaxRanks];           // symmetric flag arrays of every rank:   [2][kMaxRanks][max_rows]
    int* row_epoch;                      // local [max_rows]
    const void* residual;                // local [rows, hidden] or null
    const void* weight;                  // [hidden]
    void* res_out;                       // local [rows, hidden] (sum + residual) or null
    void* y_out;                         // local normalised output (16-bit) or null
    uint8_t* xq;                         // NVFP4 output or null
    uint8_t* sf;
    const float* quant_scale;
    int rank, world, rows, hidden, max_rows, k64_pad;
    float eps;
    int* status;
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_peer_v4(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// One CTA per row; thread t owns 16-element blocks t, t + blockDim, ... (kUnits per thread).
template <typename T, int kUnits>
__global__ void ar_add_rmsnorm_kernel(ArParams p) {
    __shared__ float red[32];
    __shared__ int s_ok;
    pdl_prologue();
    const int row = blockIdx.x;
    const int nunits = p.hidden / 16;
    const int e = p.row_epoch[row] + 1;
    const int par = e & 1;
    T* my_buf = reinterpret_cast<T*>(p.sym_partial[p.rank]) + ((size_t)par * p.max_rows + row) * p.hidden;

    // 1. publish my partial row
    float v[kUnits][16];
#pragma unroll
    for (int u = 0; u < kUnits; ++u) {
        const int idx = threadIdx.x + u * blockDim.x;
        if (idx < nunits) {
            const T* src = reinterpret_cast<const T*>(p.x) + (size_t)row * p.hidden + idx * 16;
            const uint4 a0 = reinterpret_cast<const uint4*>(src)[0], a1 = reinterpret_cast<const uint4*>(src)[1];
            reinterpret_cast<uint4*>(my_buf + idx * 16)[0] = a0;
            reinterpret_cast<uint4*>(my_buf + idx * 16)[1] = a1;
            const T* e0 = reinterpret_cast<const T*>(&a0);
            const T* e1 = reinterpret_cast<const T*>(&a1);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[u][i] = Cvt<T>::to_f(e0[i]);
                v[u][8 + i] = Cvt<T>::to_f(e1[i]);
            }
        }
    }
    __threadfence_system();
    __syncthreads();
    // 2. tell every peer, then wait for every peer (bounded)
    if (threadIdx.x < p.world && threadIdx.x != p.rank)
        st_release_sys(p.sym_flags[threadIdx.x] + ((size_t)par * kMaxRanks + p.rank) * p.max_rows + row, e);
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < p.world && threadIdx.x != p.rank) {
        const int* f = p.sym_flags[p.rank] + ((size_t)par * kMaxRanks + threadIdx.x) * p.max_rows + row;
        const uint64_t t0 = global_timer_ns();
        uint32_t it = 0;
        while (ld_acquire_sys(f) - e < 0) {           // wrap-safe "flag < epoch"
            if ((++it & 255u) == 0 && global_timer_ns() - t0 > kWaitLimitNs) {
                atomicCAS(p.status, kStatusOk, kStatusPeerTimeout);
                s_ok = 0;
                break;
            }
        }
    }
    __syncthreads();
    // 3. sum the peers' rows (fp32), in rank order so every rank computes bit-identical sums
    if (s_ok) {
#pragma unroll
        for (int u = 0; u < kUnits; ++u) {
            const int idx = threadIdx.x + u * blockDim.x;
            if (idx < nunits) {
                // every peer's 32 bytes are requested before any of them is consumed: the NVLink round trips overlap
                uint4 pa[kMaxRanks], pb[kMaxRanks];
#pragma unroll
                for (int r = 0; r < kMaxRanks; ++r) {
                    if (r < p.world && r != p.rank) {
                        const T* src = reinterpret_cast<const T*>(p.sym_partial[r]) + ((size_t)par * p.max_rows + row) * p.hidden + idx * 16;
                        pa[r] = ld_peer_v4(src);
                        pb[r] = ld_peer_v4(src + 8);
                    }
                }
                float acc[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[i] = 0.f;
#pragma unroll
                for (int r = 0; r < kMaxRanks; ++r) {
                    if (r >= p.world) continue;
                    if (r == p.rank) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) acc[i] += v[u][i];
                    } else {
                        const T* e0 = reinterpret_cast<const T*>(&pa[r]);
                        const T* e1 = reinterpret_cast<const T*>(&pb[r]);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            acc[i] += Cvt<T>::to_f(e0[i]);
                            acc[8 + i] += Cvt<T>::to_f(e1[i]);
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) v[u][i] = acc[i];
            }
        }
    }
    // 4. residual add (rounded to the activation type), RMSNorm, optional quantisation
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < kUnits; ++u) {
        const int idx = threadIdx.x + u * blockDim.x;
        if (idx < nunits) {
            T o[16];
            if (p.residual) {
                const T* rs = reinterpret_cast<const T*>(p.residual) + (size_t)row * p.hidden + idx * 16;
                const uint4 r0 = reinterpret_cast<const uint4*>(rs)[0], r1 = reinterpret_cast<const uint4*>(rs)[1];
                const T* f0 = reinterpret_cast<const T*>(&r0);
                const T* f1 = reinterpret_cast<const T*>(&r1);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    // the reduced projection is rounded once, like an all-reduce result in 16 bits
                    o[i] = Cvt<T>::from_f(Cvt<T>::to_f(Cvt<T>::from_f(v[u][i])) + Cvt<T>::to_f(f0[i]));
                    o[8 + i] = Cvt<T>::from_f(Cvt<T>::to_f(Cvt<T>::from_f(v[u][8 + i])) + Cvt<T>::to_f(f1[i]));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) o[i] = Cvt<T>::from_f(v[u][i]);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                v[u][i] = Cvt<T>::to_f(o[i]);
                ss += v[u][i] * v[u][i];
            }
            if (p.res_out) {
                T* dst = reinterpret_cast<T*>(p.res_out) + (size_t)row * p.hidden + idx * 16;
                reinterpret_cast<uint4*>(dst)[0] = *reinterpret_cast<uint4*>(&o[0]);
                reinterpret_cast<uint4*>(dst)[1] = *reinterpret_cast<uint4*>(&o[8]);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) red[wid] = ss;
    __syncthreads();
    float tot = lane < nw ? red[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    const float inv = rsqrtf(tot / p.hidden + p.eps);
    const float gs = p.quant_scale ? *p.quant_scale : 1.f;
    const float inv_gs = 1.f / gs;
    if (p.weight) {
#pragma unroll
        for (int u = 0; u < kUnits; ++u) {
            const int idx = threadIdx.x + u * blockDim.x;
            if (idx < nunits) {
                const T* wp = reinterpret_cast<const T*>(p.weight) + idx * 16;
                const uint4 w0 = reinterpret_cast<const uint4*>(wp)[0], w1 = reinterpret_cast<const uint4*>(wp)[1];
                const T* g0 = reinterpret_cast<const T*>(&w0);
                const T* g1 = reinterpret_cast<const T*>(&w1);
                float y[16];
                T yo[16];
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float n = Cvt<T>::to_f(Cvt<T>::from_f(v[u][i] * inv));
                    yo[i] = Cvt<T>::from_f(n * Cvt<T>::to_f(i < 8 ? g0[i] : g1[i - 8]));
                    y[i] = Cvt<T>::to_f(yo[i]);
                    amax = fmaxf(amax, fabsf(y[i]));
                }
                if (p.y_out) {
                    T* dst = reinterpret_cast<T*>(p.y_out) + (size_t)row * p.hidden + idx * 16;
                    reinterpret_cast<uint4*>(dst)[0] = *reinterpret_cast<uint4*>(&yo[0]);
                    reinterpret_cast<uint4*>(dst)[1] = *reinterpret_cast<uint4*>(&yo[8]);
                }
                if (p.xq) {
                    uint8_t s8;
                    const uint2 packed = nvfp4_quantize_block16(y, amax, gs, inv_gs, s8);
                    *reinterpret_cast<uint2*>(p.xq + (size_t)row * (p.hidden / 2) + idx * 8) = packed;
                    p.sf[sf_atom_offset(row, idx, p.k64_pad)] = s8;
                }
            }
        }
    }
    if (threadIdx.x == 0) p.row_epoch[row] = e;
}


// ---- reduce-scatter → residual add → RMSNorm (→ NVFP4) → all-gather ---------------------------------
// Prefill-size messages.  The row-parallel GEMM before this kernel stored every output row straight
// into its owner's partial buffer (reduce-scatter epilogue, peer stores); here the owner of a row
//   1. learns that every rank's GEMM has finished (flag per source rank),
//   2. sums the `world` partial rows in rank order (local reads), adds its shard of the residual
//      stream (which stays token-sharded between layers) and normalises,
//   3. pushes the normalised row — 16-bit, or NVFP4 values + scale bytes — into the gathered
//      activation buffer of every rank (peer stores), and
//   4. the last CTA of the grid publishes "my shard is gathered" to every rank.
// The consuming GEMM waits for those flags in its TMA producer (all-gather prologue); with
// `wait_gather` set the last CTA waits for them itself, so any later kernel may read the buffer.
struct RsAgParams {
    const void* partial;                 // local [world][rows_per_rank][hidden]
    int* gemm_flags[kMaxRanks];          // every rank's "GEMM finished" flags [world]
    int* ag_flags[kMaxRanks];            // every rank's "shard gathered" flags [world]
    int* epoch;                          // local: number of completed calls
    int* ticket;                         // local: CTA arrival counter (0 between calls)
    const void* residual;                // local shard [rows_local, hidden], or all rows when residual_full
    int residual_full;
    const void* weight;
    void* res_out;                       // local shard [rows_local, hidden]
    void* gather_y[kMaxRanks];           // every rank's gathered 16-bit activations [rows, hidden] (or null)
    uint8_t* gather_xq[kMaxRanks];       // every rank's gathered NVFP4 activations [rows, hidden / 2] (or null)
    uint8_t* gather_sf[kMaxRanks];
    const float* quant_scale;
    int rank, world, rows, rows_per_rank, hidden, k64_pad, wait_gather;
    // partial slots summed: [slot_base, slot_base + sum_slots).  A single local slot (an expert-parallel MoE block already
    // delivered complete rows for this rank's tokens) needs no "GEMM finished" handshake.
    int sum_slots, slot_base;
    float eps;
    int* status;
};

__device__ __forceinline__ bool wait_flag_ge(const int* f, int e, int* status) {
    const uint64_t t0 = global_timer_ns();
    uint32_t it = 0;
    while (ld_acquire_sys(f) - e < 0) {
        if ((++it & 255u) == 0 && global_timer_ns() - t0 > kWaitLimitNs) {
            atomicCAS(status, kStatusOk, kStatusPeerTimeout);
            return false;
        }
    }
    return true;
}

template <typename T, int kUnits>
__global__ void rs_add_rmsnorm_ag_kernel(RsAgParams p) {
    __shared__ float red[32];
    __shared__ int s_ok, s_last;
    // one row of NVFP4 output staged for the push: packed codes (hidden / 2 bytes) and scale bytes (hidden / 16)
    __shared__ uint4 s_codes[kMaxHidden / 32];
    __shared__ uint32_t s_sf4[kMaxHidden / 64];
    pdl_prologue();
    const int rows_local = max(0, min(p.rows_per_rank, p.rows - p.rank * p.rows_per_rank));
    const int nunits = p.hidden / 16;
    const int e = *p.epoch + 1;
    const bool has_rows = (int)blockIdx.x < rows_local;

    // 1. my GEMM has finished (this kernel runs after it): tell every rank; then wait for theirs
    if (blockIdx.x == 0 && threadIdx.x < p.world) st_release_sys(p.gemm_flags[threadIdx.x] + p.rank, e);
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (has_rows && p.sum_slots > 1 && threadIdx.x < p.world && threadIdx.x != p.rank) {
        if (!wait_flag_ge(p.gemm_flags[p.rank] + threadIdx.x, e, p.status)) s_ok = 0;
    }
    __syncthreads();

    // A CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ...: the flag handshake above and the system-scope fence below
    // (a round trip over the link) are paid once per CTA, not once per row.
    float v[kUnits][16];
    for (int row = blockIdx.x; row < rows_local; row += gridDim.x) {
        const int grow = p.rank * p.rows_per_rank + row;     // global row
        // 2. sum the partial rows in rank order
#pragma unroll
        for (int u = 0; u < kUnits; ++u) {
            const int idx = threadIdx.x + u * blockDim.x;
            if (idx < nunits) {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[u][i] = 0.f;
                for (int r = p.slot_base; r < p.slot_base + p.sum_slots; ++r) {
                    const T* src = reinterpret_cast<const T*>(p.partial) + ((size_t)r * p.rows_per_rank + row) * p.hidden + idx * 16;
                    const uint4 a0 = __ldcg(reinterpret_cast<const uint4*>(src)), a1 = __ldcg(reinterpret_cast<const uint4*>(src) + 1);
                    const T* e0 = reinterpret_cast<const T*>(&a0);
                    const T* e1 = reinterpret_cast<const T*>(&a1);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        v[u][i] += Cvt<T>::to_f(e0[i]);
                        v[u][8 + i] += Cvt<T>::to_f(e1[i]);
                    }
                }
            }
        }
        // residual add (the reduced projection is rounded once, like a 16-bit all-reduce result)
        float ss = 0.f;
        const size_t rrow = p.residual_full ? (size_t)grow : (size_t)row;
#pragma unroll
        for (int u = 0; u < kUnits; ++u) {
            const int idx = threadIdx.x + u * blockDim.x;
            if (idx < nunits) {
                T o[16];
                if (p.residual) {
                    const T* rs = reinterpret_cast<const T*>(p.residual) + rrow * p.hidden + idx * 16;
                    const uint4 r0 = reinterpret_cast<const uint4*>(rs)[0], r1 = reinterpret_cast<const uint4*>(rs)[1];
                    const T* f0 = reinterpret_cast<const T*>(&r0);
                    const T* f1 = reinterpret_cast<const T*>(&r1);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        o[i] = Cvt<T>::from_f(Cvt<T>::to_f(Cvt<T>::from_f(v[u][i])) + Cvt<T>::to_f(f0[i]));
                        o[8 + i] = Cvt<T>::from_f(Cvt<T>::to_f(Cvt<T>::from_f(v[u][8 + i])) + Cvt<T>::to_f(f1[i]));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = Cvt<T>::from_f(v[u][i]);
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    v[u][i] = Cvt<T>::to_f(o[i]);
                    ss += v[u][i] * v[u][i];
                }
                if (p.res_out) {
                    T* dst = reinterpret_cast<T*>(p.res_out) + (size_t)row * p.hidden + idx * 16;
                    reinterpret_cast<uint4*>(dst)[0] = *reinterpret_cast<uint4*>(&o[0]);
                    reinterpret_cast<uint4*>(dst)[1] = *reinterpret_cast<uint4*>(&o[8]);
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
        if (lane == 0) red[wid] = ss;
        __syncthreads();
        float tot = lane < nw ? red[lane] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
        const float inv = p.weight ? rsqrtf(tot / p.hidden + p.eps) : 1.f;
        const float gs = p.quant_scale ? *p.quant_scale : 1.f;
        const float inv_gs = 1.f / gs;
        const bool vec_push = (p.hidden % 64) == 0;
        // 3. normalise and push the row to every rank
#pragma unroll
        for (int u = 0; u < kUnits; ++u) {
            const int idx = threadIdx.x + u * blockDim.x;
            if (idx < nunits) {
                float y[16];
                T yo[16];
                float amax = 0.f;
                if (p.weight) {
                    const T* wp = reinterpret_cast<const T*>(p.weight) + idx * 16;
                    const uint4 w0 = reinterpret_cast<const uint4*>(wp)[0], w1 = reinterpret_cast<const uint4*>(wp)[1];
                    const T* g0 = reinterpret_cast<const T*>(&w0);
                    const T* g1 = reinterpret_cast<const T*>(&w1);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float n = Cvt<T>::to_f(Cvt<T>::from_f(v[u][i] * inv));
                        yo[i] = Cvt<T>::from_f(n * Cvt<T>::to_f(i < 8 ? g0[i] : g1[i - 8]));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) yo[i] = Cvt<T>::from_f(v[u][i]);
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    y[i] = Cvt<T>::to_f(yo[i]);
                    amax = fmaxf(amax, fabsf(y[i]));
                }
                if (p.gather_y[0]) {
                    const uint4 q0 = *reinterpret_cast<uint4*>(&yo[0]), q1 = *reinterpret_cast<uint4*>(&yo[8]);
                    for (int r = 0; r < p.world; ++r) {
                        T* dst = reinterpret_cast<T*>(p.gather_y[r]) + (size_t)grow * p.hidden + idx * 16;
                        reinterpret_cast<uint4*>(dst)[0] = q0;
                        reinterpret_cast<uint4*>(dst)[1] = q1;
                    }
                }
                if (p.gather_xq[0]) {
                    uint8_t s8;
                    const uint2 packed = nvfp4_quantize_block16(y, amax, gs, inv_gs, s8);
                    if (vec_push) {
                        reinterpret_cast<uint2*>(s_codes)[idx] = packed;
                        reinterpret_cast<uint8_t*>(s_sf4)[idx] = s8;
                    } else {
                        const size_t sfo = sf_atom_offset(grow, idx, p.k64_pad);
                        for (int r = 0; r < p.world; ++r) {
                            *reinterpret_cast<uint2*>(p.gather_xq[r] + (size_t)grow * (p.hidden / 2) + idx * 8) = packed;
                            p.gather_sf[r][sfo] = s8;
                        }
                    }
                }
            }
        }
        if (p.gather_xq[0] && vec_push) {
            // The quantised row leaves as 16-byte code stores and 4-byte scale stores (the four scales of 64 consecutive
            // inputs are adjacent in the atom layout), consecutive threads on consecutive addresses of one peer, all peers
            // in flight at once — not one 8-byte and one 1-byte store per block and peer in a serial loop.
            __syncthreads();
            const int nchunk = p.hidden / 32, nsf = p.hidden / 64, per_peer = nchunk + nsf;
            for (int i = threadIdx.x; i < p.world * per_peer; i += blockDim.x) {
                const int r = i / per_peer, j = i - r * per_peer;
                if (j < nchunk)
                    *reinterpret_cast<uint4*>(p.gather_xq[r] + (size_t)grow * (p.hidden / 2) + (size_t)j * 16) = s_codes[j];
                else
                    *reinterpret_cast<uint32_t*>(p.gather_sf[r] + sf_atom_offset(grow, (j - nchunk) * 4, p.k64_pad)) = s_sf4[j - nchunk];
            }
        }
        __syncthreads();          // red[] and the staged row are reused by the next row
    }
    // 4. the last CTA publishes this rank's shard
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(p.ticket, 1) == (int)gridDim.x - 1;
    __syncthreads();
    if (s_last) {
        __threadfence_system();
        if (threadIdx.x < p.world) st_release_sys(p.ag_flags[threadIdx.x] + p.rank, e);
        if (p.wait_gather && threadIdx.x < p.world && threadIdx.x != p.rank)
            wait_flag_ge(p.ag_flags[p.rank] + threadIdx.x, e, p.status);
        __syncthreads();
        if (threadIdx.x == 0) {
            *p.ticket = 0;
            *p.epoch = e;
        }
    }
}

// ---- vocabulary-sharded greedy pick ----------------------------------------------------------------
// Each rank holds the logits of its vocabulary shard only.  Instead of gathering [rows, vocab] logits on
// every rank, a rank finds the best (value, index) of its shard per row (arg-max kernel), packs it into an
// order-preserving 64-bit key with the *global* token id, stores the key into every peer's table (one
// 8-byte peer store per row and peer), publishes an epoch flag and, once all peers' flags have arrived,
// takes the maximum over the `world` keys of each row.  Ties resolve to the lower global id, the same
// answer as an arg-max over the gathered logits.  world * rows * 8 bytes cross NVLink instead of
// rows * vocab * 2.  Tables alternate with the epoch parity, like the all-reduce buffers above.
struct ArgmaxMergeParams {
    const void* logits;                  // local shard [rows, vocab_local], row pitch `stride`
    const int* local_idx;                // [rows] arg-max within the shard
    unsigned long long* sym_keys[kMaxRanks];   // every rank's table [2][kMaxRanks][max_rows]
    int* sym_flags[kMaxRanks];           // every rank's flags [2][kMaxRanks]
    int* epoch;                          // local: completed calls
    int* out;                            // [rows] global token ids
    long long stride;
    int rank, world, rows, max_rows, vocab_local, dtype;
    int* status;
};

__global__ void argmax_merge_kernel(ArgmaxMergeParams p) {
    __shared__ int s_ok;
    pdl_prologue();
    const int e = *p.epoch + 1;
    const int par = e & 1;
    const int row = threadIdx.x;
    if (row < p.rows) {
        const int li = p.local_idx[row];
        float v;
        if (p.dtype == 2) v = reinterpret_cast<const float*>(p.logits)[(size_t)row * p.stride + li];
        else if (p.dtype == 1) v = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.logits)[(size_t)row * p.stride + li]);
        else v = __half2float(reinterpret_cast<const __half*>(p.logits)[(size_t)row * p.stride + li]);
        uint32_t u = __float_as_uint(v);
        u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
        const uint32_t gid = (uint32_t)(p.rank * p.vocab_local + li);
        const unsigned long long key = ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - gid);
        for (int r = 0; r < p.world; ++r) p.sym_keys[r][((size_t)par * kMaxRanks + p.rank) * p.max_rows + row] = key;
    }
    __threadfence_system();
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < p.world && threadIdx.x != p.rank) st_release_sys(p.sym_flags[threadIdx.x] + par * kMaxRanks + p.rank, e);
    if (threadIdx.x < p.world && threadIdx.x != p.rank) {
        if (!wait_flag_ge(p.sym_flags[p.rank] + par * kMaxRanks + threadIdx.x, e, p.status)) s_ok = 0;
    }
    __syncthreads();
    if (row < p.rows) {
        unsigned long long best = 0ull;
        if (s_ok) {
            for (int r = 0; r < p.world; ++r) {
                const unsigned long long k = __ldcg(&p.sym_keys[p.rank][((size_t)par * kMaxRanks + r) * p.max_rows + row]);
                best = k > best ? k : best;
            }
        }
        p.out[row] = (int)(0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull));
    }
    __syncthreads();
    if (threadIdx.x == 0) *p.epoch = e;
}

}  // namespace telb

using namespace telb;

extern "C" int telb_nvfp4_k64_pad(int k);

// Global greedy token per row from vocabulary-sharded logits (see argmax_merge_kernel).  `local_idx` is the arg-max of
// each row within this rank's shard; sym_keys / sym_flags hold `world` peer mappings of the symmetric tables
// ([2][8][max_rows] keys, [2][8] flags, zero-initialised); rows <= max_rows <= 1024.
extern "C" int telb_argmax_merge(const void* logits, long long stride, const int* local_idx, void* const* sym_keys, int* const* sym_flags,
                                 int* epoch, int* out, int rank, int world, int rows, int max_rows, int vocab_local, int dtype,
                                 int* status, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (world < 1 || world > kMaxRanks) return fail("telb_argmax_merge: world size must be in [1, 8]");
    if (rows > max_rows || max_rows > 1024) return fail("telb_argmax_merge: rows <= max_rows <= 1024 is required");
    if (dtype < 0 || dtype > 2) return fail("telb_argmax_merge: dtype must be 0 (fp16), 1 (bf16) or 2 (fp32)");
    ArgmaxMergeParams p{};
    p.logits = logits;
    p.local_idx = local_idx;
    for (int r = 0; r < world; ++r) {
        p.sym_keys[r] = (unsigned long long*)sym_keys[r];
        p.sym_flags[r] = sym_flags[r];
    }
    p.epoch = epoch;
    p.out = out;
    p.stride = stride;
    p.rank = rank;
    p.world = world;
    p.rows = rows;
    p.max_rows = max_rows;
    p.vocab_local = vocab_local;
    p.dtype = dtype;
    p.status = status;
    int threads = ((rows > world ? rows : world) + 31) / 32 * 32;
    TELB_LAUNCH("argmax_merge_kernel", (argmax_merge_kernel), dim3(1), dim3(threads), 0, stream, p);
    return 0;
}

// All-reduce(x) + residual → res_out; RMSNorm(res_out) * weight → y_out and/or NVFP4 (xq, sf).
//   sym_partial / sym_flags: `world` device pointers each (peer mappings of the symmetric buffers);
//   weight == null skips the norm (plain all-reduce + residual into res_out).
extern "C" int telb_ar_add_rmsnorm(const void* x, void* const* sym_partial, int* const* sym_flags, int* row_epoch,
                                   const void* residual, const void* weight, void* res_out, void* y_out, void* xq,
                                   void* sf, const float* quant_scale, int rank, int world, int rows, int hidden,
                                   int max_rows, float eps, int is_bf16, int* status, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (world < 1 || world > kMaxRanks) return fail("telb_ar_add_rmsnorm: world size must be in [1, 8]");
    if (rows > max_rows) return fail("telb_ar_add_rmsnorm: more rows than the symmetric buffers hold");
    if (hidden % 16) return fail("telb_ar_add_rmsnorm: hidden must be a multiple of 16");
    ArParams p{};
    p.x = x;
    for (int r = 0; r < world; ++r) {
        p.sym_partial[r] = sym_partial[r];
        p.sym_flags[r] = sym_flags[r];
    }
    p.row_epoch = row_epoch;
    p.residual = residual;
    p.weight = weight;
    p.res_out = res_out;
    p.y_out = y_out;
    p.xq = (uint8_t*)xq;
    p.sf = (uint8_t*)sf;
    p.quant_scale = quant_scale;
    p.rank = rank;
    p.world = world;
    p.rows = rows;
    p.hidden = hidden;
    p.max_rows = max_rows;
    p.k64_pad = telb_nvfp4_k64_pad(hidden);
    p.eps = eps;
    p.status = status;
    const int units = hidden / 16;
    int threads = units >= 256 ? 256 : ((units + 31) / 32) * 32;
    if (threads < 32) threads = 32;
    const int per = (units + threads - 1) / threads;
    if (per > 4) return fail("telb_ar_add_rmsnorm: hidden too large (max 16384)");
#define TELB_AR(T_, U_) TELB_LAUNCH("ar_add_rmsnorm_kernel", (ar_add_rmsnorm_kernel<T_, U_>), dim3(rows), dim3(threads), 0, stream, p)
    if (is_bf16) {
        if (per <= 1) TELB_AR(__nv_bfloat16, 1); else if (per <= 2) TELB_AR(__nv_bfloat16, 2); else TELB_AR(__nv_bfloat16, 4);
    } else {
        if (per <= 1) TELB_AR(__half, 1); else if (per <= 2) TELB_AR(__half, 2); else TELB_AR(__half, 4);
    }
#undef TELB_AR
    return 0;
}

// Reduce-scatter (already stored by the GEMM epilogue) + residual + RMSNorm (+ NVFP4) + all-gather push.
// Pointer tables hold `world` peer mappings each.  gather_y or (gather_xq, gather_sf) selects the output
// form; weight == null skips the norm.  rows = global row count, rows_per_rank = ceil(rows / world).
extern "C" int telb_rs_add_rmsnorm_ag(const void* partial, int* const* gemm_flags, int* const* ag_flags, int* epoch, int* ticket,
                                      const void* residual, int residual_full, const void* weight, void* res_out,
                                      void* const* gather_y, void* const* gather_xq, void* const* gather_sf,
                                      const float* quant_scale, int rank, int world, int rows, int rows_per_rank, int hidden,
                                      float eps, int wait_gather, int is_bf16, int* status, int sum_slots, int slot_base,
                                      cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (world < 1 || world > kMaxRanks) return fail("telb_rs_add_rmsnorm_ag: world size must be in [1, 8]");
    if (sum_slots <= 0) {
        sum_slots = world;
        slot_base = 0;
    }
    if (slot_base < 0 || slot_base + sum_slots > world) return fail("telb_rs_add_rmsnorm_ag: partial slot range outside [0, world)");
    if (hidden % 16) return fail("telb_rs_add_rmsnorm_ag: hidden must be a multiple of 16");
    if (rows_per_rank * world < rows) return fail("telb_rs_add_rmsnorm_ag: rows_per_rank * world must cover the rows");
    if (!gather_y && !gather_xq) return fail("telb_rs_add_rmsnorm_ag: no output buffer");
    RsAgParams p{};
    p.partial = partial;
    for (int r = 0; r < world; ++r) {
        p.gemm_flags[r] = gemm_flags[r];
        p.ag_flags[r] = ag_flags[r];
        if (gather_y) p.gather_y[r] = gather_y[r];
        if (gather_xq) {
            p.gather_xq[r] = (uint8_t*)gather_xq[r];
            p.gather_sf[r] = (uint8_t*)gather_sf[r];
        }
    }
    p.epoch = epoch;
    p.ticket = ticket;
    p.residual = residual;
    p.residual_full = residual_full;
    p.weight = weight;
    p.res_out = res_out;
    p.quant_scale = quant_scale;
    p.rank = rank;
    p.world = world;
    p.rows = rows;
    p.rows_per_rank = rows_per_rank;
    p.hidden = hidden;
    p.k64_pad = telb_nvfp4_k64_pad(hidden);
    p.wait_gather = wait_gather;
    p.sum_slots = sum_slots;
    p.slot_base = slot_base;
    p.eps = eps;
    p.status = status;
    int rows_local = rows - rank * rows_per_rank;
    rows_local = rows_local < 0 ? 0 : (rows_local > rows_per_rank ? rows_per_rank : rows_local);
    // one CTA per row up to four CTAs per SM; beyond that the CTAs loop over rows
    int grid = rows_local > 0 ? rows_local : 1;
    if (grid > 4 * sm_count()) grid = 4 * sm_count();
    const int units = hidden / 16;
    int threads = units >= 256 ? 256 : ((units + 31) / 32) * 32;
    if (threads < 32) threads = 32;
    const int per = (units + threads - 1) / threads;
    if (per > 4) return fail("telb_rs_add_rmsnorm_ag: hidden too large (max 16384)");
#define TELB_RS(T_, U_) TELB_LAUNCH("rs_add_rmsnorm_ag_kernel", (rs_add_rmsnorm_ag_kernel<T_, U_>), dim3(grid), dim3(threads), 0, stream, p)
    if (is_bf16) {
        if (per <= 1) TELB_RS(__nv_bfloat16, 1); else if (per <= 2) TELB_RS(__nv_bfloat16, 2); else TELB_RS(__nv_bfloat16, 4);
    } else {
        if (per <= 1) TELB_RS(__half, 1); else if (per <= 2) TELB_RS(__half, 2); else TELB_RS(__half, 4);
    }
#undef TELB_RS
    return 0;
}
