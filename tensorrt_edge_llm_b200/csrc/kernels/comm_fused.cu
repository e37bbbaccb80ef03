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
                float acc[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[i] = 0.f;
                for (int r = 0; r < p.world; ++r) {
                    if (r == p.rank) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) acc[i] += v[u][i];
                    } else {
                        const T* src = reinterpret_cast<const T*>(p.sym_partial[r]) + ((size_t)par * p.max_rows + row) * p.hidden + idx * 16;
                        const uint4 a0 = ld_peer_v4(src), a1 = ld_peer_v4(src + 8);
                        const T* e0 = reinterpret_cast<const T*>(&a0);
                        const T* e1 = reinterpret_cast<const T*>(&a1);
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

}  // namespace telb

using namespace telb;

extern "C" int telb_nvfp4_k64_pad(int k);

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
