// Two-level arg-max whose scratch lives in a file-scope device array, so the call path contains no
// allocation of any kind (no cudaMalloc, no caching allocator, no workspace object).
//
// Who needs that: code that picks the greedy token from places where asking an allocator for
// memory is off the table — a native request-engine thread that owns no framework allocator, a
// decode loop running while the KV pool has already claimed the rest of device memory, or a
// latency-critical step where an allocator call could block on a device synchronisation.  The
// general entry point (telb_argmax) takes its scratch from a caller-provided workspace instead.
//
// Scheme: `nblk` CTAs per row each reduce one slice of the vocabulary to a packed 64-bit key
// (order-preserving value bits in the high word, inverted index in the low word, so a larger key is
// a larger value or, on a tie, a lower index) and publish it with atomicMax; the CTA that arrives
// last at the row's counter writes the winner.
#include "argmax_static.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "host_utils.h"

namespace {

constexpr int kMaxRows = TELB_ARGMAX_STATIC_MAX_ROWS;
constexpr int kMaxDevices = 64;
constexpr int kThreads = 512;

struct Scratch {
    unsigned long long keys[kMaxRows];      // running maximum key per row; must start at zero
    int counters[kMaxRows];                 // CTAs of the row that have published; must start at zero
};

// 3 KB per device, part of the module image: exists from module load to process exit.
static __device__ __align__(256) Scratch g_scratch;

std::mutex g_setup_mutex;
Scratch* g_scratch_ptr[kMaxDevices] = {nullptr};

template <typename T>
__device__ __forceinline__ float as_float(T v);
template <> __device__ __forceinline__ float as_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float as_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float as_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ unsigned long long key_max(unsigned long long a, unsigned long long b) { return a > b ? a : b; }

template <typename T>
__global__ void __launch_bounds__(kThreads)
argmax_static_kernel(const T* __restrict__ logits, int* __restrict__ out, int vocab, long long stride, Scratch* __restrict__ scratch) {
    __shared__ unsigned long long warp_best[kThreads / 32];
    const int row = blockIdx.y;
    const int nblk = gridDim.x;
    const int per = (vocab + nblk - 1) / nblk;
    const int lo = blockIdx.x * per;
    const int hi = min(vocab, lo + per);
    const T* p = logits + (size_t)row * stride;
    unsigned long long best = 0ull;
    for (int i = lo + threadIdx.x; i < hi; i += kThreads) {
        uint32_t u = __float_as_uint(as_float<T>(p[i]));
        u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
        best = key_max(best, ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)i));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = key_max(best, __shfl_xor_sync(0xffffffffu, best, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) warp_best[warp] = best;
    __syncthreads();
    if (warp != 0) return;
    best = lane < kThreads / 32 ? warp_best[lane] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = key_max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if (lane != 0) return;
    atomicMax(&scratch->keys[row], best);
    __threadfence();
    if (atomicAdd(&scratch->counters[row], 1) == nblk - 1) {
        __threadfence();
        const unsigned long long k = atomicMax(&scratch->keys[row], 0ull);      // atomic read of the final key
        out[row] = (int)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull));
    }
}

// Device address of g_scratch on the current device, looked up once per device.  The kernel runs on the device
// that owns `stream`, so a stream that belongs to another device than the current one is refused: the scratch
// pointer cached for the current device would be another GPU's memory there.
int scratch_for_current_device(Scratch** ptr, cudaStream_t stream, const void* logits) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return telb::fail("telb_argmax_static: cudaGetDevice", e);
    if (dev < 0 || dev >= kMaxDevices) return telb::fail("telb_argmax_static: device ordinal out of range");
    if (stream != nullptr && stream != cudaStreamLegacy && stream != cudaStreamPerThread) {
        int sdev = -1;
        e = cudaStreamGetDevice(stream, &sdev);
        if (e != cudaSuccess) return telb::fail("telb_argmax_static: cudaStreamGetDevice", e);
        if (sdev != dev) {
            snprintf(telb::g_last_error, sizeof(telb::g_last_error),
                     "telb_argmax_static: the stream belongs to device %d but device %d is current; make the stream's device current first", sdev, dev);
            return -1;
        }
    }
    cudaPointerAttributes attr{};
    e = cudaPointerGetAttributes(&attr, logits);
    if (e != cudaSuccess) return telb::fail("telb_argmax_static: cudaPointerGetAttributes", e);
    if (attr.type == cudaMemoryTypeDevice && attr.device != dev) {
        snprintf(telb::g_last_error, sizeof(telb::g_last_error),
                 "telb_argmax_static: logits live on device %d but device %d is current", attr.device, dev);
        return -1;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        Scratch* found = nullptr;
        e = cudaGetSymbolAddress((void**)&found, g_scratch);
        if (e != cudaSuccess) return telb::fail("telb_argmax_static: cudaGetSymbolAddress", e);
        if (found == nullptr) return telb::fail("telb_argmax_static: scratch symbol has no device address");
        g_scratch_ptr[dev] = found;
    }
    *ptr = g_scratch_ptr[dev];
    return 0;
}

}  // namespace

extern "C" int telb_argmax_static(const void* logits, int* out, int rows, int vocab, long long stride, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (rows < 0 || rows > kMaxRows) {
        snprintf(telb::g_last_error, sizeof(telb::g_last_error), "telb_argmax_static: rows = %d is outside 1..%d (the fixed scratch holds %d rows)",
                 rows, kMaxRows, kMaxRows);
        return -1;
    }
    if (vocab < 1) return telb::fail("telb_argmax_static: vocab must be at least 1");
    if (dtype < 0 || dtype > 2) return telb::fail("telb_argmax_static: dtype must be 0 (fp16), 1 (bf16) or 2 (fp32)");
    if (logits == nullptr || out == nullptr) return telb::fail("telb_argmax_static: null pointer");
    Scratch* scratch = nullptr;
    if (scratch_for_current_device(&scratch, stream, logits) != 0) return -1;
    // Every call starts from zeroed keys and counters, whatever an earlier call left behind.
    cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(Scratch), stream);
    if (e != cudaSuccess) return telb::fail("telb_argmax_static: cudaMemsetAsync", e);
    int nblk = (2 * 148 + rows - 1) / rows;        // about two CTAs per SM in total
    if (nblk > 64) nblk = 64;
    const int max_useful = (vocab + kThreads - 1) / kThreads;
    if (nblk > max_useful) nblk = max_useful;
    if (nblk < 1) nblk = 1;
    const dim3 grid(nblk, rows), block(kThreads);
    if (dtype == 2)
        argmax_static_kernel<float><<<grid, block, 0, stream>>>((const float*)logits, out, vocab, stride, scratch);
    else if (dtype == 1)
        argmax_static_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>((const __nv_bfloat16*)logits, out, vocab, stride, scratch);
    else
        argmax_static_kernel<__half><<<grid, block, 0, stream>>>((const __half*)logits, out, vocab, stride, scratch);
    TELB_CHECK_LAUNCH("argmax_static_kernel");
    return 0;
}
