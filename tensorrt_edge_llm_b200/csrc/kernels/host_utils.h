// Host-side helpers for the kernel launchers: tensor-map encoding through the driver entry point
// (no link-time dependency on libcuda), error reporting, device property cache.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

namespace telb {

// Launchers return 0 on success or a negative code; the last message is kept per thread.
inline thread_local char g_last_error[512] = {0};

inline int fail(const char* what, cudaError_t e = cudaSuccess) {
    if (e != cudaSuccess)
        snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
    else
        snprintf(g_last_error, sizeof(g_last_error), "%s", what);
    return -1;
}

#define TELB_CHECK_LAUNCH(name)                                   \
    do {                                                          \
        cudaError_t e__ = cudaGetLastError();                     \
        if (e__ != cudaSuccess) return ::telb::fail(name, e__);   \
    } while (0)

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline PFN_encodeTiled encode_tiled_fn() {
    static PFN_encodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_encodeTiled>(p);
    }
    return fn;
}

// Encoded tensor maps are remembered per thread, keyed by everything that goes into them (base pointer, extents, pitches,
// box, type, swizzle): a map depends on nothing else, so a later launch over the same buffer and shape copies the 128
// bytes instead of calling the driver again.  Direct-mapped, 512 entries; a colliding key simply replaces the entry.
struct TmapKey {
    uint64_t base;
    uint64_t dims[5];
    uint64_t strides[4];
    uint32_t box[5];
    uint32_t dt, rank, swz, l2;
};
struct TmapEntry {
    TmapKey key;
    CUtensorMap map;
    bool used;
};
inline TmapEntry* tmap_cache_slot(const TmapKey& k) {
    static thread_local TmapEntry* table = nullptr;
    if (!table) table = static_cast<TmapEntry*>(calloc(512, sizeof(TmapEntry)));
    if (!table) return nullptr;
    uint64_t h = 1469598103934665603ull;
    const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
    for (size_t i = 0; i < sizeof(TmapKey) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
    return &table[(h ^ (h >> 29)) & 511];
}
inline int encode_tmap_cached(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const cuuint64_t* dims,
                              const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle swz, CUtensorMapL2promotion l2) {
    TmapKey k;
    memset(&k, 0, sizeof(k));
    k.base = reinterpret_cast<uint64_t>(base);
    for (int i = 0; i < rank; ++i) {
        k.dims[i] = dims[i];
        k.box[i] = box[i];
        if (i + 1 < rank) k.strides[i] = strides[i];
    }
    k.dt = (uint32_t)dt;
    k.rank = (uint32_t)rank;
    k.swz = (uint32_t)swz;
    k.l2 = (uint32_t)l2;
    TmapEntry* e = tmap_cache_slot(k);
    if (e && e->used && memcmp(&e->key, &k, sizeof(k)) == 0) {
        memcpy(out, &e->map, sizeof(CUtensorMap));
        return 0;
    }
    PFN_encodeTiled enc = encode_tiled_fn();
    if (!enc) return fail("cuTensorMapEncodeTiled entry point not found");
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = enc(out, dt, rank, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, l2,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return (int)r;
    if (e) {
        e->key = k;
        memcpy(&e->map, out, sizeof(CUtensorMap));
        e->used = true;
    }
    return 0;
}

// Row-major 2-D tensor [rows, cols] of `elem_bytes` elements with row pitch `pitch_bytes`; box
// [box_rows, box_cols].  box_cols * elem_bytes must equal the swizzle span for swizzled maps.
inline int make_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t rows,
                        uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols,
                        CUtensorMapSwizzle swz, CUtensorMapL2promotion l2 = CU_TENSOR_MAP_L2_PROMOTION_L2_256B) {
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    (void)elem_bytes;
    const int r = encode_tmap_cached(out, dt, 2, base, dims, strides, box, swz, l2);
    if (r < 0) return r;
    if (r != 0) {
        snprintf(g_last_error, sizeof(g_last_error),
                 "cuTensorMapEncodeTiled(2d) failed: %d (base %p rows %llu cols %llu pitch %llu box %u x %u)", (int)r,
                 base, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)pitch_bytes, box_rows,
                 box_cols);
        return -1;
    }
    return 0;
}

// General N-D (N <= 5) map; dims / strides innermost first, strides[i] is the byte pitch of dim i+1.
inline int make_tmap_nd(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
                        const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz) {
    cuuint64_t d[5];
    cuuint64_t s[4];
    cuuint32_t b[5];
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
        if (i + 1 < rank) s[i] = strides_bytes[i];
    }
    const int r = encode_tmap_cached(out, dt, rank, base, d, s, b, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (r < 0) return r;
    if (r != 0) {
        snprintf(g_last_error, sizeof(g_last_error), "cuTensorMapEncodeTiled(%dd) failed: %d", rank, (int)r);
        return -1;
    }
    return 0;
}

// Launch with programmatic dependent launch enabled (see pdl_wait in tc5_common.cuh).  Setting the
// environment variable TELB_DISABLE_PDL=1 (or the reference's EDGELLM_ENABLE_PDL=0) falls back to fully serialised launches.
inline bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("TELB_DISABLE_PDL");
        const char* r = getenv("EDGELLM_ENABLE_PDL");
        v = ((e && e[0] == '1') || (r && r[0] == '0')) ? 0 : 1;
    }
    return v == 1;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define TELB_LAUNCH(name, kernel, grid, block, smem, stream, ...)                                   \
    do {                                                                                            \
        cudaError_t e__ = ::telb::launch_pdl(kernel, grid, block, smem, stream, __VA_ARGS__);       \
        if (e__ != cudaSuccess) return ::telb::fail(name, e__);                                     \
    } while (0)

inline int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

}  // namespace telb
