// NVFP4 helpers shared by the quantising kernels: E2M1 packing, the per-16-element block quantiser
// and the address of a scale byte in the 512-byte atom layout read by the block-scaled tensor core.
#pragma once

#include <cuda_fp8.h>

#include "tc5_common.cuh"

namespace telb {

__device__ __forceinline__ uint32_t pack_e2m1x8(const float (&v)[8]) {
    uint32_t out = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint16_t b;
        // cvt packs {a → high nibble, b → low nibble}; the even element must land in the low nibble
        asm volatile("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u16.u8 %0, t;\n\t}"
                     : "=h"(b) : "f"(v[2 * i + 1]), "f"(v[2 * i]));
        out |= static_cast<uint32_t>(b & 0xFF) << (8 * i);
    }
    return out;
}


// Byte offset of the scale of (row r, 16-element block kb) in [row tile of 128][k64_pad][512 B].
__device__ __forceinline__ size_t sf_atom_offset(long long r, int kb, int k64_pad) {
    const int rr = (int)(r & 127);
    return ((size_t)(r >> 7) * k64_pad + (kb >> 2)) * 512 + (rr & 31) * 16 + (rr >> 5) * 4 + (kb & 3);
}

// Quantise 16 values: scale = e4m3(amax / 6 / global) (saturating at 448), codes = rn_e2m1(v / (scale * global)).
// Returns the 8 packed bytes; `s8` receives the E4M3 scale byte.
__device__ __forceinline__ uint2 nvfp4_quantize_block16(const float (&v)[16], float amax, float gs, float inv_gs, uint8_t& s8) {
    const float s = fminf(amax * (1.f / 6.f) * inv_gs, 448.f);
    const __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3);
    s8 = q;
    const float sf_f = __half2float(__half(__nv_cvt_fp8_to_halfraw(q, __NV_E4M3))) * gs;
    const float inv = sf_f > 0.f ? 1.f / sf_f : 0.f;
    float a[8], b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        a[i] = v[i] * inv;
        b[i] = v[8 + i] * inv;
    }
    uint2 packed;
    packed.x = pack_e2m1x8(a);
    packed.y = pack_e2m1x8(b);
    return packed;
}

// The same quantiser for 16 values spread over 16 consecutive lanes of a warp (lane i of the group holds value i, already
// rounded to the activation type): every lane of the group gets the block's scale byte in `s8`; the lane with
// (lane & 7) == 0 gets four packed bytes (eight codes) in the return value.  All 32 lanes must call it.
__device__ __forceinline__ uint32_t nvfp4_quantize_lane16(float y, float gs, float inv_gs, uint8_t& s8) {
    float amax = fabsf(y);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = fminf(amax * (1.f / 6.f) * inv_gs, 448.f);
    const __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3);
    s8 = q;
    const float sf_f = __half2float(__half(__nv_cvt_fp8_to_halfraw(q, __NV_E4M3))) * gs;
    const float inv = sf_f > 0.f ? 1.f / sf_f : 0.f;
    const float mine = y * inv;
    const float next = __shfl_xor_sync(0xffffffffu, mine, 1);          // even lanes: the odd neighbour's value
    uint16_t b16;
    asm volatile("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u16.u8 %0, t;\n\t}" : "=h"(b16) : "f"(next), "f"(mine));
    uint32_t w = b16 & 0xFFu;                                           // valid on even lanes: codes of (lane, lane + 1)
    w |= (__shfl_down_sync(0xffffffffu, w, 2) & 0xFFu) << 8;
    w |= (__shfl_down_sync(0xffffffffu, w, 4) & 0xFFFFu) << 16;
    return w;
}

}  // namespace telb
