// Shared device/host helpers for the sm_100a kernels of the quantized-linear path.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// dtype codes that cross the C ABI (same numbering as the reference:
// comfy_kitchen/backends/eager/quantization.py:33-41).
#define CK_F32 0
#define CK_F16 1
#define CK_BF16 2
#define CK_E4M3 5
#define CK_E5M2 6

// status codes returned by every launch_* entry point
#define CK_OK 0
#define CK_ERR_DTYPE (-1)
#define CK_ERR_SHAPE (-2)
#define CK_ERR_ALIGN (-3)
#define CK_ERR_NULL (-4)
#define CK_ERR_UNSUPPORTED (-5)
#define CK_ERR_DEVICE_TIMEOUT (-6)

namespace ck {

// Records a human-readable reason for the last non-zero status on this thread.
void set_error(const char* fmt, ...);

#define CK_FAIL(code, ...)          \
    do {                            \
        ::ck::set_error(__VA_ARGS__); \
        return (code);              \
    } while (0)

// After a launch: report a launch-configuration error without synchronising.
inline int launch_status(const char* what) {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("%s: %s", what, cudaGetErrorString(e));
        return (int)e;
    }
    return CK_OK;
}

__host__ __device__ inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }
__host__ __device__ inline int64_t ceil_div(int64_t x, int64_t m) { return (x + m - 1) / m; }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------- element types

template <typename T> struct Elem;

template <> struct Elem<float> {
    static constexpr int code = CK_F32;
    __device__ static float to_f32(float v) { return v; }
    __device__ static float from_f32(float v) { return v; }
    __device__ static float round(float v) { return v; }
};
template <> struct Elem<__half> {
    static constexpr int code = CK_F16;
    __device__ static float to_f32(__half v) { return __half2float(v); }
    __device__ static __half from_f32(float v) { return __float2half_rn(v); }
    __device__ static float round(float v) { return __half2float(__float2half_rn(v)); }
};
template <> struct Elem<__nv_bfloat16> {
    static constexpr int code = CK_BF16;
    __device__ static float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
    __device__ static float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

// 8 consecutive elements as fp32, loaded with 128-bit accesses.
template <typename T>
__device__ __forceinline__ void load8(const T* __restrict__ p, float (&v)[8]);

template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* __restrict__ p, float (&v)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* __restrict__ p, float (&v)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
        float2 f = __half22float2(h);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
template <>
__device__ __forceinline__ void load8<float>(const float* __restrict__ p, float (&v)[8]) {
    float4 a = *reinterpret_cast<const float4*>(p);
    float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// 8 consecutive fp32 values rounded to T and stored with 128-bit accesses.
template <typename T>
__device__ __forceinline__ void store8(T* __restrict__ p, const float (&v)[8]);

template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* __restrict__ p, const float (&v)[8]) {
    uint4 u;
    uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = u;
}
template <>
__device__ __forceinline__ void store8<__half>(__half* __restrict__ p, const float (&v)[8]) {
    uint4 u;
    uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = u;
}
template <>
__device__ __forceinline__ void store8<float>(float* __restrict__ p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

// ------------------------------------------------------------ scale-factor layout

// Byte offset of block scale (r, c) in the 128-row x 4-column tiled layout that
// the block-scaled MMA consumes (each 512-byte tile: 32 rows x 16 bytes, the 16
// bytes holding rows r, r+32, r+64, r+96 x 4 columns).  cpad = columns rounded
// up to 4.  Same layout as comfy_kitchen/float_utils.py:292-326 (to_blocked).
__host__ __device__ __forceinline__ int64_t sf_offset(int64_t r, int64_t c, int64_t cpad) {
    return ((r >> 7) * (cpad >> 2) + (c >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (c & 3);
}
// Offset inside one 512-byte tile for row-in-tile r (0..127) and column c (0..3).
__device__ __forceinline__ int sf_tile_offset(int r, int c) { return (r & 31) * 16 + (r >> 5) * 4 + c; }

// ------------------------------------------------------------ narrow conversions

// Two floats -> one byte of two E2M1 codes, round-to-nearest-even, saturating
// at +-6.  `hi` lands in bits 7:4, `lo` in bits 3:0.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float hi, float lo) {
    uint16_t out;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; mov.b16 %0, {t, 0}; }"
        : "=h"(out) : "f"(hi), "f"(lo));
    return out;
}

// Two floats -> two E4M3 bytes (`hi` in bits 15:8), RNE, saturating at +-448.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float hi, float lo) {
    uint16_t out;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(out) : "f"(hi), "f"(lo));
    return out;
}
__device__ __forceinline__ uint32_t cvt_e5m2x2(float hi, float lo) {
    uint16_t out;
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(out) : "f"(hi), "f"(lo));
    return out;
}

// One E4M3 / E5M2 byte -> float (exact).
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
    uint32_t h2;
    asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(h2) : "r"(b & 0xffu));
    return __half2float(__ushort_as_half((unsigned short)(h2 & 0xffffu)));
}
__device__ __forceinline__ float e5m2_to_f32(uint32_t b) {
    return __half2float(__ushort_as_half((unsigned short)((b & 0xffu) << 8)));
}
// Two packed E4M3 bytes (low 16 bits) -> two floats, x = low byte.
__device__ __forceinline__ float2 e4m3x2_to_f32x2(uint32_t b) {
    uint32_t h2;
    asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(h2) : "r"(b & 0xffffu));
    return __half22float2(*reinterpret_cast<__half2*>(&h2));
}

__device__ __forceinline__ float e2m1_value(uint32_t code) {
    // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 = 2 * {0,1,2,3,4,6,8,12} / 4, packed as nibbles
    uint32_t m = (0xC8643210u >> ((code & 7u) * 4)) & 0xfu;
    float v = 0.5f * (float)m;
    return (code & 8u) ? -v : v;
}

// Raw 8-element vectors kept in registers without widening (4 registers for the
// 16-bit types, 8 for fp32).
template <typename T> struct Raw8 { uint4 u; };
template <> struct Raw8<float> { float4 a, b; };

template <typename T>
__device__ __forceinline__ Raw8<T> load_raw8(const T* __restrict__ p) {
    Raw8<T> r;
    r.u = *reinterpret_cast<const uint4*>(p);
    return r;
}
template <>
__device__ __forceinline__ Raw8<float> load_raw8<float>(const float* __restrict__ p) {
    Raw8<float> r;
    r.a = *reinterpret_cast<const float4*>(p);
    r.b = *reinterpret_cast<const float4*>(p + 4);
    return r;
}
template <typename T>
__device__ __forceinline__ Raw8<T> zero_raw8() {
    Raw8<T> r;
    r.u = make_uint4(0u, 0u, 0u, 0u);
    return r;
}
template <>
__device__ __forceinline__ Raw8<float> zero_raw8<float>() {
    Raw8<float> r;
    r.a = make_float4(0.f, 0.f, 0.f, 0.f);
    r.b = r.a;
    return r;
}
__device__ __forceinline__ void unpack8(const Raw8<__nv_bfloat16>& r, float (&v)[8]) {
    const uint32_t w[4] = {r.u.x, r.u.y, r.u.z, r.u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void unpack8(const Raw8<__half>& r, float (&v)[8]) {
    const uint32_t w[4] = {r.u.x, r.u.y, r.u.z, r.u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void unpack8(const Raw8<float>& r, float (&v)[8]) {
    v[0] = r.a.x; v[1] = r.a.y; v[2] = r.a.z; v[3] = r.a.w;
    v[4] = r.b.x; v[5] = r.b.y; v[6] = r.b.z; v[7] = r.b.w;
}

// ------------------------------------------------------------ block encoders

// NVFP4: this lane holds 8 of the 16 elements of a block (its partner is lane^1).
// Returns 4 bytes of E2M1 codes and the block's E4M3 scale byte.  Must be called
// by all 32 lanes.  Arithmetic order: see quant_nvfp4.cu.
__device__ __forceinline__ uint32_t nvfp4_encode_half_block(const float (&v)[8], float g, bool hi_first, uint32_t& s8) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const float bs = __fdiv_rn(amax, 6.0f);
    const float sbs = fminf(__fdiv_rn(bs, g), 448.0f);
    s8 = cvt_e4m3x2(0.0f, sbs) & 0xffu;
    const float tot = __fmul_rn(g, e4m3_to_f32(s8));
    uint32_t packed = 0;
    if (tot != 0.0f) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float a = __fdiv_rn(v[2 * i], tot);
            const float b = __fdiv_rn(v[2 * i + 1], tot);
            const uint32_t byte = hi_first ? cvt_e2m1x2(a, b) : cvt_e2m1x2(b, a);
            packed |= (byte & 0xffu) << (8 * i);
        }
    }
    return packed;
}

// E8M0 byte for a block amax: clamp(ceil(log2(max(amax/448, 2^-127))) + 127, 0, 254),
// read off the bits of the quotient.
__device__ __forceinline__ uint32_t mx_scale_byte(float amax) {
    float r = __fdiv_rn(amax, 448.0f);
    const float tiny = __uint_as_float(0x00400000u);  // 2^-127
    if (!(r > tiny)) r = tiny;
    const uint32_t u = __float_as_uint(r);
    const uint32_t ef = (u >> 23) & 0xffu, mant = u & 0x7fffffu;
    uint32_t e;
    if (ef == 0) e = mant > 0x400000u ? 1u : 0u;
    else if (ef == 0xffu) e = 254u;
    else e = ef + (mant != 0u);
    return e > 254u ? 254u : e;
}

// MXFP8: this lane holds 8 of the 32 elements of a block (lanes ^1, ^2 hold the
// rest).  Returns 8 E4M3 bytes and the block's E8M0 byte (0 for an all-zero block).
__device__ __forceinline__ uint2 mxfp8_encode_quarter_block(const float (&v)[8], uint32_t& e) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    e = 0;
    uint32_t w[2] = {0u, 0u};
    if (amax != 0.0f) {
        e = mx_scale_byte(amax);
        if (e != 0u) {
            // 2^(127-e); for e == 254 that is the subnormal 2^-127
            const float inv = __uint_as_float(e == 254u ? 0x00400000u : ((254u - e) << 23));
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t two = cvt_e4m3x2(__fmul_rn(v[2 * i + 1], inv), __fmul_rn(v[2 * i], inv));
                w[i >> 1] |= two << (16 * (i & 1));
            }
        } else {
            // the reference decodes e == 0 as a scale of 0.0: x/0 -> +-448, 0/0 -> NaN
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float xv = v[i];
                const uint32_t b = xv > 0.0f ? 0x7eu : (xv < 0.0f ? 0xfeu : 0xffu);
                w[i >> 2] |= b << (8 * (i & 3));
            }
        }
    }
    return make_uint2(w[0], w[1]);
}

}  // namespace ck
