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

// Status codes and the declaration of every extern "C" entry point: including the public header here
// makes the compiler check each definition in csrc/*.cu against what callers bind to.
#include "comfy_kitchen_b200.h"
#include "ck_options.h"

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
inline bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

// ---------------------------------------------------------------- element types

template <typename T> struct Elem;

template <> struct Elem<float> {
    static constexpr int code = CK_F32;
    __device__ static float to_f32(float v) { return v; }
    __device__ static float from_f32(float v) { return v; }
    __device__ static float round(float v) { return v; }
    __device__ static void round2(float&, float&) {}
};
template <> struct Elem<__half> {
    static constexpr int code = CK_F16;
    __device__ static float to_f32(__half v) { return __half2float(v); }
    __device__ static __half from_f32(float v) { return __float2half_rn(v); }
    __device__ static float round(float v) { return __half2float(__float2half_rn(v)); }
    // both values rounded to the type and back with one packed conversion each way
    __device__ static void round2(float& a, float& b) {
        const float2 f = __half22float2(__floats2half2_rn(a, b));
        a = f.x; b = f.y;
    }
};
template <> struct Elem<__nv_bfloat16> {
    static constexpr int code = CK_BF16;
    __device__ static float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
    __device__ static float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
    __device__ static void round2(float& a, float& b) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);   // .x = a in the low half
        const uint32_t w = *reinterpret_cast<const uint32_t*>(&h);
        a = __uint_as_float(w << 16); b = __uint_as_float(w & 0xffff0000u);
    }
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

// ---- NVFP4 block arithmetic --------------------------------------------------------------
// The reference divides three times per block/element with IEEE fp32 division:
//   bs = amax / 6;  sbs = bs / g;  q = x / tot   (tot = g * e4m3(sbs)).
// A correctly rounded quotient a/b can also be had from the correctly rounded reciprocal
// r = RN(1/b):  q0 = RN(a*r);  rem = a - b*q0 (exact, one FMA);  q = RN(q0 + rem*r)
// (Markstein's sequence; it needs b's significand not to be all ones and no under/overflow
// in q0 and rem).  r is shared by every element of a block (1/tot) or of the tensor (1/g),
// so the per-element cost drops from a full division to three FMAs.  Wherever the conditions
// are not met the code below takes the plain IEEE division, so results are bit-identical by
// construction; where a tiny operand makes `rem` inexact the quotient is far below the
// smallest rounding boundary that matters (2^-10 for the E4M3 scale, 0.25 for E2M1 codes).
struct Nvfp4Ctx {
    float g;    // per-tensor scale
    float rg;   // RN(1/g)
    bool fast;  // g admits the reciprocal sequence
};

__device__ __forceinline__ Nvfp4Ctx nvfp4_ctx(float g) {
    Nvfp4Ctx c;
    c.g = g;
    c.rg = __frcp_rn(g);
    const uint32_t u = __float_as_uint(g), e = (u >> 23) & 0xffu;
    c.fast = (u >> 31) == 0u && e >= 40u && e <= 214u && (u & 0x7fffffu) != 0x7fffffu;  // 2^-87 <= g < 2^88
    return c;
}

// Written as q0 - (b*q0 - a)*r rather than q0 + (a - b*q0)*r: the same value, but a zero result keeps
// the sign of `a` (b > 0), which is the sign an IEEE division gives (-0.0 / b = -0.0 -> E2M1 code 8).
__device__ __forceinline__ float div_by_reciprocal(float a, float b, float r) {
    const float q0 = __fmul_rn(a, r);
    const float e = __fmaf_rn(b, q0, -a);
    return __fmaf_rn(-e, r, q0);
}

struct Nvfp4Block {
    uint32_t s8;  // E4M3 scale byte
    float tot;    // g * float(s8)
    float rtot;   // RN(1/tot) when `fast`
    bool fast;    // per-element quotients may use the reciprocal sequence
};

// amax of a 16-element block -> its scale byte and the divisor of its elements.
template <bool kExactDiv>
__device__ __forceinline__ Nvfp4Block nvfp4_block_scale(float amax, const Nvfp4Ctx& c) {
    float sbs;
    if (!kExactDiv && c.fast) {
        // exact for every amax >= 2^-125; below that sbs < 2^-38 rounds to scale 0 either way
        const float bs = div_by_reciprocal(amax, 6.0f, 0.16666667163372040f /* RN(1/6) */);
        // an overflowing quotient turns into NaN here and fminf returns the other operand, 448
        sbs = div_by_reciprocal(bs, c.g, c.rg);
    } else {
        sbs = __fdiv_rn(__fdiv_rn(amax, 6.0f), c.g);
    }
    sbs = fminf(sbs, 448.0f);
    Nvfp4Block b;
    b.s8 = cvt_e4m3x2(0.0f, sbs) & 0xffu;
    b.tot = __fmul_rn(c.g, e4m3_to_f32(b.s8));
    const uint32_t u = __float_as_uint(b.tot), e = (u >> 23) & 0xffu;
    // 2^-64 <= tot < 2^65, significand not all ones, |x| <= amax < 2^60 (no overflow in x * rtot)
    b.fast = !kExactDiv && e >= 63u && e <= 191u && (u & 0x7fffffu) != 0x7fffffu &&
             ((__float_as_uint(amax) >> 23) & 0xffu) < 187u;
    b.rtot = b.fast ? __frcp_rn(b.tot) : 0.0f;
    return b;
}

// Eight elements of a block -> four bytes of E2M1 codes (element 2i and 2i+1 share byte i).
__device__ __forceinline__ uint32_t nvfp4_codes8(const float (&v)[8], const Nvfp4Block& b, bool hi_first) {
    if (b.tot == 0.0f) return 0u;
    float q[8];
    if (b.fast) {
        // div_by_reciprocal on pairs: sm_100's packed fp32 instructions do two IEEE operations each
        const float2 r2 = make_float2(b.rtot, b.rtot), b2 = make_float2(b.tot, b.tot);
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            const float2 a2 = make_float2(v[i], v[i + 1]);
            const float2 q0 = __fmul2_rn(a2, r2);
            const float2 e = __ffma2_rn(b2, q0, make_float2(-a2.x, -a2.y));
            const float2 qq = __ffma2_rn(make_float2(-e.x, -e.y), r2, q0);
            q[i] = qq.x; q[i + 1] = qq.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = __fdiv_rn(v[i], b.tot);
    }
    uint32_t out;
    if (hi_first) {
        asm("{ .reg .b8 t0, t1, t2, t3;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t0, %1, %2; cvt.rn.satfinite.e2m1x2.f32 t1, %3, %4;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t2, %5, %6; cvt.rn.satfinite.e2m1x2.f32 t3, %7, %8;\n"
            "mov.b32 %0, {t0, t1, t2, t3}; }"
            : "=r"(out) : "f"(q[0]), "f"(q[1]), "f"(q[2]), "f"(q[3]), "f"(q[4]), "f"(q[5]), "f"(q[6]), "f"(q[7]));
    } else {
        asm("{ .reg .b8 t0, t1, t2, t3;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1; cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5; cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n"
            "mov.b32 %0, {t0, t1, t2, t3}; }"
            : "=r"(out) : "f"(q[0]), "f"(q[1]), "f"(q[2]), "f"(q[3]), "f"(q[4]), "f"(q[5]), "f"(q[6]), "f"(q[7]));
    }
    return out;
}

// A whole block -> eight bytes of codes.  The reciprocal sequence runs for every block (its operands are
// harmless where it does not apply: rtot is 0 there) and a single branch replaces the quotients of the rare
// blocks that need the IEEE division or have a zero scale, so the common path has no divergence region.
__device__ __forceinline__ uint2 nvfp4_codes16(const float (&v)[16], const Nvfp4Block& b, bool hi_first) {
    float q[16];
    const float2 r2 = make_float2(b.rtot, b.rtot), b2 = make_float2(b.tot, b.tot);
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
        const float2 a2 = make_float2(v[i], v[i + 1]);
        const float2 q0 = __fmul2_rn(a2, r2);
        const float2 e = __ffma2_rn(b2, q0, make_float2(-a2.x, -a2.y));
        const float2 qq = __ffma2_rn(make_float2(-e.x, -e.y), r2, q0);
        q[i] = qq.x; q[i + 1] = qq.y;
    }
    if (!b.fast) {
        if (b.tot == 0.0f) return make_uint2(0u, 0u);
#pragma unroll
        for (int i = 0; i < 16; ++i) q[i] = __fdiv_rn(v[i], b.tot);
    }
    uint2 out;
    if (hi_first) {
        asm("{ .reg .b8 t0, t1, t2, t3;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t0, %1, %2; cvt.rn.satfinite.e2m1x2.f32 t1, %3, %4;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t2, %5, %6; cvt.rn.satfinite.e2m1x2.f32 t3, %7, %8;\n"
            "mov.b32 %0, {t0, t1, t2, t3}; }"
            : "=r"(out.x) : "f"(q[0]), "f"(q[1]), "f"(q[2]), "f"(q[3]), "f"(q[4]), "f"(q[5]), "f"(q[6]), "f"(q[7]));
        asm("{ .reg .b8 t0, t1, t2, t3;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t0, %1, %2; cvt.rn.satfinite.e2m1x2.f32 t1, %3, %4;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t2, %5, %6; cvt.rn.satfinite.e2m1x2.f32 t3, %7, %8;\n"
            "mov.b32 %0, {t0, t1, t2, t3}; }"
            : "=r"(out.y) : "f"(q[8]), "f"(q[9]), "f"(q[10]), "f"(q[11]), "f"(q[12]), "f"(q[13]), "f"(q[14]), "f"(q[15]));
    } else {
        asm("{ .reg .b8 t0, t1, t2, t3;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1; cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5; cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n"
            "mov.b32 %0, {t0, t1, t2, t3}; }"
            : "=r"(out.x) : "f"(q[0]), "f"(q[1]), "f"(q[2]), "f"(q[3]), "f"(q[4]), "f"(q[5]), "f"(q[6]), "f"(q[7]));
        asm("{ .reg .b8 t0, t1, t2, t3;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1; cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5; cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n"
            "mov.b32 %0, {t0, t1, t2, t3}; }"
            : "=r"(out.y) : "f"(q[8]), "f"(q[9]), "f"(q[10]), "f"(q[11]), "f"(q[12]), "f"(q[13]), "f"(q[14]), "f"(q[15]));
    }
    return out;
}

// This lane holds 8 of the 16 elements of a block (its partner is lane^1).  Returns 4 bytes of
// codes and the block's scale byte.  Must be called by all 32 lanes.
template <bool kExactDiv = false>
__device__ __forceinline__ uint32_t nvfp4_encode_half_block(const float (&v)[8], const Nvfp4Ctx& c, bool hi_first,
                                                            uint32_t& s8) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const Nvfp4Block b = nvfp4_block_scale<kExactDiv>(amax, c);
    s8 = b.s8;
    return nvfp4_codes8(v, b, hi_first);
}

// A whole 16-element block held by one thread -> 8 bytes of codes and the scale byte.
template <bool kExactDiv = false>
__device__ __forceinline__ uint2 nvfp4_encode_block(const float (&v)[16], const Nvfp4Ctx& c, bool hi_first, uint32_t& s8) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const Nvfp4Block b = nvfp4_block_scale<kExactDiv>(amax, c);
    s8 = b.s8;
    float lo[8], hi[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { lo[i] = v[i]; hi[i] = v[8 + i]; }
    return make_uint2(nvfp4_codes8(lo, b, hi_first), nvfp4_codes8(hi, b, hi_first));
}

// The same result through nvfp4_codes16: fewer instructions and no divergence region on the common path, which
// pays in the instruction-bound fused norm -> quantize kernels (the HBM-bound stand-alone quantizer measured
// 8 % faster with the form above).
__device__ __forceinline__ uint2 nvfp4_encode_block_lean(const float (&v)[16], const Nvfp4Ctx& c, bool hi_first, uint32_t& s8) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const Nvfp4Block b = nvfp4_block_scale<false>(amax, c);
    s8 = b.s8;
    return nvfp4_codes16(v, b, hi_first);
}

// nvfp4_encode_block_lean with the scale byte, too, on a straight-line common path; same bytes.
__device__ __forceinline__ uint2 nvfp4_encode_block_straight(const float (&v)[16], const Nvfp4Ctx& c, bool hi_first, uint32_t& s8) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    // Common path, straight-line: scale byte and divisor through the reciprocal sequence, whether or not it
    // applies; one test at the end sends the rare blocks (and tensors) where it does not through the IEEE
    // divisions instead (the same conditions as nvfp4_block_scale).
    const float bs = div_by_reciprocal(amax, 6.0f, 0.16666667163372040f /* RN(1/6) */);
    const float sbs = fminf(div_by_reciprocal(bs, c.g, c.rg), 448.0f);
    s8 = cvt_e4m3x2(0.0f, sbs) & 0xffu;
    const float tot = __fmul_rn(c.g, e4m3_to_f32(s8));
    const uint32_t u = __float_as_uint(tot);
    const float r = __frcp_rn(tot);
    // 2^-64 <= tot < 2^65 (one unsigned comparison on the bits), significand not all ones, amax < 2^60
    const bool fast = c.fast && (u - (63u << 23)) < (129u << 23) && (u & 0x7fffffu) != 0x7fffffu && amax < 1152921504606846976.0f;
    float q[16];
    const float2 r2 = make_float2(r, r), b2 = make_float2(tot, tot);
#pragma unroll
    for (int i = 0; i < 16; i += 2) {   // div_by_reciprocal on pairs
        const float2 a2 = make_float2(v[i], v[i + 1]);
        const float2 q0 = __fmul2_rn(a2, r2);
        const float2 e = __ffma2_rn(b2, q0, make_float2(-a2.x, -a2.y));
        const float2 qq = __ffma2_rn(make_float2(-e.x, -e.y), r2, q0);
        q[i] = qq.x; q[i + 1] = qq.y;
    }
    if (!fast) {
        const Nvfp4Block b = nvfp4_block_scale<true>(amax, c);
        s8 = b.s8;
        if (b.tot == 0.0f) return make_uint2(0u, 0u);
#pragma unroll
        for (int i = 0; i < 16; ++i) q[i] = __fdiv_rn(v[i], b.tot);
    }
    uint2 out;
    if (hi_first) {
        asm("{ .reg .b8 t0, t1, t2, t3;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t0, %1, %2; cvt.rn.satfinite.e2m1x2.f32 t1, %3, %4;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t2, %5, %6; cvt.rn.satfinite.e2m1x2.f32 t3, %7, %8;\n"
            "mov.b32 %0, {t0, t1, t2, t3}; }"
            : "=r"(out.x) : "f"(q[0]), "f"(q[1]), "f"(q[2]), "f"(q[3]), "f"(q[4]), "f"(q[5]), "f"(q[6]), "f"(q[7]));
        asm("{ .reg .b8 t0, t1, t2, t3;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t0, %1, %2; cvt.rn.satfinite.e2m1x2.f32 t1, %3, %4;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t2, %5, %6; cvt.rn.satfinite.e2m1x2.f32 t3, %7, %8;\n"
            "mov.b32 %0, {t0, t1, t2, t3}; }"
            : "=r"(out.y) : "f"(q[8]), "f"(q[9]), "f"(q[10]), "f"(q[11]), "f"(q[12]), "f"(q[13]), "f"(q[14]), "f"(q[15]));
    } else {
        asm("{ .reg .b8 t0, t1, t2, t3;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1; cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5; cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n"
            "mov.b32 %0, {t0, t1, t2, t3}; }"
            : "=r"(out.x) : "f"(q[0]), "f"(q[1]), "f"(q[2]), "f"(q[3]), "f"(q[4]), "f"(q[5]), "f"(q[6]), "f"(q[7]));
        asm("{ .reg .b8 t0, t1, t2, t3;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1; cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n"
            "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5; cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n"
            "mov.b32 %0, {t0, t1, t2, t3}; }"
            : "=r"(out.y) : "f"(q[8]), "f"(q[9]), "f"(q[10]), "f"(q[11]), "f"(q[12]), "f"(q[13]), "f"(q[14]), "f"(q[15]));
    }
    return out;
}

// ---- 256-bit global accesses (sm_100) -------------------------------------------------------
__device__ __forceinline__ void ldg256(const void* p, uint32_t (&r)[8]) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "l"(p));
}
__device__ __forceinline__ void stg256(void* p, const uint32_t (&r)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"l"(p), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

// 16 consecutive elements (32-byte aligned) as fp32.
template <typename T>
__device__ __forceinline__ void load16(const T* __restrict__ p, float (&v)[16]);
template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* __restrict__ p, float (&v)[16]) {
    uint32_t w[8];
    ldg256(p, w);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <>
__device__ __forceinline__ void load16<__half>(const __half* __restrict__ p, float (&v)[16]) {
    uint32_t w[8];
    ldg256(p, w);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
template <>
__device__ __forceinline__ void load16<float>(const float* __restrict__ p, float (&v)[16]) {
    uint32_t w[8];
    ldg256(p, w);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(w[i]);
    ldg256(p + 8, w);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[8 + i] = __uint_as_float(w[i]);
}

// 16 consecutive elements kept packed in registers (8 registers for 16-bit types, 16 for fp32).
template <typename T> struct Raw16 { uint32_t w[8]; };
template <> struct Raw16<float> { uint32_t w[16]; };

template <typename T>
__device__ __forceinline__ void load_raw16(const T* __restrict__ p, Raw16<T>& r) { ldg256(p, r.w); }
template <>
__device__ __forceinline__ void load_raw16<float>(const float* __restrict__ p, Raw16<float>& r) {
    uint32_t a[8], b[8];
    ldg256(p, a);
    ldg256(p + 8, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) { r.w[i] = a[i]; r.w[8 + i] = b[i]; }
}
template <typename T>
__device__ __forceinline__ void zero_raw16(Raw16<T>& r) {
#pragma unroll
    for (int i = 0; i < (int)(sizeof(r.w) / 4); ++i) r.w[i] = 0u;
}
__device__ __forceinline__ void unpack16(const Raw16<__nv_bfloat16>& r, float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[2 * i] = __uint_as_float(r.w[i] << 16);
        v[2 * i + 1] = __uint_as_float(r.w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void unpack16(const Raw16<__half>& r, float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&r.w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void unpack16(const Raw16<float>& r, float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r.w[i]);
}

// 16 consecutive fp32 values rounded to T and stored (32-byte aligned).
template <typename T>
__device__ __forceinline__ void store16(T* __restrict__ p, const float (&v)[16]);
template <>
__device__ __forceinline__ void store16<__nv_bfloat16>(__nv_bfloat16* __restrict__ p, const float (&v)[16]) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    stg256(p, w);
}
template <>
__device__ __forceinline__ void store16<__half>(__half* __restrict__ p, const float (&v)[16]) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    stg256(p, w);
}
template <>
__device__ __forceinline__ void store16<float>(float* __restrict__ p, const float (&v)[16]) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = __float_as_uint(v[i]);
    stg256(p, w);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = __float_as_uint(v[8 + i]);
    stg256(p + 8, w);
}

// Four bytes of E2M1 codes -> eight fp32 values in element order.
__device__ __forceinline__ void e2m1x8_to_f32(uint32_t codes, bool hi_first, float (&v)[8]) {
    uint32_t h[4];
    asm("{ .reg .b8 t0, t1, t2, t3; mov.b32 {t0, t1, t2, t3}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, t0; cvt.rn.f16x2.e2m1x2 %1, t1;\n"
        "cvt.rn.f16x2.e2m1x2 %2, t2; cvt.rn.f16x2.e2m1x2 %3, t3; }"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3]) : "r"(codes));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[i]));  // x = low nibble, y = high nibble
        v[2 * i] = hi_first ? f.y : f.x;
        v[2 * i + 1] = hi_first ? f.x : f.y;
    }
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

// MXFP8: eight elements of a block whose amax is already known -> eight E4M3 bytes and the E8M0 byte.
__device__ __forceinline__ uint2 mxfp8_encode8(const float (&v)[8], float amax, uint32_t& e) {
    e = 0;
    uint32_t w[2] = {0u, 0u};
    if (amax != 0.0f) {
        e = mx_scale_byte(amax);
        if (e != 0u) {
            const float inv = __uint_as_float(e == 254u ? 0x00400000u : ((254u - e) << 23));  // 2^(127-e)
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

// MXFP8: this lane holds 8 of the 32 elements of a block (lanes ^1, ^2 hold the
// rest).  Returns 8 E4M3 bytes and the block's E8M0 byte (0 for an all-zero block).
__device__ __forceinline__ uint2 mxfp8_encode_quarter_block(const float (&v)[8], uint32_t& e) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    return mxfp8_encode8(v, amax, e);
}

}  // namespace ck
