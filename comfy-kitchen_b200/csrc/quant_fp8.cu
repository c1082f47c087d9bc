// Per-tensor FP8 quantize / dequantize for sm_100a.
//
// quantize (comfy_kitchen/backends/eager/quantization.py:43-57):
//   inv = (1/scale) rounded to x's dtype;  t = x*inv rounded to x's dtype;
//   out = fp8_rne(clamp(t, +-max))           (max 448 for E4M3, 57344 for E5M2)
// The product of two bf16 (or two fp16) values is exact in fp32, so rounding the
// fp32 product once to the narrow type reproduces the reference's 16-bit
// multiply bit for bit.  (A true x/scale in fp32 does not: about 3 % of codes
// differ on bf16 inputs.)
// dequantize (same file :59-63): out = x.to(T) * scale.to(T), product in T.
//
// Pure streaming (3 bytes per element for 16-bit tensors): each thread moves 16
// elements per step as two fully coalesced 128-bit accesses on the wide side and
// two 64-bit accesses on the byte side; grid-stride over 4096-element chunks.
#include "ck_common.cuh"

namespace ck {
namespace {

constexpr int kThreads = 256;
constexpr int kChunk = kThreads * 16;  // elements per CTA step

template <bool kE4M3>
__device__ __forceinline__ uint32_t to_fp8x2(float hi, float lo) {
    return kE4M3 ? cvt_e4m3x2(hi, lo) : cvt_e5m2x2(hi, lo);
}

template <typename T, bool kE4M3>
__device__ __forceinline__ uint2 quantize8(const float (&v)[8], float inv) {
    constexpr float kMax = kE4M3 ? 448.0f : 57344.0f;
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float a = Elem<T>::round(__fmul_rn(v[2 * i], inv));
        float b = Elem<T>::round(__fmul_rn(v[2 * i + 1], inv));
        a = fminf(fmaxf(a, -kMax), kMax);
        b = fminf(fmaxf(b, -kMax), kMax);
        w[i >> 1] |= to_fp8x2<kE4M3>(b, a) << (16 * (i & 1));
    }
    return make_uint2(w[0], w[1]);
}

template <typename T, bool kE4M3>
__global__ void __launch_bounds__(kThreads)
quantize_fp8_kernel(const T* __restrict__ x, const float* __restrict__ scale, uint8_t* __restrict__ out, int64_t numel,
                    bool vec_ok) {
    constexpr float kMax = kE4M3 ? 448.0f : 57344.0f;
    const float inv = Elem<T>::round(__fdiv_rn(1.0f, __ldg(scale)));
    const int64_t full = vec_ok ? (numel / kChunk) * kChunk : 0;
    for (int64_t base = (int64_t)blockIdx.x * kChunk; base < full; base += (int64_t)gridDim.x * kChunk) {
        float v0[8], v1[8];
        const int64_t i0 = base + threadIdx.x * 8, i1 = i0 + kThreads * 8;
        load8<T>(x + i0, v0);
        load8<T>(x + i1, v1);
        *reinterpret_cast<uint2*>(out + i0) = quantize8<T, kE4M3>(v0, inv);
        *reinterpret_cast<uint2*>(out + i1) = quantize8<T, kE4M3>(v1, inv);
    }
    // tail (and the whole tensor when the pointers are not 16-byte aligned)
    for (int64_t i = full + (int64_t)blockIdx.x * kThreads + threadIdx.x; i < numel; i += (int64_t)gridDim.x * kThreads) {
        float t = Elem<T>::round(__fmul_rn(Elem<T>::to_f32(x[i]), inv));
        t = fminf(fmaxf(t, -kMax), kMax);
        out[i] = (uint8_t)(to_fp8x2<kE4M3>(0.0f, t) & 0xffu);
    }
}

template <bool kE4M3>
__device__ __forceinline__ float from_fp8(uint32_t b) {
    return kE4M3 ? e4m3_to_f32(b) : e5m2_to_f32(b);
}

template <typename T, bool kE4M3>
__device__ __forceinline__ void dequantize8(uint2 d, float s, float (&v)[8]) {
    const uint32_t w[2] = {d.x, d.y};
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(from_fp8<kE4M3>((w[i >> 2] >> (8 * (i & 3))) & 0xffu), s);
}

template <typename T, bool kE4M3>
__global__ void __launch_bounds__(kThreads)
dequantize_fp8_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scale, T* __restrict__ out,
                      int64_t numel, bool vec_ok) {
    const float s = Elem<T>::round(__ldg(scale));
    const int64_t full = vec_ok ? (numel / kChunk) * kChunk : 0;
    for (int64_t base = (int64_t)blockIdx.x * kChunk; base < full; base += (int64_t)gridDim.x * kChunk) {
        const int64_t i0 = base + threadIdx.x * 8, i1 = i0 + kThreads * 8;
        const uint2 d0 = *reinterpret_cast<const uint2*>(q + i0);
        const uint2 d1 = *reinterpret_cast<const uint2*>(q + i1);
        float v0[8], v1[8];
        dequantize8<T, kE4M3>(d0, s, v0);
        dequantize8<T, kE4M3>(d1, s, v1);
        store8<T>(out + i0, v0);
        store8<T>(out + i1, v1);
    }
    for (int64_t i = full + (int64_t)blockIdx.x * kThreads + threadIdx.x; i < numel; i += (int64_t)gridDim.x * kThreads)
        out[i] = Elem<T>::from_f32(__fmul_rn(from_fp8<kE4M3>(q[i]), s));
}

int grid_for(int64_t numel) {
    // enough CTAs to cover the tensor once, capped at a few waves of 148 SMs x 8 CTAs
    int64_t want = ceil_div(numel, kChunk);
    const int64_t cap = 148 * 8 * 4;
    if (want < 1) want = 1;
    return (int)(want > cap ? cap : want);
}

template <typename T>
int quantize_dispatch(const void* x, const float* scale, uint8_t* out, int64_t numel, int out_code, cudaStream_t st) {
    const bool vec_ok = aligned16(x) && ((reinterpret_cast<uintptr_t>(out) & 7u) == 0);
    const int grid = grid_for(numel);
    if (out_code == CK_E4M3)
        quantize_fp8_kernel<T, true><<<grid, kThreads, 0, st>>>((const T*)x, scale, out, numel, vec_ok);
    else
        quantize_fp8_kernel<T, false><<<grid, kThreads, 0, st>>>((const T*)x, scale, out, numel, vec_ok);
    return launch_status("quantize_fp8");
}

template <typename T>
int dequantize_dispatch(const uint8_t* q, const float* scale, void* out, int64_t numel, int in_code, cudaStream_t st) {
    const bool vec_ok = aligned16(out) && ((reinterpret_cast<uintptr_t>(q) & 7u) == 0);
    const int grid = grid_for(numel);
    if (in_code == CK_E4M3)
        dequantize_fp8_kernel<T, true><<<grid, kThreads, 0, st>>>(q, scale, (T*)out, numel, vec_ok);
    else
        dequantize_fp8_kernel<T, false><<<grid, kThreads, 0, st>>>(q, scale, (T*)out, numel, vec_ok);
    return launch_status("dequantize_fp8");
}

}  // namespace
// ---- stochastic rounding to FP8 -------------------------------------------------------------
// stochastic_rounding_fp8(x, rng, output_type) of the reference's eager backend
// (comfy_kitchen/backends/eager/quantization.py:66-114; its CUDA kernel is
// backends/cuda/ops/per_tensor_quantize.cu:121-161, which evaluates the same formula in fp32 and therefore
// differs from eager on inputs just below a power of two).  Eager works on x.half() in torch's half
// arithmetic: each operation evaluated in fp32 and rounded to fp16.  The device function makes every one of
// those roundings explicit; floor(log2|x|) as fp16 sees it is decided from the input's bits: for
// |x| = 2^k (1 + m/1024) the fp16 rounding of log2 reaches k + 1 when the mantissa code m is at or above a
// threshold set by how coarse fp16 is around k.
namespace {

__device__ __forceinline__ float h16(float v) { return __half2float(__float2half_rn(v)); }
__device__ __forceinline__ float pow2i(int n) { return __uint_as_float((uint32_t)(n + 127) << 23); }   // -126 <= n <= 127

__device__ __forceinline__ int floor_log2_half(uint32_t bits) {   // finite positive fp16 bits
    const int ef = (bits >> 10) & 0x1f, m = bits & 0x3ff;
    int k, thr;
    if (ef == 0) {   // fp16 subnormal: m * 2^-24
        k = 31 - __clz(m) - 24;
        thr = k == -15 ? 1022 : (k == -16 ? 511 : (k == -17 ? 255 : (1 << 30)));
    } else {
        k = ef - 15;
        thr = (k >= 8 || k <= -9) ? 1019 : ((k >= 4 || k <= -5) ? 1022 : ((k >= 2 || k <= -3) ? 1023 : (1 << 30)));
    }
    return k + (m >= thr ? 1 : 0);
}

template <bool kE4M3>
__device__ __forceinline__ uint32_t stochastic_round_one(float xin, uint32_t r) {
    constexpr int kEBits = kE4M3 ? 4 : 5, kMBits = kE4M3 ? 3 : 2, kBias = kE4M3 ? 7 : 15;
    constexpr float kMax = kE4M3 ? 448.0f : 57344.0f;
    const __half hx = __float2half_rn(xin);   // x.half()
    const float v = __half2float(hx);
    if (v != v) return 0xffu;
    const float a = fabsf(v);
    const float sign = a == 0.0f ? 0.0f : (v < 0.0f ? -1.0f : 1.0f);
    int e;   // clamp(floor(log2 a) + bias, 0, 2^E - 1)
    if (a == 0.0f) e = 0;
    else if (isinf(a)) e = (1 << kEBits) - 1;
    else e = min(max(floor_log2_half(__half_as_ushort(hx) & 0x7fffu) + kBias, 0), (1 << kEBits) - 1);
    const bool normal = e != 0;
    const float scale = h16(pow2i(e - kBias));   // 2^16 (e5m2, top exponent) is inf in fp16, as in eager
    float t;
    if (normal) {
        t = h16(__fdiv_rn(a, scale));
        t = h16(t - 1.0f);
        t = h16(t * (float)(1 << kMBits));
    } else {
        t = h16(a * pow2i(kBias - 1 + kMBits));   // a / 2^(-bias + 1 - M), exact
    }
    const float rr = (float)r * (1.0f / 256.0f);   // exact in fp16
    t = floorf(h16(t + rr));
    const float m = h16(t * (1.0f / (float)(1 << kMBits)));
    const float val = normal ? h16(scale * h16(1.0f + m)) : h16(pow2i(-kBias + 1) * m);
    float res = h16(sign * val);
    if (res != res) return 0xffu;
    res = fminf(fmaxf(res, -kMax), kMax);
    return (kE4M3 ? cvt_e4m3x2(0.0f, res) : cvt_e5m2x2(0.0f, res)) & 0xffu;
}

template <typename T, bool kE4M3>
__global__ void __launch_bounds__(256)
stochastic_rounding_fp8_kernel(const T* __restrict__ x, const uint8_t* __restrict__ rng, uint8_t* __restrict__ out,
                               int64_t numel, bool vec) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t done = 0;
    if (vec) {   // 8 elements per step: 8 random bytes in, 8 codes out
        const int64_t n8 = numel >> 3;
        for (int64_t i = tid; i < n8; i += stride) {
            float v[8];
            if (sizeof(T) == 4) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = Elem<T>::to_f32(x[i * 8 + j]);
            } else {
                load8<T>(x + i * 8, v);
            }
            const uint2 rb = *reinterpret_cast<const uint2*>(rng + i * 8);
            uint32_t lo = 0, hi = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                lo |= stochastic_round_one<kE4M3>(v[j], (rb.x >> (8 * j)) & 0xffu) << (8 * j);
                hi |= stochastic_round_one<kE4M3>(v[4 + j], (rb.y >> (8 * j)) & 0xffu) << (8 * j);
            }
            *reinterpret_cast<uint2*>(out + i * 8) = make_uint2(lo, hi);
        }
        done = n8 << 3;
    }
    for (int64_t i = done + tid; i < numel; i += stride)
        out[i] = (uint8_t)stochastic_round_one<kE4M3>(Elem<T>::to_f32(x[i]), rng[i]);
}

template <typename T>
int launch_stochastic(const void* x, const uint8_t* rng, uint8_t* out, int64_t numel, int out_code, cudaStream_t stream) {
    const bool vec = aligned16(x) && (reinterpret_cast<uintptr_t>(rng) & 7u) == 0 && (reinterpret_cast<uintptr_t>(out) & 7u) == 0;
    int64_t blocks = ceil_div(ceil_div(numel, (int64_t)8), (int64_t)256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    auto xt = static_cast<const T*>(x);
    if (out_code == CK_E4M3) stochastic_rounding_fp8_kernel<T, true><<<(unsigned)blocks, 256, 0, stream>>>(xt, rng, out, numel, vec);
    else stochastic_rounding_fp8_kernel<T, false><<<(unsigned)blocks, 256, 0, stream>>>(xt, rng, out, numel, vec);
    return launch_status("stochastic_rounding_fp8");
}

}  // namespace
}  // namespace ck

extern "C" int launch_quantize_fp8_kernel(const void* input, void* output, const void* scale, int64_t numel,
                                          int input_dtype_code, int output_dtype_code, cudaStream_t stream) {
    using namespace ck;
    if (numel == 0) return CK_OK;
    if (!input || !output || !scale) CK_FAIL(CK_ERR_NULL, "quantize_fp8: null pointer");
    if (numel < 0) CK_FAIL(CK_ERR_SHAPE, "quantize_fp8: negative element count");
    if (output_dtype_code != CK_E4M3 && output_dtype_code != CK_E5M2)
        CK_FAIL(CK_ERR_DTYPE, "quantize_fp8: output dtype code %d is not an FP8 type", output_dtype_code);
    auto* s = static_cast<const float*>(scale);
    auto* o = static_cast<uint8_t*>(output);
    switch (input_dtype_code) {
    case CK_F32: return quantize_dispatch<float>(input, s, o, numel, output_dtype_code, stream);
    case CK_F16: return quantize_dispatch<__half>(input, s, o, numel, output_dtype_code, stream);
    case CK_BF16: return quantize_dispatch<__nv_bfloat16>(input, s, o, numel, output_dtype_code, stream);
    default: CK_FAIL(CK_ERR_DTYPE, "quantize_fp8: unsupported input dtype code %d", input_dtype_code);
    }
}

extern "C" int launch_dequantize_fp8_kernel(const void* input, void* output, const void* scale, int64_t numel,
                                            int input_dtype_code, int output_dtype_code, cudaStream_t stream) {
    using namespace ck;
    if (numel == 0) return CK_OK;
    if (!input || !output || !scale) CK_FAIL(CK_ERR_NULL, "dequantize_fp8: null pointer");
    if (numel < 0) CK_FAIL(CK_ERR_SHAPE, "dequantize_fp8: negative element count");
    if (input_dtype_code != CK_E4M3 && input_dtype_code != CK_E5M2)
        CK_FAIL(CK_ERR_DTYPE, "dequantize_fp8: input dtype code %d is not an FP8 type", input_dtype_code);
    auto* s = static_cast<const float*>(scale);
    auto* q = static_cast<const uint8_t*>(input);
    switch (output_dtype_code) {
    case CK_F32: return dequantize_dispatch<float>(q, s, output, numel, input_dtype_code, stream);
    case CK_F16: return dequantize_dispatch<__half>(q, s, output, numel, input_dtype_code, stream);
    case CK_BF16: return dequantize_dispatch<__nv_bfloat16>(q, s, output, numel, input_dtype_code, stream);
    default: CK_FAIL(CK_ERR_DTYPE, "dequantize_fp8: unsupported output dtype code %d", output_dtype_code);
    }
}

// Replaces the reference's stochastic_rounding_fp8 binding (backends/cuda/ops/per_tensor_quantize.cu:121-161,
// which works in place on the random bytes); here `rng` is read and `output` written, numel bytes each.
extern "C" int launch_stochastic_rounding_fp8_kernel(const void* input, const void* rng, void* output, int64_t numel,
                                                     int input_dtype_code, int output_dtype_code, cudaStream_t stream) {
    using namespace ck;
    if (numel == 0) return CK_OK;
    if (!input || !rng || !output) CK_FAIL(CK_ERR_NULL, "stochastic_rounding_fp8: null pointer");
    if (numel < 0) CK_FAIL(CK_ERR_SHAPE, "stochastic_rounding_fp8: negative element count");
    if (output_dtype_code != CK_E4M3 && output_dtype_code != CK_E5M2)
        CK_FAIL(CK_ERR_DTYPE, "stochastic_rounding_fp8: output dtype code %d is not an FP8 type", output_dtype_code);
    auto* r = static_cast<const uint8_t*>(rng);
    auto* o = static_cast<uint8_t*>(output);
    switch (input_dtype_code) {
    case CK_F32: return launch_stochastic<float>(input, r, o, numel, output_dtype_code, stream);
    case CK_F16: return launch_stochastic<__half>(input, r, o, numel, output_dtype_code, stream);
    case CK_BF16: return launch_stochastic<__nv_bfloat16>(input, r, o, numel, output_dtype_code, stream);
    default: CK_FAIL(CK_ERR_DTYPE, "stochastic_rounding_fp8: unsupported input dtype code %d", input_dtype_code);
    }
}
