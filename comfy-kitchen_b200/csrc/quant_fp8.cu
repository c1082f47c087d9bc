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
