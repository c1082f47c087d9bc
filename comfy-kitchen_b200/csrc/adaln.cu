// AdaLN / RMSNorm for sm_100a, standalone and fused with the activation quantizers.
//
//   LayerNorm form: y = (x - mean) * rstd * (1 + scale) + shift      (rstd = 1/sqrt(var + eps), biased var)
//   RMSNorm form:   y = x * rstd * weight                            (rstd = 1/sqrt(mean(x^2) + eps))
// with fp32 statistics and one rounding to x's dtype at the end — the formulation
// of comfy_kitchen/backends/cuda/ops/adaln.cu:105-189; the eager definition is
// comfy_kitchen/backends/eager/adaln.py:11-14.  Modulation rows are grouped as in
// comfy_kitchen/backends/_modulation.py:12-57: row r reads row r / group.
//
// Fast path (D a multiple of 8, D <= 4096): one warp per row.  The row is read
// once with 128-bit loads and held in registers; mean and variance are two passes
// over registers (no E[x^2]-mean^2 cancellation); the result is either stored in
// x's dtype, or — fused variants — rounded to x's dtype in registers and pushed
// through the same block encoders as quantize_nvfp4 / quantize_mxfp8, so the
// packed output is byte-identical to "adaln kernel, then quantize kernel" while
// the intermediate activation never reaches HBM (2.5625 instead of 6.5625
// bytes per element for NVFP4).
#include "ck_common.cuh"

namespace ck {
namespace {

enum OutMode { kOutPlain = 0, kOutNvfp4 = 1, kOutMxfp8 = 2 };

struct NormArgs {
    const void* x;
    const void* scale;  // LayerNorm: AdaLN scale rows; RMSNorm: weight row(s) or null
    const void* shift;  // may be null
    void* out;          // plain: T[N,D]; nvfp4: bytes [N,D/2]; mxfp8: bytes [N,D]
    uint8_t* sf;        // tiled block scales (fused modes)
    const float* global_scale;  // nvfp4 only
    int64_t N, D;
    int64_t scale_group, shift_group;
    int64_t sf_cpad;
    float eps;
    int rms;
    int hi_first;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename T, int kNV, int kMode>
__global__ void __launch_bounds__(256)
norm_warp_kernel(const NormArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t D = a.D;
    const int nvec = (int)(D >> 3);  // 8-element vectors per row

    if (row >= a.N) {
        // rows that exist only as padding of the tiled scale buffer: zero their scale bytes
        if (kMode != kOutPlain && row < round_up(a.N, 128)) {
            for (int64_t c4 = lane; c4 < (a.sf_cpad >> 2); c4 += 32)
                *reinterpret_cast<uint32_t*>(a.sf + sf_offset(row, c4 * 4, a.sf_cpad)) = 0u;
        }
        return;
    }

    const T* __restrict__ x = static_cast<const T*>(a.x) + row * D;
    Raw8<T> raw[kNV];
#pragma unroll
    for (int i = 0; i < kNV; ++i) {
        const int v = i * 32 + lane;
        raw[i] = v < nvec ? load_raw8<T>(x + (int64_t)v * 8) : zero_raw8<T>();
    }

    float mean = 0.0f;
    if (!a.rms) {
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < kNV; ++i) {
            float f[8];
            unpack8(raw[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) s += f[j];
        }
        mean = warp_sum(s) / (float)D;
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < kNV; ++i) {
        if (i * 32 + lane < nvec) {
            float f[8];
            unpack8(raw[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float d = f[j] - mean;
                ss = fmaf(d, d, ss);
            }
        }
    }
    const float rstd = rsqrtf(warp_sum(ss) / (float)D + a.eps);

    const T* __restrict__ sc = a.scale ? static_cast<const T*>(a.scale) + (row / a.scale_group) * D : nullptr;
    const T* __restrict__ sh = a.shift ? static_cast<const T*>(a.shift) + (row / a.shift_group) * D : nullptr;
    const Nvfp4Ctx ctx = nvfp4_ctx(kMode == kOutNvfp4 ? __ldg(a.global_scale) : 1.0f);

#pragma unroll
    for (int i = 0; i < kNV; ++i) {
        const int v = i * 32 + lane;
        const bool ok = v < nvec;
        float y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = 0.0f;
        if (ok) {
            float f[8], m[8], b[8];
            unpack8(raw[i], f);
            if (sc) load8<T>(sc + (int64_t)v * 8, m);
            if (sh) load8<T>(sh + (int64_t)v * 8, b);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float mul = sc ? (a.rms ? m[j] : 1.0f + m[j]) : 1.0f;
                const float add = sh ? b[j] : 0.0f;
                y[j] = fmaf((f[j] - mean) * rstd, mul, add);
            }
        }
        if (kMode == kOutPlain) {
            if (ok) store8<T>(static_cast<T*>(a.out) + row * D + (int64_t)v * 8, y);
        } else {
            // the quantizers see the activation as it would have been stored
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = Elem<T>::round(y[j]);
            if (kMode == kOutNvfp4) {
                uint32_t s8;
                const uint32_t packed = nvfp4_encode_half_block(y, ctx, a.hi_first != 0, s8);
                if (!ok) s8 = 0u;
                // four scale bytes (lanes L, L+2, L+4, L+6) leave as one 32-bit store
                uint32_t w = s8;
                w |= __shfl_down_sync(0xffffffffu, s8, 2) << 8;
                w |= __shfl_down_sync(0xffffffffu, s8, 4) << 16;
                w |= __shfl_down_sync(0xffffffffu, s8, 6) << 24;
                if (ok) *reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(a.out) + row * (D >> 1) + (int64_t)v * 4) = packed;
                const int64_t c = (int64_t)i * 16 + (lane >> 1);  // block column of this lane pair
                if ((lane & 7) == 0 && c < a.sf_cpad)
                    *reinterpret_cast<uint32_t*>(a.sf + sf_offset(row, c, a.sf_cpad)) = w;
            } else {
                uint32_t e;
                const uint2 packed = mxfp8_encode_quarter_block(y, e);
                if (!ok) e = 0u;
                uint32_t w = e;
                w |= __shfl_down_sync(0xffffffffu, e, 4) << 8;
                w |= __shfl_down_sync(0xffffffffu, e, 8) << 16;
                w |= __shfl_down_sync(0xffffffffu, e, 12) << 24;
                if (ok) *reinterpret_cast<uint2*>(static_cast<uint8_t*>(a.out) + row * D + (int64_t)v * 8) = packed;
                const int64_t c = (int64_t)i * 8 + (lane >> 2);
                if ((lane & 15) == 0 && c < a.sf_cpad)
                    *reinterpret_cast<uint32_t*>(a.sf + sf_offset(row, c, a.sf_cpad)) = w;
            }
        }
    }
}

// Any D, any alignment: one CTA per row, x read twice (the second pass hits L2).
template <typename T>
__global__ void __launch_bounds__(256)
norm_generic_kernel(const NormArgs a) {
    __shared__ float red[8];
    __shared__ float bcast;
    const int64_t row = blockIdx.x;
    const int64_t D = a.D;
    const T* __restrict__ x = static_cast<const T*>(a.x) + row * D;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    auto block_sum = [&](float v) {
        v = warp_sum(v);
        __syncthreads();
        if (lane == 0) red[warp] = v;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.0f;
            for (int w = 0; w < 8; ++w) t += red[w];
            bcast = t;
        }
        __syncthreads();
        return bcast;
    };

    float mean = 0.0f;
    if (!a.rms) {
        float s = 0.0f;
        for (int64_t j = threadIdx.x; j < D; j += 256) s += Elem<T>::to_f32(x[j]);
        mean = block_sum(s) / (float)D;
    }
    float ss = 0.0f;
    for (int64_t j = threadIdx.x; j < D; j += 256) {
        const float d = Elem<T>::to_f32(x[j]) - mean;
        ss = fmaf(d, d, ss);
    }
    const float rstd = rsqrtf(block_sum(ss) / (float)D + a.eps);
    const T* __restrict__ sc = a.scale ? static_cast<const T*>(a.scale) + (row / a.scale_group) * D : nullptr;
    const T* __restrict__ sh = a.shift ? static_cast<const T*>(a.shift) + (row / a.shift_group) * D : nullptr;
    T* __restrict__ out = static_cast<T*>(a.out) + row * D;
    for (int64_t j = threadIdx.x; j < D; j += 256) {
        const float mul = sc ? (a.rms ? Elem<T>::to_f32(sc[j]) : 1.0f + Elem<T>::to_f32(sc[j])) : 1.0f;
        const float add = sh ? Elem<T>::to_f32(sh[j]) : 0.0f;
        out[j] = Elem<T>::from_f32(fmaf((Elem<T>::to_f32(x[j]) - mean) * rstd, mul, add));
    }
}

template <typename T, int kMode>
int launch_warp(const NormArgs& a, cudaStream_t stream) {
    const int need = (int)ceil_div(a.D, 256);  // vectors per lane
    const int64_t rows = kMode == kOutPlain ? a.N : round_up(a.N, 128);
    const unsigned grid = (unsigned)ceil_div(rows, 8);
#define CK_NORM_CASE(NV) \
    if (need <= NV) { norm_warp_kernel<T, NV, kMode><<<grid, 256, 0, stream>>>(a); return launch_status("adaln"); }
    CK_NORM_CASE(1)
    CK_NORM_CASE(2)
    CK_NORM_CASE(4)
    CK_NORM_CASE(8)
    CK_NORM_CASE(12)
    CK_NORM_CASE(16)
#undef CK_NORM_CASE
    CK_FAIL(CK_ERR_SHAPE, "adaln: row length %lld exceeds the fused path's limit of 4096", (long long)a.D);
}

bool warp_path_ok(const NormArgs& a) {
    return a.D % 8 == 0 && a.D <= 4096 && aligned16(a.x) && (!a.scale || aligned16(a.scale)) &&
           (!a.shift || aligned16(a.shift)) && aligned16(a.out);
}

template <typename T>
int launch_plain(const NormArgs& a, cudaStream_t stream) {
    if (warp_path_ok(a)) return launch_warp<T, kOutPlain>(a, stream);
    if (a.N > 0x7fffffffLL) CK_FAIL(CK_ERR_SHAPE, "adaln: too many rows");
    norm_generic_kernel<T><<<(unsigned)a.N, 256, 0, stream>>>(a);
    return launch_status("adaln");
}

int check_common(const char* what, const NormArgs& a, int dtype_code) {
    if (!a.x || !a.out) CK_FAIL(CK_ERR_NULL, "%s: null pointer", what);
    if (a.N <= 0 || a.D <= 0) CK_FAIL(CK_ERR_SHAPE, "%s: bad shape N=%lld D=%lld", what, (long long)a.N, (long long)a.D);
    if ((a.scale && (a.scale_group <= 0 || a.N % a.scale_group)) || (a.shift && (a.shift_group <= 0 || a.N % a.shift_group)))
        CK_FAIL(CK_ERR_SHAPE, "%s: modulation group must divide the row count", what);
    if (dtype_code != CK_F32 && dtype_code != CK_F16 && dtype_code != CK_BF16)
        CK_FAIL(CK_ERR_DTYPE, "%s: unsupported dtype code %d", what, dtype_code);
    return CK_OK;
}

}  // namespace
}  // namespace ck

extern "C" int launch_adaln_kernel(const void* x, const void* scale, const void* shift, void* out, int64_t N, int64_t D,
                                   int64_t scale_group, int64_t shift_group, float eps, int dtype_code,
                                   cudaStream_t stream) {
    using namespace ck;
    NormArgs a{x, scale, shift, out, nullptr, nullptr, N, D, scale_group, shift_group, 0, eps, 0, 1};
    if (!scale || !shift) CK_FAIL(CK_ERR_NULL, "adaln: null pointer");
    if (int rc = check_common("adaln", a, dtype_code)) return rc;
    switch (dtype_code) {
    case CK_F32: return launch_plain<float>(a, stream);
    case CK_F16: return launch_plain<__half>(a, stream);
    default: return launch_plain<__nv_bfloat16>(a, stream);
    }
}

extern "C" int launch_rmsnorm_kernel(const void* x, const void* weight, void* out, int64_t N, int64_t D, float eps,
                                     int dtype_code, cudaStream_t stream) {
    using namespace ck;
    NormArgs a{x, weight, nullptr, out, nullptr, nullptr, N, D, N, N, 0, eps, 1, 1};
    if (int rc = check_common("rmsnorm", a, dtype_code)) return rc;
    switch (dtype_code) {
    case CK_F32: return launch_plain<float>(a, stream);
    case CK_F16: return launch_plain<__half>(a, stream);
    default: return launch_plain<__nv_bfloat16>(a, stream);
    }
}

namespace ck {
namespace {
template <int kMode>
int launch_fused(NormArgs a, int dtype_code, cudaStream_t stream) {
    const char* what = kMode == kOutNvfp4 ? "adaln_quantize_nvfp4" : "adaln_quantize_mxfp8";
    if (int rc = check_common(what, a, dtype_code)) return rc;
    if (!a.sf || (kMode == kOutNvfp4 && !a.global_scale)) CK_FAIL(CK_ERR_NULL, "%s: null pointer", what);
    const int blk = kMode == kOutNvfp4 ? 16 : 32;
    if (a.D % blk != 0) CK_FAIL(CK_ERR_SHAPE, "%s: row length %lld must be a multiple of %d", what, (long long)a.D, blk);
    a.sf_cpad = round_up(a.D / blk, 4);
    if (!warp_path_ok(a) || (reinterpret_cast<uintptr_t>(a.sf) & 3u))
        CK_FAIL(CK_ERR_UNSUPPORTED, "%s: needs 16-byte aligned tensors and row length <= 4096", what);
    switch (dtype_code) {
    case CK_F32: return launch_warp<float, kMode>(a, stream);
    case CK_F16: return launch_warp<__half, kMode>(a, stream);
    default: return launch_warp<__nv_bfloat16, kMode>(a, stream);
    }
}
}  // namespace
}  // namespace ck

// norm_kind: 0 = LayerNorm + AdaLN modulation (scale, shift required), 1 = RMSNorm (scale = weight row or null).
extern "C" int launch_adaln_quantize_nvfp4_kernel(const void* x, const void* scale, const void* shift,
                                                  const void* global_scale, void* output, void* block_scales, int64_t N,
                                                  int64_t D, int64_t scale_group, int64_t shift_group, float eps,
                                                  int dtype_code, bool hi_first, int norm_kind, cudaStream_t stream) {
    using namespace ck;
    if (norm_kind == 0 && (!scale || !shift)) CK_FAIL(CK_ERR_NULL, "adaln_quantize_nvfp4: null modulation pointer");
    NormArgs a{x, scale, shift, output, static_cast<uint8_t*>(block_scales), static_cast<const float*>(global_scale),
               N, D, scale_group, shift_group, 0, eps, norm_kind != 0, hi_first ? 1 : 0};
    return launch_fused<kOutNvfp4>(a, dtype_code, stream);
}

extern "C" int launch_adaln_quantize_mxfp8_kernel(const void* x, const void* scale, const void* shift, void* output,
                                                  void* block_scales, int64_t N, int64_t D, int64_t scale_group,
                                                  int64_t shift_group, float eps, int dtype_code, int norm_kind,
                                                  cudaStream_t stream) {
    using namespace ck;
    if (norm_kind == 0 && (!scale || !shift)) CK_FAIL(CK_ERR_NULL, "adaln_quantize_mxfp8: null modulation pointer");
    NormArgs a{x, scale, shift, output, static_cast<uint8_t*>(block_scales), nullptr,
               N, D, scale_group, shift_group, 0, eps, norm_kind != 0, 1};
    return launch_fused<kOutMxfp8>(a, dtype_code, stream);
}
