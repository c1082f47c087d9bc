// NVFP4 quantize / dequantize for sm_100a.
//
// Format: 16-element blocks along a row, each block stored as 16 E2M1 codes
// (two per byte) plus one E4M3 block scale; one fp32 per-tensor scale g.
// Arithmetic follows the reference's eager backend so codes and scale bytes are
// bit-identical (comfy_kitchen/backends/eager/quantization.py:117-221):
//   amax -> bs = amax/6 -> sbs = min(bs/g, 448) -> s8 = e4m3_rne(sbs)
//   tot = g*float(s8);  tot == 0 -> codes 0;  else code = e2m1_rne(clamp(x/tot, +-6))
// All divisions are IEEE (this file is compiled without fast-math).
//
// Work decomposition (HBM-bound, 2.5625 algorithmic bytes per element for bf16):
// one CTA of 256 threads owns a tile of 128 rows x 256 columns.  A warp reads one
// 512-byte row segment per step with one 128-bit load per lane (8 elements = half
// a block; the two lanes of a block combine their amax with one shuffle), and
// writes 4 bytes of codes per lane.  The tile's block scales are staged in shared
// memory in the GEMM's 128x4 tiled order and leave as 16-byte stores, so every
// byte of the padded scale buffer is written by exactly one CTA (no memset pass).
#include "ck_common.cuh"

namespace ck {
namespace {

constexpr int kTileRows = 128;
constexpr int kTileCols = 256;
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kSfTiles = kTileCols / 64;  // 512-byte scale tiles per CTA tile

// Scalar tail loader: 8 elements with bounds checks, zero beyond the source.
template <typename T>
__device__ __forceinline__ void load8_guarded(const T* __restrict__ x, int64_t row, int64_t col, int64_t orig_rows,
                                              int64_t orig_cols, float (&v)[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int64_t c = col + i;
        v[i] = (row < orig_rows && c < orig_cols) ? Elem<T>::to_f32(x[row * orig_cols + c]) : 0.0f;
    }
}

template <typename T, bool kVec>
__global__ void __launch_bounds__(kThreads)
quantize_nvfp4_kernel(const T* __restrict__ x, const float* __restrict__ global_scale, uint8_t* __restrict__ q,
                      uint8_t* __restrict__ sf, int64_t rows, int64_t cols, int64_t orig_rows, int64_t orig_cols,
                      int64_t sf_cpad, bool hi_first) {
    __shared__ __align__(16) uint8_t s_sf[kSfTiles * 512];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t row0 = (int64_t)blockIdx.y * kTileRows;
    const int64_t col0 = (int64_t)blockIdx.x * kTileCols;
    const float g = __ldg(global_scale);

    // scale bytes of rows/columns outside the tensor must read as zero
    reinterpret_cast<uint2*>(s_sf)[tid] = make_uint2(0u, 0u);
    __syncthreads();

    const int64_t col = col0 + lane * 8;
    const bool col_ok = col < cols;
    const int blk_in_tile = lane >> 1;  // 16-element block index inside the 256-column tile

    constexpr int kUnroll = 4;
#pragma unroll 1
    for (int it = 0; it < kTileRows / kWarps; it += kUnroll) {
        float v[kUnroll][8];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t row = row0 + (it + u) * kWarps + warp;
            if (kVec) {
                if (col < orig_cols && row < orig_rows) {
                    load8<T>(x + row * orig_cols + col, v[u]);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[u][i] = 0.0f;
                }
            } else {
                load8_guarded<T>(x, row, col, orig_rows, orig_cols, v[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int r_in_tile = (it + u) * kWarps + warp;
            const int64_t row = row0 + r_in_tile;
            uint32_t s8;
            const uint32_t packed = nvfp4_encode_half_block(v[u], g, hi_first, s8);
            if (col_ok && row < rows) {
                *reinterpret_cast<uint32_t*>(q + row * (cols >> 1) + (col >> 1)) = packed;
                if ((lane & 1) == 0)
                    s_sf[(blk_in_tile >> 2) * 512 + sf_tile_offset(r_in_tile, blk_in_tile & 3)] = (uint8_t)s8;
            }
        }
    }
    __syncthreads();

    // 2 KB of staged scales -> 128 x 16-byte stores; tiles past the padded width are skipped
    if (tid < kSfTiles * 32) {
        const int t = tid >> 5;
        const int64_t tile_col = (col0 >> 6) + t;
        if (tile_col < (sf_cpad >> 2)) {
            uint8_t* dst = sf + ((int64_t)blockIdx.y * (sf_cpad >> 2) + tile_col) * 512 + (tid & 31) * 16;
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(s_sf + t * 512 + (tid & 31) * 16);
        }
    }
}

// Dequantize: lut[code] * (g * s8), each product rounded to the output dtype as
// the eager reference does (backends/eager/quantization.py:213-219).
template <typename T>
__global__ void __launch_bounds__(kThreads)
dequantize_nvfp4_kernel(const uint8_t* __restrict__ q, const float* __restrict__ global_scale,
                        const uint8_t* __restrict__ sf, T* __restrict__ out, int64_t rows, int64_t cols,
                        int64_t sf_cpad, bool hi_first) {
    __shared__ __align__(16) uint8_t s_sf[kSfTiles * 512];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t row0 = (int64_t)blockIdx.y * kTileRows;
    const int64_t col0 = (int64_t)blockIdx.x * kTileCols;

    if (tid < kSfTiles * 32) {
        const int t = tid >> 5;
        const int64_t tile_col = (col0 >> 6) + t;
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (tile_col < (sf_cpad >> 2))
            val = *reinterpret_cast<const uint4*>(sf + ((int64_t)blockIdx.y * (sf_cpad >> 2) + tile_col) * 512 +
                                                  (tid & 31) * 16);
        *reinterpret_cast<uint4*>(s_sf + t * 512 + (tid & 31) * 16) = val;
    }
    __syncthreads();

    const float g = Elem<T>::round(__ldg(global_scale));
    const int64_t col = col0 + lane * 8;
    if (col >= cols) return;
    const int blk_in_tile = lane >> 1;

#pragma unroll 4
    for (int it = 0; it < kTileRows / kWarps; ++it) {
        const int r_in_tile = it * kWarps + warp;
        const int64_t row = row0 + r_in_tile;
        if (row >= rows) break;
        const uint32_t codes = *reinterpret_cast<const uint32_t*>(q + row * (cols >> 1) + (col >> 1));
        const uint32_t s8 = s_sf[(blk_in_tile >> 2) * 512 + sf_tile_offset(r_in_tile, blk_in_tile & 3)];
        const float tot = Elem<T>::round(__fmul_rn(g, e4m3_to_f32(s8)));
        float v[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t byte = (codes >> (8 * i)) & 0xffu;
            const uint32_t first = hi_first ? (byte >> 4) : (byte & 0xfu);
            const uint32_t second = hi_first ? (byte & 0xfu) : (byte >> 4);
            v[2 * i] = __fmul_rn(e2m1_value(first), tot);
            v[2 * i + 1] = __fmul_rn(e2m1_value(second), tot);
        }
        store8<T>(out + row * cols + col, v);
    }
}

template <typename T>
int launch_quantize(const void* x, const float* g, uint8_t* q, uint8_t* sf, int64_t rows, int64_t cols,
                    int64_t orig_rows, int64_t orig_cols, bool hi_first, cudaStream_t stream) {
    const int64_t sf_cpad = round_up(cols / 16, 4);
    dim3 grid((unsigned)ceil_div(sf_cpad * 16, kTileCols), (unsigned)ceil_div(rows, kTileRows));
    const bool vec = aligned16(x) && (orig_cols % 8 == 0);
    if (vec)
        quantize_nvfp4_kernel<T, true><<<grid, kThreads, 0, stream>>>((const T*)x, g, q, sf, rows, cols, orig_rows,
                                                                      orig_cols, sf_cpad, hi_first);
    else
        quantize_nvfp4_kernel<T, false><<<grid, kThreads, 0, stream>>>((const T*)x, g, q, sf, rows, cols, orig_rows,
                                                                       orig_cols, sf_cpad, hi_first);
    return launch_status("quantize_nvfp4");
}

template <typename T>
int launch_dequantize(const uint8_t* q, const float* g, const uint8_t* sf, void* out, int64_t rows, int64_t cols,
                      bool hi_first, cudaStream_t stream) {
    const int64_t sf_cpad = round_up(cols / 16, 4);
    dim3 grid((unsigned)ceil_div(cols, kTileCols), (unsigned)ceil_div(rows, kTileRows));
    dequantize_nvfp4_kernel<T><<<grid, kThreads, 0, stream>>>(q, g, sf, (T*)out, rows, cols, sf_cpad, hi_first);
    return launch_status("dequantize_nvfp4");
}

}  // namespace
}  // namespace ck

extern "C" int launch_quantize_nvfp4_kernel(const void* input, const void* global_scale, void* output,
                                            void* block_scales, int64_t num_rows, int64_t num_cols,
                                            int64_t orig_rows, int64_t orig_cols, float epsilon,
                                            int input_dtype_code, bool hi_first, cudaStream_t stream) {
    using namespace ck;
    (void)epsilon;  // accepted and ignored, as in every backend of the reference
    if (!input || !global_scale || !output || !block_scales) CK_FAIL(CK_ERR_NULL, "quantize_nvfp4: null pointer");
    if (num_rows <= 0 || num_cols <= 0 || num_cols % 16 != 0 || orig_rows > num_rows || orig_cols > num_cols ||
        orig_rows <= 0 || orig_cols <= 0)
        CK_FAIL(CK_ERR_SHAPE, "quantize_nvfp4: bad shape rows=%lld cols=%lld orig=%lldx%lld (cols must be a multiple of 16)",
                (long long)num_rows, (long long)num_cols, (long long)orig_rows, (long long)orig_cols);
    if (ceil_div(num_rows, 128) > 65535) CK_FAIL(CK_ERR_SHAPE, "quantize_nvfp4: more than 65535*128 rows");
    if (!aligned16(block_scales) || (reinterpret_cast<uintptr_t>(output) & 3u))
        CK_FAIL(CK_ERR_ALIGN, "quantize_nvfp4: outputs must be 16-byte (scales) / 4-byte (codes) aligned");
    auto* g = static_cast<const float*>(global_scale);
    auto* q = static_cast<uint8_t*>(output);
    auto* sf = static_cast<uint8_t*>(block_scales);
    switch (input_dtype_code) {
    case CK_F32: return launch_quantize<float>(input, g, q, sf, num_rows, num_cols, orig_rows, orig_cols, hi_first, stream);
    case CK_F16: return launch_quantize<__half>(input, g, q, sf, num_rows, num_cols, orig_rows, orig_cols, hi_first, stream);
    case CK_BF16: return launch_quantize<__nv_bfloat16>(input, g, q, sf, num_rows, num_cols, orig_rows, orig_cols, hi_first, stream);
    default: CK_FAIL(CK_ERR_DTYPE, "quantize_nvfp4: unsupported input dtype code %d", input_dtype_code);
    }
}

extern "C" int launch_dequantize_nvfp4_kernel(const void* input, const void* global_scale, const void* block_scales,
                                              void* output, int64_t num_rows, int64_t num_cols,
                                              int output_dtype_code, bool hi_first, cudaStream_t stream) {
    using namespace ck;
    if (!input || !global_scale || !output || !block_scales) CK_FAIL(CK_ERR_NULL, "dequantize_nvfp4: null pointer");
    if (num_rows <= 0 || num_cols <= 0 || num_cols % 16 != 0)
        CK_FAIL(CK_ERR_SHAPE, "dequantize_nvfp4: bad shape %lldx%lld (cols must be a multiple of 16)",
                (long long)num_rows, (long long)num_cols);
    if (ceil_div(num_rows, 128) > 65535) CK_FAIL(CK_ERR_SHAPE, "dequantize_nvfp4: more than 65535*128 rows");
    if (!aligned16(block_scales) || !aligned16(output) || (reinterpret_cast<uintptr_t>(input) & 3u))
        CK_FAIL(CK_ERR_ALIGN, "dequantize_nvfp4: scales/output must be 16-byte aligned, codes 4-byte aligned");
    auto* q = static_cast<const uint8_t*>(input);
    auto* g = static_cast<const float*>(global_scale);
    auto* sf = static_cast<const uint8_t*>(block_scales);
    switch (output_dtype_code) {
    case CK_F32: return launch_dequantize<float>(q, g, sf, output, num_rows, num_cols, hi_first, stream);
    case CK_F16: return launch_dequantize<__half>(q, g, sf, output, num_rows, num_cols, hi_first, stream);
    case CK_BF16: return launch_dequantize<__nv_bfloat16>(q, g, sf, output, num_rows, num_cols, hi_first, stream);
    default: CK_FAIL(CK_ERR_DTYPE, "dequantize_nvfp4: unsupported output dtype code %d", output_dtype_code);
    }
}
