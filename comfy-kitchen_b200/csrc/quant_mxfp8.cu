// MXFP8 quantize / dequantize for sm_100a.
//
// Format: 32-element blocks along a row, E4M3 data, one E8M0 (power-of-two)
// scale byte per block.  Arithmetic follows the reference's eager backend
// (comfy_kitchen/backends/eager/quantization.py:259-366):
//   r = max(amax/448, 2^-127);  e = clamp(ceil(log2 r) + 127, 0, 254)
//   zero block -> scale byte 0, data 0;  else data = e4m3_rne(clamp(x / 2^(e-127), +-448))
// ceil(log2 r) is taken from the bits of r (exponent, plus one when the mantissa
// is non-zero), which equals the reference wherever log2 is exact at powers of
// two.  x / 2^(e-127) is evaluated as x * 2^(127-e): both are the correctly
// rounded value of the same real number.  e == 0 is decoded by the reference as
// a scale of 0.0 (division by zero -> +-448, 0/0 -> NaN byte 0xff); that corner
// (|amax| < 2^-118) is reproduced explicitly.
//
// Work decomposition (HBM-bound, 3.03125 algorithmic bytes per element for
// bf16): CTA = 256 threads = 128 rows x 256 columns; a thread owns 16 consecutive
// elements (one 256-bit load), two lanes a block (one shuffle for the amax), and
// writes 16 bytes; 16 rows per step, four steps in flight.  Scale bytes
// are staged in shared memory in the GEMM's 128x4 tiled order (two 512-byte
// tiles per CTA) and leave as 16-byte stores, padding included.
#include "ck_common.cuh"

namespace ck {
namespace {

constexpr int kTileRows = 128;
constexpr int kTileCols = 256;
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kSfTiles = kTileCols / 128;

// Scalar loader: 16 elements with bounds checks, zero beyond the source.
template <typename T>
__device__ __forceinline__ void load16_guarded(const T* __restrict__ x, int64_t row, int64_t col, int64_t orig_rows,
                                               int64_t orig_cols, float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        int64_t c = col + i;
        v[i] = (row < orig_rows && c < orig_cols) ? Elem<T>::to_f32(x[row * orig_cols + c]) : 0.0f;
    }
}

// A thread owns 16 consecutive elements (one 256-bit load for 16-bit inputs), two neighbouring lanes a
// 32-element block (one shuffle for its amax); 16 threads cover a 256-column row segment, so a 256-thread CTA
// takes 16 rows per step and four steps are in flight per thread.
template <typename T, bool kVec>
__global__ void __launch_bounds__(kThreads)
quantize_mxfp8_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int64_t rows,
                      int64_t cols, int64_t orig_rows, int64_t orig_cols, int64_t sf_cpad) {
    __shared__ __align__(16) uint8_t s_sf[kSfTiles * 512];
    const int tid = threadIdx.x;
    const int seg = tid & 15;          // 16-element segment inside the 256-column tile
    const int sub = tid >> 4;          // row inside one step
    constexpr int kRowsPerStep = kThreads / 16;
    const int64_t row0 = (int64_t)blockIdx.y * kTileRows;
    const int64_t col = (int64_t)blockIdx.x * kTileCols + seg * 16;

    reinterpret_cast<uint32_t*>(s_sf)[tid] = 0u;
    __syncthreads();

    const bool col_ok = col < cols;
    const int blk_in_tile = seg >> 1;  // 32-element block index inside the tile (0..7)

    constexpr int kUnroll = 4;
#pragma unroll 1
    for (int it = 0; it < kTileRows / kRowsPerStep; it += kUnroll) {
        Raw16<T> raw[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t row = row0 + (it + u) * kRowsPerStep + sub;
            if (kVec) {
                if (col < orig_cols && row < orig_rows) load_raw16<T>(x + row * orig_cols + col, raw[u]);
                else zero_raw16<T>(raw[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int r_in_tile = (it + u) * kRowsPerStep + sub;
            const int64_t row = row0 + r_in_tile;
            float v[16];
            if (kVec) unpack16(raw[u], v);
            else load16_guarded<T>(x, row, col, orig_rows, orig_cols, v);
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            float lo[8], hi[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { lo[i] = v[i]; hi[i] = v[8 + i]; }
            uint32_t e;
            const uint2 p0 = mxfp8_encode8(lo, amax, e), p1 = mxfp8_encode8(hi, amax, e);
            if (col_ok && row < rows) {
                *reinterpret_cast<uint4*>(q + row * cols + col) = make_uint4(p0.x, p0.y, p1.x, p1.y);
                if ((seg & 1) == 0)
                    s_sf[(blk_in_tile >> 2) * 512 + sf_tile_offset(r_in_tile, blk_in_tile & 3)] = (uint8_t)e;
            }
        }
    }
    __syncthreads();

    if (tid < kSfTiles * 32) {
        const int t = tid >> 5;
        const int64_t tile_col = ((int64_t)blockIdx.x * kTileCols >> 7) + t;
        if (tile_col < (sf_cpad >> 2)) {
            uint8_t* dst = sf + ((int64_t)blockIdx.y * (sf_cpad >> 2) + tile_col) * 512 + (tid & 31) * 16;
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(s_sf + t * 512 + (tid & 31) * 16);
        }
    }
}

// out = (float(q) * 2^(e-127)).to(T), e == 0 decoding to a scale of 0.0
// (comfy_kitchen/backends/eager/quantization.py:329-366, float_utils.py:376-382).
template <typename T>
__global__ void __launch_bounds__(kThreads)
dequantize_mxfp8_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sf, T* __restrict__ out,
                        int64_t rows, int64_t cols, int64_t sf_cpad, const bool vec32) {
    __shared__ __align__(16) uint8_t s_sf[kSfTiles * 512];
    const int tid = threadIdx.x;
    const int64_t row0 = (int64_t)blockIdx.y * kTileRows;
    const int64_t col0 = (int64_t)blockIdx.x * kTileCols;

    if (tid < kSfTiles * 32) {
        const int t = tid >> 5;
        const int64_t tile_col = (col0 >> 7) + t;
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (tile_col < (sf_cpad >> 2))
            val = *reinterpret_cast<const uint4*>(sf + ((int64_t)blockIdx.y * (sf_cpad >> 2) + tile_col) * 512 +
                                                  (tid & 31) * 16);
        *reinterpret_cast<uint4*>(s_sf + t * 512 + (tid & 31) * 16) = val;
    }
    __syncthreads();

    // a thread owns 16 consecutive elements: one 16-byte load, 32 (16-bit outputs) or 64 bytes stored; four rows in flight
    const int seg = tid & 15, sub = tid >> 4;
    constexpr int kRowsPerStep = kThreads / 16;
    const int64_t col = col0 + seg * 16;
    if (col >= cols) return;
    const int blk_in_tile = seg >> 1;
    constexpr int kUnroll = 4;
#pragma unroll 1
    for (int it = 0; it < kTileRows / kRowsPerStep; it += kUnroll) {
        uint4 data[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t row = row0 + (it + u) * kRowsPerStep + sub;
            data[u] = make_uint4(0u, 0u, 0u, 0u);
            if (row < rows) data[u] = *reinterpret_cast<const uint4*>(q + row * cols + col);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int r_in_tile = (it + u) * kRowsPerStep + sub;
            const int64_t row = row0 + r_in_tile;
            if (row >= rows) continue;
            const uint32_t e = s_sf[(blk_in_tile >> 2) * 512 + sf_tile_offset(r_in_tile, blk_in_tile & 3)];
            const float s = e == 0u ? 0.0f : __uint_as_float(e << 23);
            const uint32_t w[4] = {data[u].x, data[u].y, data[u].z, data[u].w};
            float v[16];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 f = e4m3x2_to_f32x2(w[i >> 1] >> (16 * (i & 1)));
                v[2 * i] = __fmul_rn(f.x, s);
                v[2 * i + 1] = __fmul_rn(f.y, s);
            }
            T* dst = out + row * cols + col;
            if (vec32) {
                store16<T>(dst, v);
            } else {
                float lo[8], hi[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) { lo[i] = v[i]; hi[i] = v[8 + i]; }
                store8<T>(dst, lo);
                store8<T>(dst + 8, hi);
            }
        }
    }
}

template <typename T>
int launch_quantize(const void* x, uint8_t* q, uint8_t* sf, int64_t rows, int64_t cols, int64_t orig_rows,
                    int64_t orig_cols, cudaStream_t stream) {
    const int64_t sf_cpad = round_up(cols / 32, 4);
    dim3 grid((unsigned)ceil_div(sf_cpad * 32, kTileCols), (unsigned)ceil_div(rows, kTileRows));
    const bool vec = aligned32(x) && (orig_cols % 16 == 0);   // 256-bit loads of whole 16-element segments
    if (vec)
        quantize_mxfp8_kernel<T, true><<<grid, kThreads, 0, stream>>>((const T*)x, q, sf, rows, cols, orig_rows, orig_cols, sf_cpad);
    else
        quantize_mxfp8_kernel<T, false><<<grid, kThreads, 0, stream>>>((const T*)x, q, sf, rows, cols, orig_rows, orig_cols, sf_cpad);
    return launch_status("quantize_mxfp8");
}

template <typename T>
int launch_dequantize(const uint8_t* q, const uint8_t* sf, void* out, int64_t rows, int64_t cols, cudaStream_t stream) {
    const int64_t sf_cpad = round_up(cols / 32, 4);
    dim3 grid((unsigned)ceil_div(cols, kTileCols), (unsigned)ceil_div(rows, kTileRows));
    // (256-bit stores need a 32-byte aligned output; rows are multiples of 32 elements)
    dequantize_mxfp8_kernel<T><<<grid, kThreads, 0, stream>>>(q, sf, (T*)out, rows, cols, sf_cpad, aligned32(out));
    return launch_status("dequantize_mxfp8");
}

}  // namespace
}  // namespace ck

extern "C" int launch_quantize_mxfp8_kernel(const void* input, void* output, void* block_scales, int64_t num_rows,
                                            int64_t num_cols, int64_t orig_rows, int64_t orig_cols,
                                            int input_dtype_code, cudaStream_t stream) {
    using namespace ck;
    if (!input || !output || !block_scales) CK_FAIL(CK_ERR_NULL, "quantize_mxfp8: null pointer");
    if (num_rows <= 0 || num_cols <= 0 || num_cols % 32 != 0 || orig_rows > num_rows || orig_cols > num_cols ||
        orig_rows <= 0 || orig_cols <= 0)
        CK_FAIL(CK_ERR_SHAPE, "quantize_mxfp8: bad shape rows=%lld cols=%lld orig=%lldx%lld (cols must be a multiple of 32)",
                (long long)num_rows, (long long)num_cols, (long long)orig_rows, (long long)orig_cols);
    if (ceil_div(num_rows, 128) > 65535) CK_FAIL(CK_ERR_SHAPE, "quantize_mxfp8: more than 65535*128 rows");
    if (!aligned16(block_scales) || (reinterpret_cast<uintptr_t>(output) & 7u))
        CK_FAIL(CK_ERR_ALIGN, "quantize_mxfp8: scales must be 16-byte aligned, data 8-byte aligned");
    auto* q = static_cast<uint8_t*>(output);
    auto* sf = static_cast<uint8_t*>(block_scales);
    switch (input_dtype_code) {
    case CK_F32: return launch_quantize<float>(input, q, sf, num_rows, num_cols, orig_rows, orig_cols, stream);
    case CK_F16: return launch_quantize<__half>(input, q, sf, num_rows, num_cols, orig_rows, orig_cols, stream);
    case CK_BF16: return launch_quantize<__nv_bfloat16>(input, q, sf, num_rows, num_cols, orig_rows, orig_cols, stream);
    default: CK_FAIL(CK_ERR_DTYPE, "quantize_mxfp8: unsupported input dtype code %d", input_dtype_code);
    }
}

extern "C" int launch_dequantize_mxfp8_kernel(const void* input, const void* block_scales, void* output,
                                              int64_t num_rows, int64_t num_cols, int output_dtype_code,
                                              cudaStream_t stream) {
    using namespace ck;
    if (!input || !output || !block_scales) CK_FAIL(CK_ERR_NULL, "dequantize_mxfp8: null pointer");
    if (num_rows <= 0 || num_cols <= 0 || num_cols % 32 != 0)
        CK_FAIL(CK_ERR_SHAPE, "dequantize_mxfp8: bad shape %lldx%lld (cols must be a multiple of 32)",
                (long long)num_rows, (long long)num_cols);
    if (ceil_div(num_rows, 128) > 65535) CK_FAIL(CK_ERR_SHAPE, "dequantize_mxfp8: more than 65535*128 rows");
    if (!aligned16(block_scales) || !aligned16(output) || (reinterpret_cast<uintptr_t>(input) & 7u))
        CK_FAIL(CK_ERR_ALIGN, "dequantize_mxfp8: scales/output must be 16-byte aligned, data 8-byte aligned");
    auto* q = static_cast<const uint8_t*>(input);
    auto* sf = static_cast<const uint8_t*>(block_scales);
    switch (output_dtype_code) {
    case CK_F32: return launch_dequantize<float>(q, sf, output, num_rows, num_cols, stream);
    case CK_F16: return launch_dequantize<__half>(q, sf, output, num_rows, num_cols, stream);
    case CK_BF16: return launch_dequantize<__nv_bfloat16>(q, sf, output, num_rows, num_cols, stream);
    default: CK_FAIL(CK_ERR_DTYPE, "dequantize_mxfp8: unsupported output dtype code %d", output_dtype_code);
    }
}
