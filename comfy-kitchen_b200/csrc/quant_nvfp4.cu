// NVFP4 quantize / dequantize for sm_100a.
//
// Format: 16-element blocks along a row, each block stored as 16 E2M1 codes
// (two per byte) plus one E4M3 block scale; one fp32 per-tensor scale g.
// Arithmetic follows the reference's eager backend so codes and scale bytes are
// bit-identical (comfy_kitchen/backends/eager/quantization.py:117-221):
//   amax -> bs = amax/6 -> sbs = min(bs/g, 448) -> s8 = e4m3_rne(sbs)
//   tot = g*float(s8);  tot == 0 -> codes 0;  else code = e2m1_rne(clamp(x/tot, +-6))
// The divisions are IEEE-exact (ck_common.cuh: "NVFP4 block arithmetic"); this file
// is compiled without fast-math.
//
// Work decomposition (HBM-bound, 2.5625 algorithmic bytes per element for bf16):
// one CTA of 256 threads owns a tile of 128 rows x 256 columns.  A thread owns whole
// 16-element blocks: one 256-bit load in (two for fp32), 8 bytes of codes out; a
// warp covers two 512-byte row segments per step.  The tile's block scales are
// staged in shared memory in the GEMM's 128x4 tiled order and leave as 16-byte
// stores, so every byte of the padded scale buffer is written by exactly one CTA
// (no memset pass).
#include "ck_common.cuh"

namespace ck {

// 0 = reciprocal-sequence divisions (default), 1 = plain IEEE divisions everywhere.
// Both produce the same bytes; the switch exists so tests can check that on the device.

namespace {

constexpr int kTileRows = 128;
constexpr int kTileCols = 256;
constexpr int kThreads = 256;
constexpr int kRowsPerStep = kThreads / 16;  // 16 threads (one block each) cover a 256-column row segment
constexpr int kSfTiles = kTileCols / 64;     // 512-byte scale tiles per CTA tile

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

template <typename T, bool kVec, bool kExactDiv>
__global__ void __launch_bounds__(kThreads)
quantize_nvfp4_kernel(const T* __restrict__ x, const float* __restrict__ global_scale, uint8_t* __restrict__ q,
                      uint8_t* __restrict__ sf, int64_t rows, int64_t cols, int64_t orig_rows, int64_t orig_cols,
                      int64_t sf_cpad, bool hi_first) {
    __shared__ __align__(16) uint8_t s_sf[kSfTiles * 512];

    const int tid = threadIdx.x;
    const int blk = tid & 15;          // block index inside the 256-column tile
    const int sub = tid >> 4;          // row inside one step
    const int64_t row0 = (int64_t)blockIdx.y * kTileRows;
    const int64_t col = (int64_t)blockIdx.x * kTileCols + blk * 16;
    const Nvfp4Ctx ctx = nvfp4_ctx(__ldg(global_scale));

    // scale bytes of rows/columns outside the tensor must read as zero
    reinterpret_cast<uint2*>(s_sf)[tid] = make_uint2(0u, 0u);
    __syncthreads();

    const bool col_ok = col < cols;
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
            uint32_t s8;
            const uint2 packed = nvfp4_encode_block<kExactDiv>(v, ctx, hi_first, s8);
            if (col_ok && row < rows) {
                *reinterpret_cast<uint2*>(q + row * (cols >> 1) + (col >> 1)) = packed;
                s_sf[(blk >> 2) * 512 + sf_tile_offset(r_in_tile, blk & 3)] = (uint8_t)s8;
            }
        }
    }
    __syncthreads();

    // 2 KB of staged scales -> 128 x 16-byte stores; tiles past the padded width are skipped
    if (tid < kSfTiles * 32) {
        const int t = tid >> 5;
        const int64_t tile_col = ((int64_t)blockIdx.x * kTileCols >> 6) + t;
        if (tile_col < (sf_cpad >> 2)) {
            uint8_t* dst = sf + ((int64_t)blockIdx.y * (sf_cpad >> 2) + tile_col) * 512 + (tid & 31) * 16;
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(s_sf + t * 512 + (tid & 31) * 16);
        }
    }
}

// ---- quantizer with a gathered source and an optional activation ------------------------------
// The logical [rows, cols] input is the concatenation along columns of up to two segments.  Element
// (row, c) of a segment lives at  base + (c / group) * group_stride + row * row_stride + c % group
// (elements): group = the segment's width and group_stride = 0 describe a row-major matrix with any row
// pitch (a column slice of a wider matrix, say); group = head_dim, group_stride = tokens * head_dim,
// row_stride = head_dim describe attention's [heads, tokens, head_dim] output read as [tokens,
// heads * head_dim].  A segment may pass through GELU (tanh form) first; the activation is rounded to the
// input dtype before it is quantized, as if it had been stored.  Same tiling and the same block encoder as
// quantize_nvfp4_kernel, so without an activation the bytes equal a gather followed by that kernel.
struct QuantSegment {
    const void* base;
    int64_t cols, group, group_stride, row_stride;
    int act;   // 0 none, 1 gelu(tanh)
};

__device__ __forceinline__ float gelu_tanh(float x) {
    const float kBeta = 0.7978845608028654f, kKappa = 0.044715f;   // sqrt(2/pi)
    const float inner = kBeta * (x + kKappa * (x * x * x));
    return 0.5f * x * (1.0f + tanhf(inner));
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
quantize_nvfp4_gather_kernel(const QuantSegment s0, const QuantSegment s1, const float* __restrict__ global_scale,
                             uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int64_t rows, int64_t cols,
                             int64_t sf_cpad, bool hi_first) {
    __shared__ __align__(16) uint8_t s_sf[kSfTiles * 512];
    const int tid = threadIdx.x;
    const int blk = tid & 15, sub = tid >> 4;
    const int64_t row0 = (int64_t)blockIdx.y * kTileRows;
    const int64_t col = (int64_t)blockIdx.x * kTileCols + blk * 16;
    const Nvfp4Ctx ctx = nvfp4_ctx(__ldg(global_scale));
    reinterpret_cast<uint2*>(s_sf)[tid] = make_uint2(0u, 0u);
    __syncthreads();

    const bool col_ok = col < cols;
    // which segment this thread's blocks come from, and where they start in it (a block never straddles
    // segments or groups: all widths are multiples of 16)
    const bool second = col >= s0.cols;
    const QuantSegment& sg = second ? s1 : s0;
    const int64_t c = second ? col - s0.cols : col;
    const T* src = nullptr;
    int64_t row_stride = 0;
    int act = 0;
    if (col_ok) {
        src = static_cast<const T*>(sg.base) + (c / sg.group) * sg.group_stride + c % sg.group;
        row_stride = sg.row_stride;
        act = sg.act;
    }
    constexpr int kUnroll = 4;
#pragma unroll 1
    for (int it = 0; it < kTileRows / kRowsPerStep; it += kUnroll) {
        Raw16<T> raw[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t row = row0 + (it + u) * kRowsPerStep + sub;
            if (col_ok && row < rows) load_raw16<T>(src + row * row_stride, raw[u]);
            else zero_raw16<T>(raw[u]);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int r_in_tile = (it + u) * kRowsPerStep + sub;
            const int64_t row = row0 + r_in_tile;
            float v[16];
            unpack16(raw[u], v);
            if (act == 1) {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = Elem<T>::round(gelu_tanh(v[i]));
            }
            uint32_t s8;
            const uint2 packed = nvfp4_encode_block<false>(v, ctx, hi_first, s8);
            if (col_ok && row < rows) {
                *reinterpret_cast<uint2*>(q + row * (cols >> 1) + (col >> 1)) = packed;
                s_sf[(blk >> 2) * 512 + sf_tile_offset(r_in_tile, blk & 3)] = (uint8_t)s8;
            }
        }
    }
    __syncthreads();
    if (tid < kSfTiles * 32) {
        const int t = tid >> 5;
        const int64_t tile_col = ((int64_t)blockIdx.x * kTileCols >> 6) + t;
        if (tile_col < (sf_cpad >> 2)) {
            uint8_t* dst = sf + ((int64_t)blockIdx.y * (sf_cpad >> 2) + tile_col) * 512 + (tid & 31) * 16;
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(s_sf + t * 512 + (tid & 31) * 16);
        }
    }
}

// The same operator for large activated inputs.  GELU(tanh) with the accurate tanhf costs ~30 instructions per
// element and made the kernel above instruction-bound (2 TB/s); a 16-bit input has only 65536 possible values,
// so every CTA first tabulates round(gelu(x)) for all of them in shared memory (128 KB, filled with the very
// function the kernel above applies, hence the same bits) and then looks elements up: two 16-bit loads per
// pair instead of the arithmetic.  One persistent CTA of 1024 threads per SM; each quarter of it walks tiles
// of the kernel above with its own staging area and named barrier.  The fill costs 64 evaluations per thread,
// so the launcher takes this path only when the activated part is large (>= 8 Mi elements: with 14 M activated
// elements the table path measured 20.9 us against 26.6 us for the arithmetic).
constexpr int kLutThreads = 1024;
constexpr int kLutGroups = kLutThreads / kThreads;
constexpr int kLutSmem = 65536 * 2 + kLutGroups * kSfTiles * 512;

template <typename T>
__device__ __forceinline__ uint32_t gelu_bits(uint32_t bits);
// Most of the table needs no evaluation.  |x| >= 8: the tanh argument exceeds 24, tanhf is exactly +-1, so the
// result is x for positive and 0.5 * x * 0 = -0.0 for negative inputs.  bf16 with |x| < 2^-26: the tanh is below
// 2^-26 and 1 + tanh rounds to 1, so the result is 0.5 * x, an exponent decrement.  Infinities and NaNs take the
// arithmetic.  (The parity test compares the table path with the arithmetic kernel on all 65536 inputs.)
template <>
__device__ __forceinline__ uint32_t gelu_bits<__nv_bfloat16>(uint32_t bits) {
    const uint32_t e = (bits >> 7) & 0xffu;
    if (e >= 130u && e != 255u) return (bits & 0x8000u) ? 0x8000u : bits;
    if (e >= 2u && e <= 100u) return bits - 0x80u;
    const float y = Elem<__nv_bfloat16>::round(gelu_tanh(__uint_as_float(bits << 16)));
    return __float_as_uint(y) >> 16;
}
template <>
__device__ __forceinline__ uint32_t gelu_bits<__half>(uint32_t bits) {
    const uint32_t e = (bits >> 10) & 0x1fu;
    if (e >= 18u && e != 31u) return (bits & 0x8000u) ? 0x8000u : bits;
    const __half_raw in{(unsigned short)bits};
    const __half out = __float2half_rn(gelu_tanh(__half2float(__half(in))));
    return (uint32_t)__half_raw(out).x;
}

template <typename T>
__device__ __forceinline__ float lut_bits_to_f32(uint16_t b);
template <>
__device__ __forceinline__ float lut_bits_to_f32<__nv_bfloat16>(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
template <>
__device__ __forceinline__ float lut_bits_to_f32<__half>(uint16_t b) { return __half2float(__ushort_as_half(b)); }

template <typename T>
__global__ void __launch_bounds__(kLutThreads, 1)
quantize_nvfp4_gather_lut_kernel(const QuantSegment s0, const QuantSegment s1, const float* __restrict__ global_scale,
                                 uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int64_t rows, int64_t cols,
                                 int64_t sf_cpad, bool hi_first, int tiles_x, int64_t num_tiles) {
    extern __shared__ __align__(16) uint8_t lut_smem[];
    uint16_t* lut = reinterpret_cast<uint16_t*>(lut_smem);
    const int grp = threadIdx.x / kThreads, tid = threadIdx.x % kThreads;
    uint8_t* s_sf = lut_smem + 65536 * 2 + grp * (kSfTiles * 512);
    for (uint32_t i = threadIdx.x; i < 65536u; i += kLutThreads) lut[i] = (uint16_t)gelu_bits<T>(i);
    __syncthreads();

    const int blk = tid & 15, sub = tid >> 4;
    const Nvfp4Ctx ctx = nvfp4_ctx(__ldg(global_scale));
    const uint32_t bar_id = 1 + grp;
    for (int64_t tile = (int64_t)blockIdx.x * kLutGroups + grp; tile < num_tiles; tile += (int64_t)gridDim.x * kLutGroups) {
        const int64_t tile_x = tile % tiles_x, tile_y = tile / tiles_x;
        const int64_t row0 = tile_y * kTileRows;
        const int64_t col = tile_x * kTileCols + blk * 16;
        reinterpret_cast<uint2*>(s_sf)[tid] = make_uint2(0u, 0u);
        asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(kThreads) : "memory");

        const bool col_ok = col < cols;
        const bool second = col >= s0.cols;
        const QuantSegment& sg = second ? s1 : s0;
        const int64_t c = second ? col - s0.cols : col;
        const T* src = nullptr;
        int64_t row_stride = 0;
        int act = 0;
        if (col_ok) {
            src = static_cast<const T*>(sg.base) + (c / sg.group) * sg.group_stride + c % sg.group;
            row_stride = sg.row_stride;
            act = sg.act;
        }
        constexpr int kUnroll = 4;
#pragma unroll 1
        for (int it = 0; it < kTileRows / kRowsPerStep; it += kUnroll) {
            Raw16<T> raw[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int64_t row = row0 + (it + u) * kRowsPerStep + sub;
                if (col_ok && row < rows) load_raw16<T>(src + row * row_stride, raw[u]);
                else zero_raw16<T>(raw[u]);
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int r_in_tile = (it + u) * kRowsPerStep + sub;
                const int64_t row = row0 + r_in_tile;
                float v[16];
                if (act == 1) {
                    // looked-up bits go straight to fp32 (no repacking of the pair in between)
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const uint32_t w = raw[u].w[k];
                        v[2 * k] = lut_bits_to_f32<T>(lut[w & 0xffffu]);
                        v[2 * k + 1] = lut_bits_to_f32<T>(lut[w >> 16]);
                    }
                } else {
                    unpack16(raw[u], v);
                }
                uint32_t s8;
                const uint2 packed = nvfp4_encode_block<false>(v, ctx, hi_first, s8);
                if (col_ok && row < rows) {
                    *reinterpret_cast<uint2*>(q + row * (cols >> 1) + (col >> 1)) = packed;
                    s_sf[(blk >> 2) * 512 + sf_tile_offset(r_in_tile, blk & 3)] = (uint8_t)s8;
                }
            }
        }
        asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(kThreads) : "memory");
        if (tid < kSfTiles * 32) {
            const int t = tid >> 5;
            const int64_t tile_col = (tile_x * kTileCols >> 6) + t;
            if (tile_col < (sf_cpad >> 2)) {
                uint8_t* dst = sf + (tile_y * (sf_cpad >> 2) + tile_col) * 512 + (tid & 31) * 16;
                *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(s_sf + t * 512 + (tid & 31) * 16);
            }
        }
        asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(kThreads) : "memory");   // staging is read before the next tile clears it
    }
}

// Dequantize: lut[code] * (g * s8), each product rounded to the output dtype as
// the eager reference does (backends/eager/quantization.py:213-219).  Same tiling
// as the quantizer: a thread expands one block (8 bytes in, one 256-bit store out).
template <typename T, bool kVec>
__global__ void __launch_bounds__(kThreads)
dequantize_nvfp4_kernel(const uint8_t* __restrict__ q, const float* __restrict__ global_scale,
                        const uint8_t* __restrict__ sf, T* __restrict__ out, int64_t rows, int64_t cols,
                        int64_t sf_cpad, bool hi_first) {
    __shared__ __align__(16) uint8_t s_sf[kSfTiles * 512];
    const int tid = threadIdx.x;
    const int blk = tid & 15, sub = tid >> 4;
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
    const int64_t col = col0 + blk * 16;
    if (col >= cols) return;

    // four rows per thread in flight: the code loads of a batch are issued before any of them is expanded
    constexpr int kUnroll = 4;
#pragma unroll 1
    for (int it = 0; it < kTileRows / kRowsPerStep; it += kUnroll) {
        uint2 codes[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t row = row0 + (it + u) * kRowsPerStep + sub;
            codes[u] = make_uint2(0u, 0u);
            if (row < rows) codes[u] = *reinterpret_cast<const uint2*>(q + row * (cols >> 1) + (col >> 1));
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int r_in_tile = (it + u) * kRowsPerStep + sub;
            const int64_t row = row0 + r_in_tile;
            if (row >= rows) continue;
            const uint32_t s8 = s_sf[(blk >> 2) * 512 + sf_tile_offset(r_in_tile, blk & 3)];
            const float tot = Elem<T>::round(__fmul_rn(g, e4m3_to_f32(s8)));
            float lo[8], hi[8], v[16];
            e2m1x8_to_f32(codes[u].x, hi_first, lo);
            e2m1x8_to_f32(codes[u].y, hi_first, hi);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[i] = __fmul_rn(lo[i], tot);
                v[8 + i] = __fmul_rn(hi[i], tot);
            }
            T* dst = out + row * cols + col;
            if (kVec) {
                store16<T>(dst, v);
            } else {
                float a[8], b[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) { a[i] = v[i]; b[i] = v[8 + i]; }
                store8<T>(dst, a);
                store8<T>(dst + 8, b);
            }
        }
    }
}


template <typename T>
int launch_quantize(const void* x, const float* g, uint8_t* q, uint8_t* sf, int64_t rows, int64_t cols,
                    int64_t orig_rows, int64_t orig_cols, bool hi_first, cudaStream_t stream) {
    const int64_t sf_cpad = round_up(cols / 16, 4);
    dim3 grid((unsigned)ceil_div(sf_cpad * 16, kTileCols), (unsigned)ceil_div(rows, kTileRows));
    const bool vec = aligned32(x) && (orig_cols % 16 == 0);
    auto xt = static_cast<const T*>(x);
#define CK_LAUNCH_Q(VEC, EXACT) \
    quantize_nvfp4_kernel<T, VEC, EXACT><<<grid, kThreads, 0, stream>>>(xt, g, q, sf, rows, cols, orig_rows, orig_cols, sf_cpad, hi_first)
    if (g_nvfp4_exact_div) { if (vec) CK_LAUNCH_Q(true, true); else CK_LAUNCH_Q(false, true); }
    else { if (vec) CK_LAUNCH_Q(true, false); else CK_LAUNCH_Q(false, false); }
#undef CK_LAUNCH_Q
    return launch_status("quantize_nvfp4");
}

template <typename T>
int launch_dequantize(const uint8_t* q, const float* g, const uint8_t* sf, void* out, int64_t rows, int64_t cols,
                      bool hi_first, cudaStream_t stream) {
    const int64_t sf_cpad = round_up(cols / 16, 4);
    dim3 grid((unsigned)ceil_div(cols, kTileCols), (unsigned)ceil_div(rows, kTileRows));
    if (aligned32(out))
        dequantize_nvfp4_kernel<T, true><<<grid, kThreads, 0, stream>>>(q, g, sf, (T*)out, rows, cols, sf_cpad, hi_first);
    else
        dequantize_nvfp4_kernel<T, false><<<grid, kThreads, 0, stream>>>(q, g, sf, (T*)out, rows, cols, sf_cpad, hi_first);
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
    if (!aligned16(block_scales) || (reinterpret_cast<uintptr_t>(output) & 7u))
        CK_FAIL(CK_ERR_ALIGN, "quantize_nvfp4: outputs must be 16-byte (scales) / 8-byte (codes) aligned");
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
    if (!aligned16(block_scales) || !aligned16(output) || (reinterpret_cast<uintptr_t>(input) & 7u))
        CK_FAIL(CK_ERR_ALIGN, "dequantize_nvfp4: scales/output must be 16-byte aligned, codes 8-byte aligned");
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

// NVFP4 quantize of [seg0 | seg1] (seg1 optional: cols1 = 0), each segment addressed as
//   base + (c / group) * group_stride + row * row_stride + c % group   (elements of the input dtype)
// and optionally passed through GELU(tanh) (act = 1) first.  No counterpart in the reference: it replaces a
// gather / concatenation / activation kernel followed by launch_quantize_nvfp4_kernel.  Widths, groups and
// strides must be multiples of 16 elements and the bases 32-byte aligned; rows are not padded.
extern "C" int launch_quantize_nvfp4_gather_kernel(const void* base0, int64_t cols0, int64_t group0, int64_t group_stride0,
                                                   int64_t row_stride0, int act0, const void* base1, int64_t cols1,
                                                   int64_t group1, int64_t group_stride1, int64_t row_stride1, int act1,
                                                   const void* global_scale, void* output, void* block_scales,
                                                   int64_t num_rows, int input_dtype_code, bool hi_first,
                                                   cudaStream_t stream) {
    using namespace ck;
    if (!base0 || !global_scale || !output || !block_scales || (cols1 > 0 && !base1))
        CK_FAIL(CK_ERR_NULL, "quantize_nvfp4_gather: null pointer");
    const int64_t cols = cols0 + (cols1 > 0 ? cols1 : 0);
    auto seg_ok = [](const void* b, int64_t c, int64_t g, int64_t gs, int64_t rs, int act) {
        return c > 0 && g > 0 && c % 16 == 0 && g % 16 == 0 && c % g == 0 && gs % 16 == 0 && rs % 16 == 0 && gs >= 0 &&
               rs > 0 && (act == 0 || act == 1) && (reinterpret_cast<uintptr_t>(b) & 31u) == 0;
    };
    if (num_rows <= 0 || !seg_ok(base0, cols0, group0, group_stride0, row_stride0, act0) ||
        (cols1 > 0 && !seg_ok(base1, cols1, group1, group_stride1, row_stride1, act1)))
        CK_FAIL(CK_ERR_SHAPE, "quantize_nvfp4_gather: widths, groups and strides must be positive multiples of 16 elements, "
                              "bases 32-byte aligned, act 0 or 1");
    if (ceil_div(num_rows, 128) > 65535) CK_FAIL(CK_ERR_SHAPE, "quantize_nvfp4_gather: more than 65535*128 rows");
    if (!aligned16(block_scales) || (reinterpret_cast<uintptr_t>(output) & 7u))
        CK_FAIL(CK_ERR_ALIGN, "quantize_nvfp4_gather: outputs must be 16-byte (scales) / 8-byte (codes) aligned");
    if (input_dtype_code != CK_BF16 && input_dtype_code != CK_F16)
        CK_FAIL(CK_ERR_DTYPE, "quantize_nvfp4_gather: dtype code %d (bf16 or fp16)", input_dtype_code);
    const QuantSegment s0{base0, cols0, group0, group_stride0, row_stride0, act0};
    const QuantSegment s1{base1, cols1 > 0 ? cols1 : 0, cols1 > 0 ? group1 : 16, group_stride1, row_stride1, act1};
    const int64_t sf_cpad = round_up(cols / 16, 4);
    dim3 grid((unsigned)ceil_div(sf_cpad * 16, kTileCols), (unsigned)ceil_div(num_rows, kTileRows));
    auto* g = static_cast<const float*>(global_scale);
    auto* q = static_cast<uint8_t*>(output);
    auto* sf = static_cast<uint8_t*>(block_scales);
    const int64_t act_elems = num_rows * ((act0 == 1 ? cols0 : 0) + ((cols1 > 0 && act1 == 1) ? cols1 : 0));
    if (act_elems >= g_gelu_table_min && g_gelu_table_min >= 0) {
        // large activated input: tabulate the activation per CTA and look it up
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const int64_t num_tiles = (int64_t)grid.x * grid.y;
        int64_t ctas = ceil_div(num_tiles, (int64_t)kLutGroups);
        if (ctas > sms) ctas = sms;
        static bool attr_set[2][64] = {};
        const int ti = input_dtype_code == CK_BF16 ? 0 : 1;
        if (dev < 0 || dev >= 64 || !attr_set[ti][dev]) {
            cudaError_t e = ti == 0 ? cudaFuncSetAttribute(quantize_nvfp4_gather_lut_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kLutSmem)
                                    : cudaFuncSetAttribute(quantize_nvfp4_gather_lut_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kLutSmem);
            if (e != cudaSuccess) CK_FAIL((int)e, "quantize_nvfp4_gather: cannot reserve shared memory: %s", cudaGetErrorString(e));
            if (dev >= 0 && dev < 64) attr_set[ti][dev] = true;
        }
        if (ti == 0)
            quantize_nvfp4_gather_lut_kernel<__nv_bfloat16><<<(unsigned)ctas, kLutThreads, kLutSmem, stream>>>(s0, s1, g, q, sf, num_rows, cols, sf_cpad, hi_first, (int)grid.x, num_tiles);
        else
            quantize_nvfp4_gather_lut_kernel<__half><<<(unsigned)ctas, kLutThreads, kLutSmem, stream>>>(s0, s1, g, q, sf, num_rows, cols, sf_cpad, hi_first, (int)grid.x, num_tiles);
        return launch_status("quantize_nvfp4_gather");
    }
    if (input_dtype_code == CK_BF16)
        quantize_nvfp4_gather_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(s0, s1, g, q, sf, num_rows, cols, sf_cpad, hi_first);
    else
        quantize_nvfp4_gather_kernel<__half><<<grid, kThreads, 0, stream>>>(s0, s1, g, q, sf, num_rows, cols, sf_cpad, hi_first);
    return launch_status("quantize_nvfp4_gather");
}
