// Per-head RMSNorm of q and k, rotary embedding of both, and the move of q, k, v from the layout a fused
// QKV projection writes ([tokens, 3, heads, 128], possibly a column slice of a wider matrix) to the layout
// attention reads ([heads, total_tokens, 128]), in one pass.
//
// The reference has the pieces as separate operators (apply_rope: comfy_kitchen/backends/eager/rope.py:9-32;
// rms_norm is torch's) and leaves the layout changes to the caller; between a QKV GEMM and attention that is
// two normalisation launches, one rope launch and four tensor copies.  Arithmetic per (token, head), all in
// fp32 with the roundings the separate operators would make:
//   y  = round_x( (x * rsqrt(mean(x^2) + eps)) * w )            for q and k (v is copied)
//   o0 = round_x( F[p,0,0]*y[2p] + F[p,0,1]*y[2p+1] ),  o1 = round_x( F[p,1,0]*y[2p] + F[p,1,1]*y[2p+1] )
// with the table F in fp32, first product rounded, then the sum (the order of rope.cu).
//
// One warp per (token, head) by default: it loads the token's 64 rotation matrices (two per lane; the table is a
// few MB and stays in L2), then a lane moves 4 consecutive elements (8 bytes) of q, k and v, so every access is a
// whole 256-byte row.  A warp can also walk several heads of its token with the matrices kept in registers, but
// the walk is a chain of dependent reductions and more warps hide it better — measured on 4608 tokens x 24
// heads: 33.8 us with one head per warp, 35.0 with three, 39.8 with six, 42.6 with all 24 (and 5.3 against 21.0 us
// for 512 tokens).  Memory-bound: 2 x 3 x tokens x heads x 128 elements + the table.
#include "ck_common.cuh"

namespace ck {
namespace {

constexpr int kHeadDim = 128;

template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xffff0000u);
    v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xffff0000u);
}
template <>
__device__ __forceinline__ void load4<__half>(const __half* p, float (&v)[4]) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&a);
    u.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}
template <>
__device__ __forceinline__ void store4<__half>(__half* p, const float (&v)[4]) {
    const __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&a);
    u.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

struct QkParams {
    const void* qkv;
    const void* q_w;
    const void* k_w;
    const float* freqs;   // [total_tokens, 64, 2, 2]
    void* q_out;
    void* k_out;
    void* v_out;
    int64_t row_stride;   // elements between consecutive tokens of qkv
    int64_t tokens, heads, token_offset, total_tokens;
    float eps;
    int heads_per_warp;   // a warp walks this many heads of its token (blockIdx.y picks which)
};

template <typename T>
__device__ __forceinline__ void norm_rope4(const float (&x)[4], const float (&w)[4], const float (&f)[2][4], float eps,
                                           float (&o)[4]) {
    const float ss = warp_sum(fmaf(x[0], x[0], fmaf(x[1], x[1], fmaf(x[2], x[2], x[3] * x[3]))));
    const float rstd = rsqrtf(ss * (1.0f / kHeadDim) + eps);
    float y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) y[i] = Elem<T>::round(__fmul_rn(__fmul_rn(x[i], rstd), w[i]));
#pragma unroll
    for (int p = 0; p < 2; ++p) {
        o[2 * p] = __fadd_rn(__fmul_rn(f[p][0], y[2 * p]), __fmul_rn(f[p][1], y[2 * p + 1]));
        o[2 * p + 1] = __fadd_rn(__fmul_rn(f[p][2], y[2 * p]), __fmul_rn(f[p][3], y[2 * p + 1]));
    }
}

// kHpw > 0: heads per warp known at compile time (the walk is fully unrolled); 0: p.heads_per_warp.
template <typename T, int kHpw>
__global__ void __launch_bounds__(256) qk_norm_rope_kernel(const QkParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= p.tokens) return;
    const int64_t tok = p.token_offset + t;
    // this lane's two rotation matrices (pairs 2*lane, 2*lane + 1): 32 contiguous bytes
    float f[2][4];
    {
        const float4* fp = reinterpret_cast<const float4*>(p.freqs + (tok * (kHeadDim / 2) + 2 * lane) * 4);
        const float4 a = __ldg(fp), b = __ldg(fp + 1);
        f[0][0] = a.x; f[0][1] = a.y; f[0][2] = a.z; f[0][3] = a.w;
        f[1][0] = b.x; f[1][1] = b.y; f[1][2] = b.z; f[1][3] = b.w;
    }
    float wq[4], wk[4];
    load4<T>(static_cast<const T*>(p.q_w) + 4 * lane, wq);
    load4<T>(static_cast<const T*>(p.k_w) + 4 * lane, wk);
    const T* row = static_cast<const T*>(p.qkv) + t * p.row_stride + 4 * lane;
    const int64_t head_pitch = p.total_tokens * kHeadDim;
    T* qo = static_cast<T*>(p.q_out) + tok * kHeadDim + 4 * lane;
    T* ko = static_cast<T*>(p.k_out) + tok * kHeadDim + 4 * lane;
    T* vo = static_cast<T*>(p.v_out) + tok * kHeadDim + 4 * lane;
    const int64_t part = p.heads * kHeadDim;   // distance from a head of q to the same head of k, and of k to v
    const int hpw = kHpw > 0 ? kHpw : p.heads_per_warp;
    const int64_t h0 = (int64_t)blockIdx.y * hpw;
#pragma unroll(kHpw > 0 ? kHpw : 2)
    for (int i = 0; i < hpw; ++i) {
        const int64_t h = h0 + i;
        if (kHpw == 0 && h >= p.heads) break;   // (compile-time counts divide the heads)
        float xq[4], xk[4], oq[4], ok[4];
        load4<T>(row + h * kHeadDim, xq);
        load4<T>(row + part + h * kHeadDim, xk);
        const uint2 v = *reinterpret_cast<const uint2*>(row + 2 * part + h * kHeadDim);
        norm_rope4<T>(xq, wq, f, p.eps, oq);
        norm_rope4<T>(xk, wk, f, p.eps, ok);
        store4<T>(qo + h * head_pitch, oq);
        store4<T>(ko + h * head_pitch, ok);
        *reinterpret_cast<uint2*>(vo + h * head_pitch) = v;
    }
}

}  // namespace
}  // namespace ck

// qkv: [tokens, >= 3*heads*128] with `row_stride` elements between tokens, columns [q heads | k heads | v heads];
// q_weight, k_weight: [128] in qkv's dtype; freqs: fp32 [total_tokens, 64, 2, 2]; outputs: [heads, total_tokens, 128],
// rows token_offset .. token_offset + tokens - 1 of every head are written.
extern "C" int launch_qk_norm_rope_kernel(const void* qkv, int64_t row_stride, const void* q_weight, const void* k_weight,
                                          const float* freqs, void* q_out, void* k_out, void* v_out, int64_t tokens,
                                          int64_t heads, int64_t token_offset, int64_t total_tokens, float eps,
                                          int dtype_code, cudaStream_t stream) {
    using namespace ck;
    if (!qkv || !q_weight || !k_weight || !freqs || !q_out || !k_out || !v_out)
        CK_FAIL(CK_ERR_NULL, "qk_norm_rope: null pointer");
    if (tokens <= 0 || heads <= 0 || token_offset < 0 || token_offset + tokens > total_tokens ||
        row_stride < 3 * heads * kHeadDim)
        CK_FAIL(CK_ERR_SHAPE, "qk_norm_rope: bad shape tokens=%lld heads=%lld offset=%lld total=%lld row_stride=%lld",
                (long long)tokens, (long long)heads, (long long)token_offset, (long long)total_tokens, (long long)row_stride);
    if (dtype_code != CK_BF16 && dtype_code != CK_F16) CK_FAIL(CK_ERR_DTYPE, "qk_norm_rope: dtype code %d (bf16 or fp16)", dtype_code);
    if ((reinterpret_cast<uintptr_t>(qkv) & 7) || (row_stride & 3) || (reinterpret_cast<uintptr_t>(q_out) & 7) ||
        (reinterpret_cast<uintptr_t>(k_out) & 7) || (reinterpret_cast<uintptr_t>(v_out) & 7) ||
        (reinterpret_cast<uintptr_t>(q_weight) & 7) || (reinterpret_cast<uintptr_t>(k_weight) & 7) || !aligned16(freqs))
        CK_FAIL(CK_ERR_ALIGN, "qk_norm_rope: tensors must be 8-byte aligned (table 16), row stride a multiple of 4 elements");
    // heads of a token that one warp walks (blockIdx.y picks which): one, unless the tuning option says otherwise
    int hpw = 1;
    if (g_qk_heads_per_warp > 0) hpw = g_qk_heads_per_warp < heads ? g_qk_heads_per_warp : (int)heads;
    if (ceil_div(heads, (int64_t)hpw) > 65535) CK_FAIL(CK_ERR_SHAPE, "qk_norm_rope: too many heads");
    QkParams p{qkv, q_weight, k_weight, freqs, q_out, k_out, v_out, row_stride, tokens, heads, token_offset, total_tokens, eps, hpw};
    const int warps = 8;
    const dim3 grid((unsigned)ceil_div(tokens, (int64_t)warps), (unsigned)ceil_div(heads, (int64_t)hpw));
    const bool divides = heads % hpw == 0;
#define CK_QK_LAUNCH(T)                                                                                       \
    do {                                                                                                      \
        if (divides && hpw == 1) qk_norm_rope_kernel<T, 1><<<grid, warps * 32, 0, stream>>>(p);               \
        else if (divides && hpw == 2) qk_norm_rope_kernel<T, 2><<<grid, warps * 32, 0, stream>>>(p);          \
        else if (divides && hpw == 3) qk_norm_rope_kernel<T, 3><<<grid, warps * 32, 0, stream>>>(p);          \
        else if (divides && hpw == 4) qk_norm_rope_kernel<T, 4><<<grid, warps * 32, 0, stream>>>(p);          \
        else if (divides && hpw == 6) qk_norm_rope_kernel<T, 6><<<grid, warps * 32, 0, stream>>>(p);          \
        else qk_norm_rope_kernel<T, 0><<<grid, warps * 32, 0, stream>>>(p);                                   \
    } while (0)
    if (dtype_code == CK_BF16) CK_QK_LAUNCH(__nv_bfloat16);
    else CK_QK_LAUNCH(__half);
#undef CK_QK_LAUNCH
    return launch_status("qk_norm_rope");
}
