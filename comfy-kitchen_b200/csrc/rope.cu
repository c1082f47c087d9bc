// Rotary position embedding for sm_100a.
//
// For every pair p of the last dimension, with (a, b) = (x[2p], x[2p+1])
// (interleaved) or (x[p], x[p + D/2]) (split-half):
//   o_i = F[p,i,0]*a + F[p,i,1]*b,  i in {0, 1}
// evaluated in the dtype of the table F (first product rounded, then the sum of
// it and the second product rounded) and cast to x's dtype — the order of the
// eager reference (comfy_kitchen/backends/eager/rope.py:9-32).  q and k share
// one pass and one read of the table.
//
// The table is broadcast over at least one of the three leading dimensions
// (heads, usually).  A thread owns one table "site" and 4 pairs (8 with
// split-half): it loads their 2x2 matrices once into registers and then walks
// the broadcast dimension(s), moving one 128-bit vector of q and of k per step.
// Algorithmic traffic is therefore 2 tensors x (read + write) + the table once.
#include "ck_common.cuh"

namespace ck {
namespace {

struct RopeParams {
    int64_t dims[3];     // leading dims of x
    int64_t sx[3];       // x element strides (input and output)
    int64_t sf[3];       // table element strides for the leading dims
    int64_t sf_dim, sf_rot, sf_pair;
    int64_t sx_dim;
    int bc[3];           // 1 where the table is broadcast over that dim
    int D;
    int n_vec;           // threads per row
    int64_t n_sites;     // product of the non-broadcast dims
    int64_t n_bcast;     // product of the broadcast dims
    int64_t chunk;       // broadcast steps per thread
    int64_t n_chunks;
};

template <typename TF>
__device__ __forceinline__ float rot(float f0, float f1, float a, float b) {
    const float t = Elem<TF>::round(__fmul_rn(f0, a));
    return Elem<TF>::round(__fadd_rn(t, __fmul_rn(f1, b)));
}

template <typename TF, int kPairs>
__device__ __forceinline__ void load_table(const TF* __restrict__ f, float (&m)[kPairs][4]) {
    // kPairs contiguous 2x2 matrices
    if (sizeof(TF) == 4) {
#pragma unroll
        for (int p = 0; p < kPairs; ++p) {
            const float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(f) + 4 * p);
            m[p][0] = t.x; m[p][1] = t.y; m[p][2] = t.z; m[p][3] = t.w;
        }
    } else {
#pragma unroll
        for (int p = 0; p < kPairs; p += 2) {
            float v[8];
            load8<TF>(f + 4 * p, v);
#pragma unroll
            for (int i = 0; i < 4; ++i) { m[p][i] = v[i]; m[p + 1][i] = v[4 + i]; }
        }
    }
}

// 16 bytes through the read-only path without allocating in L1 (every byte is used once).
__device__ __forceinline__ uint4 ldg128(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
template <typename T>
__device__ __forceinline__ void unpack8_16(const uint4& u, float (&v)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (sizeof(T) == 2 && Elem<T>::code == CK_BF16) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        } else {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
}

template <typename TX, typename TF, bool kSplit>
__global__ void __launch_bounds__(256, 3)
rope_vec_kernel(const TX* __restrict__ xq, const TX* __restrict__ xk, const TF* __restrict__ freqs,
                TX* __restrict__ oq, TX* __restrict__ ok, const RopeParams p) {
    constexpr int kPairs = kSplit ? 8 : 4;
    // work item = (vector of the row, site, chunk of the broadcast walk); the grid is sized to the machine
    // (a whole number of resident blocks per SM) and strides over the items
    const int64_t n_items = (int64_t)p.n_vec * p.n_sites * p.n_chunks;
    for (int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gid < n_items; gid += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(gid % p.n_vec);
    int64_t t = gid / p.n_vec;
    const int64_t site = t % p.n_sites;
    const int64_t c = t / p.n_sites;

    // site -> indices of the non-broadcast dims
    int64_t s = site, xoff = 0, foff = 0;
#pragma unroll
    for (int k = 2; k >= 0; --k) {
        const int64_t n = p.bc[k] ? 1 : p.dims[k];
        const int64_t i = s % n;
        s /= n;
        xoff += i * p.sx[k];
        foff += i * p.sf[k];
    }
    float m[kPairs][4];
    load_table<TF, kPairs>(freqs + foff + (int64_t)v * kPairs * 4, m);

    // first broadcast step of this chunk -> indices of the broadcast dims
    int64_t j = c * p.chunk;
    const int64_t j_end = min(j + p.chunk, p.n_bcast);
    int64_t idx[3], lim[3];
    {
        int64_t r = j;
#pragma unroll
        for (int k = 2; k >= 0; --k) {
            lim[k] = p.bc[k] ? p.dims[k] : 1;
            idx[k] = r % lim[k];
            r /= lim[k];
        }
    }
    const int64_t col = kSplit ? (int64_t)v * 8 : (int64_t)v * 8;
    const int64_t half = p.D / 2;

    // Interleaved layout with 16-bit activations (the shape a DiT runs): steps are taken four at a time, with the
    // eight 16-byte loads (q and k of four steps) issued before anything is computed or stored, so that each
    // thread keeps 128 bytes of reads in flight.
    if (!kSplit && sizeof(TX) == 2) {
        constexpr int kBatch = 4;
        for (; j + kBatch <= j_end; j += kBatch) {
            int64_t offs[kBatch];
            uint4 raw[2][kBatch];
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                offs[b] = xoff + idx[0] * p.sx[0] + idx[1] * p.sx[1] + idx[2] * p.sx[2] + col;
                if (++idx[2] == lim[2]) {
                    idx[2] = 0;
                    if (++idx[1] == lim[1]) { idx[1] = 0; ++idx[0]; }
                }
            }
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                raw[0][b] = ldg128(xq + offs[b]);
                if (xk != nullptr) raw[1][b] = ldg128(xk + offs[b]);
            }
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
#pragma unroll
                for (int which = 0; which < 2; ++which) {
                    TX* __restrict__ dst = which ? ok : oq;
                    if ((which ? xk : xq) == nullptr) continue;
                    float x[8], o[8];
                    unpack8_16<TX>(raw[which][b], x);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float a = Elem<TF>::round(x[2 * q]), bb = Elem<TF>::round(x[2 * q + 1]);
                        o[2 * q] = rot<TF>(m[q][0], m[q][1], a, bb);
                        o[2 * q + 1] = rot<TF>(m[q][2], m[q][3], a, bb);
                    }
                    store8<TX>(dst + offs[b], o);
                }
            }
        }
    }
#pragma unroll 2
    for (; j < j_end; ++j) {
        const int64_t off = xoff + idx[0] * p.sx[0] + idx[1] * p.sx[1] + idx[2] * p.sx[2] + col;
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            const TX* __restrict__ src = which ? xk : xq;
            TX* __restrict__ dst = which ? ok : oq;
            if (src == nullptr) continue;
            if (!kSplit) {
                float x[8], o[8];
                load8<TX>(src + off, x);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float a = Elem<TF>::round(x[2 * q]), b = Elem<TF>::round(x[2 * q + 1]);
                    o[2 * q] = rot<TF>(m[q][0], m[q][1], a, b);
                    o[2 * q + 1] = rot<TF>(m[q][2], m[q][3], a, b);
                }
                store8<TX>(dst + off, o);
            } else {
                float lo[8], hi[8], olo[8], ohi[8];
                load8<TX>(src + off, lo);
                load8<TX>(src + off + half, hi);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const float a = Elem<TF>::round(lo[q]), b = Elem<TF>::round(hi[q]);
                    olo[q] = rot<TF>(m[q][0], m[q][1], a, b);
                    ohi[q] = rot<TF>(m[q][2], m[q][3], a, b);
                }
                store8<TX>(dst + off, olo);
                store8<TX>(dst + off + half, ohi);
            }
        }
        // advance the broadcast index with carry
        if (++idx[2] == lim[2]) {
            idx[2] = 0;
            if (++idx[1] == lim[1]) { idx[1] = 0; ++idx[0]; }
        }
    }
    }
}

// Any strides, any D (even): one thread per pair.
template <typename TX, typename TF>
__global__ void __launch_bounds__(256)
rope_generic_kernel(const TX* __restrict__ xq, const TX* __restrict__ xk, const TF* __restrict__ freqs,
                    TX* __restrict__ oq, TX* __restrict__ ok, const RopeParams p, bool split_half) {
    const int64_t half = p.D / 2;
    const int64_t total = p.dims[0] * p.dims[1] * p.dims[2] * half;
    for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (int64_t)gridDim.x * blockDim.x) {
        const int64_t pr = g % half;
        int64_t r = g / half;
        int64_t xoff = 0, foff = 0;
#pragma unroll
        for (int k = 2; k >= 0; --k) {
            const int64_t i = r % p.dims[k];
            r /= p.dims[k];
            xoff += i * p.sx[k];
            foff += (p.bc[k] ? 0 : i) * p.sf[k];
        }
        const int64_t ia = (split_half ? pr : 2 * pr) * p.sx_dim, ib = (split_half ? pr + half : 2 * pr + 1) * p.sx_dim;
        const TF* f = freqs + foff + pr * p.sf_dim;
        const float f00 = Elem<TF>::to_f32(f[0]), f01 = Elem<TF>::to_f32(f[p.sf_pair]);
        const float f10 = Elem<TF>::to_f32(f[p.sf_rot]), f11 = Elem<TF>::to_f32(f[p.sf_rot + p.sf_pair]);
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            const TX* __restrict__ src = which ? xk : xq;
            TX* __restrict__ dst = which ? ok : oq;
            if (src == nullptr) continue;
            const float a = Elem<TF>::round(Elem<TX>::to_f32(src[xoff + ia]));
            const float b = Elem<TF>::round(Elem<TX>::to_f32(src[xoff + ib]));
            dst[xoff + ia] = Elem<TX>::from_f32(rot<TF>(f00, f01, a, b));
            dst[xoff + ib] = Elem<TX>::from_f32(rot<TF>(f10, f11, a, b));
        }
    }
}

inline int sm_count_cached() {
    static int n = 0;
    if (n == 0) {
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        n = v > 0 ? v : 148;
    }
    return n;
}

template <typename TX, typename TF>
int launch(const void* xq, const void* xk, const void* freqs, void* oq, void* ok, RopeParams p, bool split_half,
           bool vec_ok, cudaStream_t stream) {
    auto q = static_cast<const TX*>(xq), k = static_cast<const TX*>(xk);
    auto f = static_cast<const TF*>(freqs);
    auto o1 = static_cast<TX*>(oq), o2 = static_cast<TX*>(ok);
    if (vec_ok) {
        p.n_vec = split_half ? p.D / 16 : p.D / 8;
        // A thread loads its 2x2 matrices once per work item and reuses them for the item's broadcast steps.  Items
        // are chunks of 8 steps where the broadcast extent allows (two batches of four in the kernel), and the grid
        // is three resident blocks per SM striding over the items: on [B, 24, 4608, 128] that is 2, 4 or 8 items
        // per thread for B = 1, 2, 4 with at most 3 % of the last round idle.
        int64_t chunk = g_rope_threads_per_sm > 0 ? ceil_div(p.n_bcast, ceil_div(148LL * g_rope_threads_per_sm, p.n_sites * p.n_vec))
                                                  : (p.n_bcast >= 8 ? 8 : p.n_bcast);
        if (chunk < 1) chunk = 1;
        if (chunk > p.n_bcast) chunk = p.n_bcast;
        p.chunk = chunk;
        p.n_chunks = ceil_div(p.n_bcast, p.chunk);
        const int64_t threads = p.n_sites * p.n_vec * p.n_chunks;
        int64_t blocks = ceil_div(threads, 256);
        const int64_t resident = 3LL * sm_count_cached();
        if (blocks > resident) blocks = resident;
        if (split_half)
            rope_vec_kernel<TX, TF, true><<<(unsigned)blocks, 256, 0, stream>>>(q, k, f, o1, o2, p);
        else
            rope_vec_kernel<TX, TF, false><<<(unsigned)blocks, 256, 0, stream>>>(q, k, f, o1, o2, p);
    } else {
        const int64_t total = p.dims[0] * p.dims[1] * p.dims[2] * (p.D / 2);
        int64_t blocks = ceil_div(total, 256);
        if (blocks > 148 * 64) blocks = 148 * 64;
        rope_generic_kernel<TX, TF><<<(unsigned)blocks, 256, 0, stream>>>(q, k, f, o1, o2, p, split_half);
    }
    return launch_status("apply_rope");
}

template <typename TX>
int dispatch_f(int fcode, const void* xq, const void* xk, const void* freqs, void* oq, void* ok, const RopeParams& p,
               bool split_half, bool vec_ok, cudaStream_t stream) {
    switch (fcode) {
    case CK_F32: return launch<TX, float>(xq, xk, freqs, oq, ok, p, split_half, vec_ok, stream);
    case CK_F16: return launch<TX, __half>(xq, xk, freqs, oq, ok, p, split_half, vec_ok, stream);
    case CK_BF16: return launch<TX, __nv_bfloat16>(xq, xk, freqs, oq, ok, p, split_half, vec_ok, stream);
    default: CK_FAIL(CK_ERR_DTYPE, "apply_rope: unsupported freqs dtype code %d", fcode);
    }
}

}  // namespace
}  // namespace ck

extern "C" int launch_apply_rope_kernel(const void* xq, const void* xk, const void* freqs, void* xq_out, void* xk_out,
                                        int64_t batch, int64_t dim1, int64_t dim2, int64_t head_dim,
                                        int64_t freqs_batch, int64_t freqs_dim1, int64_t freqs_dim2,
                                        int64_t stride_x_batch, int64_t stride_x_dim1, int64_t stride_x_dim2,
                                        int64_t stride_x_dim, int64_t stride_freqs_batch, int64_t stride_freqs_dim1,
                                        int64_t stride_freqs_dim2, int64_t stride_freqs_dim, int64_t stride_freqs_rot,
                                        int64_t stride_freqs_pair, int input_dtype_code, int freqs_dtype_code,
                                        bool split_half, cudaStream_t stream) {
    using namespace ck;
    if (!xq || !freqs || !xq_out) CK_FAIL(CK_ERR_NULL, "apply_rope: null pointer");
    if ((xk == nullptr) != (xk_out == nullptr)) CK_FAIL(CK_ERR_NULL, "apply_rope: xk and xk_out must be given together");
    if (batch <= 0 || dim1 <= 0 || dim2 <= 0 || head_dim <= 0 || head_dim % 2 != 0)
        CK_FAIL(CK_ERR_SHAPE, "apply_rope: bad shape [%lld,%lld,%lld,%lld] (last dim must be even)", (long long)batch,
                (long long)dim1, (long long)dim2, (long long)head_dim);
    const int64_t xd[3] = {batch, dim1, dim2}, fd[3] = {freqs_batch, freqs_dim1, freqs_dim2};
    RopeParams p{};
    p.n_sites = 1;
    p.n_bcast = 1;
    for (int k = 0; k < 3; ++k) {
        if (fd[k] != 1 && fd[k] < xd[k])
            CK_FAIL(CK_ERR_SHAPE, "apply_rope: freqs dim %d is %lld, needs 1 or >= %lld", k, (long long)fd[k], (long long)xd[k]);
        p.dims[k] = xd[k];
        p.bc[k] = (fd[k] == 1 && xd[k] != 1) ? 1 : 0;
        if (p.bc[k]) p.n_bcast *= xd[k]; else p.n_sites *= xd[k];
    }
    p.sx[0] = stride_x_batch; p.sx[1] = stride_x_dim1; p.sx[2] = stride_x_dim2; p.sx_dim = stride_x_dim;
    p.sf[0] = stride_freqs_batch; p.sf[1] = stride_freqs_dim1; p.sf[2] = stride_freqs_dim2;
    p.sf_dim = stride_freqs_dim; p.sf_rot = stride_freqs_rot; p.sf_pair = stride_freqs_pair;
    p.D = (int)head_dim;

    const int fbytes = freqs_dtype_code == CK_F32 ? 4 : 2;
    bool vec_ok = stride_x_dim == 1 && head_dim % (split_half ? 16 : 8) == 0 && aligned16(xq) && aligned16(xq_out) &&
                  (!xk || (aligned16(xk) && aligned16(xk_out))) && aligned16(freqs) && stride_freqs_pair == 1 &&
                  stride_freqs_rot == 2 && stride_freqs_dim == 4;
    for (int k = 0; k < 3; ++k) {
        if (p.dims[k] > 1 && p.sx[k] % 8 != 0) vec_ok = false;
        if (!p.bc[k] && p.dims[k] > 1 && (p.sf[k] * fbytes) % 16 != 0) vec_ok = false;
    }
    switch (input_dtype_code) {
    case CK_F32: return dispatch_f<float>(freqs_dtype_code, xq, xk, freqs, xq_out, xk_out, p, split_half, vec_ok, stream);
    case CK_F16: return dispatch_f<__half>(freqs_dtype_code, xq, xk, freqs, xq_out, xk_out, p, split_half, vec_ok, stream);
    case CK_BF16: return dispatch_f<__nv_bfloat16>(freqs_dtype_code, xq, xk, freqs, xq_out, xk_out, p, split_half, vec_ok, stream);
    default: CK_FAIL(CK_ERR_DTYPE, "apply_rope: unsupported input dtype code %d", input_dtype_code);
    }
}
