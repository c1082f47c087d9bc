// AdaLN / RMSNorm for sm_100a, standalone and fused with the activation quantizers.
//
//   LayerNorm form: y = (x - mean) * rstd * (1 + scale) + shift      (rstd = 1/sqrt(var + eps), biased var)
//   RMSNorm form:   y = x * rstd * weight                            (rstd = 1/sqrt(mean(x^2) + eps))
// with fp32 statistics and one rounding to x's dtype at the end — the formulation
// of comfy_kitchen/backends/cuda/ops/adaln.cu:105-189; the eager definition is
// comfy_kitchen/backends/eager/adaln.py:11-14.  Modulation rows are grouped as in
// comfy_kitchen/backends/_modulation.py:12-57: row r reads row r / group.
//
// Fast path (D a multiple of 16, row <= 48 KB): persistent warps, one row per warp at a time (per group of
// 2 or 4 warps for rows too wide for 16 warps to stage one each).  Each warp owns a small ring of row
// buffers in shared memory that it fills with cp.async.bulk (completion on its own mbarriers), so the
// loads of the next rows are in flight while the current row is reduced and written; the row is read
// from shared memory twice (shifted sums, output) and from HBM once.  The result is either stored in
// x's dtype, or — fused variants — rounded to
// x's dtype in registers and pushed through the same block encoders as quantize_nvfp4 /
// quantize_mxfp8, so the packed output is byte-identical to "adaln kernel, then quantize kernel"
// while the intermediate activation never reaches HBM (2.5625 instead of 6.5625 bytes per element
// for NVFP4).
#include "ck_common.cuh"

// Unroll factor of the two per-row loops in the builds for rows of a known length.  Timed with builds of the same
// source on 18432 rows (fused NVFP4): 2 -> 48.6 us (rows of 3072) / 63.1 us (4096); 1 -> 50.4 / 66.5; full (6 / 8) ->
// 49.5 / 69.2: the fully unrolled loop is long enough for the warps of an SM, which sit at different places in it,
// to wait on instruction fetches.
#ifndef CK_NORM_U1
#define CK_NORM_U1 2
#endif
#ifndef CK_NORM_U2
#define CK_NORM_U2 2
#endif

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
    int64_t row_begin, row_end;   // rows to process (row_end = 0: all N rows; the launcher resolves it)
    // CTA b owns rows_per_cta rows of span b / ctas_per_span (spans of span_rows rows from row_begin on; set by
    // the launcher): with one span per modulation group no CTA has to refill its modulation cache midway
    int64_t span_rows;
    int ctas_per_span;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Row statistics of 16-bit rows on the tensor cores.  The 4 words (8 values) a lane read from its row are its
// fragment of a 16 x 16 matrix A in mma.m16n8k16's layout — which of the warp's 256 values lands where does not
// matter for sums.  A x ones gives the row sums of A (every one eight times); A x A[0:8]^T and A x A[8:16]^T hold on
// their diagonals the sums of squares of A's rows (for the B operand "A[n][k]" a lane needs exactly its own A
// words).  Products of two 16-bit values are exact in fp32 and the accumulators are fp32, so this replaces the
// unpack + add + fma per element of a scalar pass by three instructions per 8 values of a lane.
template <typename T>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint4& a, uint32_t b0, uint32_t b1) {
    if (sizeof(T) == 2 && Elem<T>::code == CK_F16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}
struct MmaStats {
    float ones[4], lo[4], hi[4];   // A x ones; A x A[0:8]^T (rows 0-7 on its diagonal: ones[0..1]); A x A[8:16]^T (rows 8-15: [2..3])
};
template <typename T>
__device__ __forceinline__ void mma_stats_add(MmaStats& st, const uint4& u, bool want_sum) {
    // fragment words: x = (row g, k 2t..), y = (row g+8, k 2t..), z = (row g, k 2t+8..), w = (row g+8, k 2t+8..)
    const uint32_t one2 = Elem<T>::code == CK_F16 ? 0x3c003c00u : 0x3f803f80u;
    if (want_sum) mma_16816<T>(st.ones, u, one2, one2);
    mma_16816<T>(st.lo, u, u.x, u.z);
    mma_16816<T>(st.hi, u, u.y, u.w);
}
// Sum and sum of squares of everything the warp fed in (every lane gets both).
__device__ __forceinline__ void mma_stats_finish(const MmaStats& st, int lane, float& sum1, float& sum2) {
    const int g = lane >> 2, t = lane & 3;
    // diagonal entries: row g of `lo` sits in column g = 2t or 2t+1, i.e. in the lanes with t == g / 2
    const float diag = (g & 1) ? st.lo[1] + st.hi[3] : st.lo[0] + st.hi[2];
    sum2 = warp_sum(t == (g >> 1) ? diag : 0.0f);
    sum1 = warp_sum((st.ones[0] + st.ones[1]) + (st.ones[2] + st.ones[3])) * 0.125f;
}

__device__ int g_norm_status = 0;  // non-zero when a bounded wait on a row copy ran out

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// A lane's 16-element chunk from a row staged linearly in shared memory.  Lanes read 32 bytes each at
// a 32-byte stride; had every lane read its low half first, lanes l and l+4 would hit the same banks.
// Lanes with bit 2 set therefore read their high half first (`ordered` = false leaves the halves in
// that order: good enough for sums; `ordered` = true puts them back).
template <typename T, bool kOrdered>
__device__ __forceinline__ void lds16(const T* p, int lane, float (&v)[16]) {
    Raw16<T> r;
    if (sizeof(T) == 2) {
        const uint4* q = reinterpret_cast<const uint4*>(p);
        const int rot = (lane >> 2) & 1;
        const uint4 first = q[rot], second = q[rot ^ 1];
        const bool swap = kOrdered && rot;
        reinterpret_cast<uint4*>(r.w)[0] = swap ? second : first;
        reinterpret_cast<uint4*>(r.w)[1] = swap ? first : second;
    } else {
        constexpr int kVecs = (int)(sizeof(r.w) / 16);
#pragma unroll
        for (int i = 0; i < kVecs; ++i) reinterpret_cast<uint4*>(r.w)[i] = reinterpret_cast<const uint4*>(p)[i];
    }
    unpack16(r, v);
}

// Position of element e (0..15) of chunk c in the shared-memory modulation cache.  Chunks are grouped
// by 32 (one per lane); within a group the layout is [quad of elements][lane][4 floats], so the four
// 128-bit loads of a lane are each contiguous across the warp.
__device__ __forceinline__ int mod_pos(int c, int e) { return (c >> 5) * 512 + (e >> 2) * 128 + (c & 31) * 4 + (e & 3); }

constexpr uint32_t kRowWaitLimit = 1u << 22;

// Fast path.  A CTA owns a contiguous range of rows; its warps take them round-robin.  Each warp
// streams its rows through a private ring of shared-memory buffers filled by cp.async.bulk.  The
// modulation of the range ((1 + scale) or the RMSNorm weight, and shift) is cached in shared memory
// as fp32 and reloaded only where the range crosses a modulation group.  Per row: one pass for the
// statistics (shifted by the row's first element, so a large common offset does not cancel), one
// pass for the output; a lane owns whole 16-element chunks.
// kIters > 0: the row is exactly kIters x 512 elements (known at compile time, so both passes unroll fully and
// no lane is ever past the row's end); 0: any row length.
// kGroup > 1: wide rows.  kGroup consecutive warps share a row, each staging and processing D / kGroup
// elements of it; they exchange their partial sums through shared memory at a named barrier of their own
// (which also carries "a copy never arrived", so that the group leaves together).
template <typename T, int kMode, int kMaxThreads, int kIters, int kGroup = 1>
__global__ void __launch_bounds__(kMaxThreads)
norm_stream_kernel(const NormArgs a, const int ring, const int64_t rows_per_cta, const int cache_mod,
                   const uint32_t poll_limit) {
    extern __shared__ __align__(128) uint8_t smem[];
    // (an odd chunk count — half a row of 3072 is three chunk steps — is unrolled whole)
    constexpr int kUnrollStats = kIters > 0 ? (CK_NORM_U1) : 2, kUnrollOut = kIters > 0 ? (kIters % 2 ? kIters : (CK_NORM_U2)) : 2;
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grp = warp / kGroup, member = warp % kGroup, n_groups = warps / kGroup;
    const int64_t D = a.D;
    const int64_t seg_elems = D / kGroup;                      // this warp's share of a row
    const uint32_t row_bytes = (uint32_t)(seg_elems * sizeof(T));
    float* s_mul = reinterpret_cast<float*>(smem);            // [D]  (only when cache_mod)
    const int64_t mod_elems = round_up(D, 512);                // whole groups of 32 chunks
    float* s_add = s_mul + mod_elems;
    uint8_t* rows_base = smem + (cache_mod ? (size_t)mod_elems * 8 : 0);
    uint8_t* my_rows = rows_base + (size_t)warp * ring * row_bytes;
    uint64_t* my_bars = reinterpret_cast<uint64_t*>(rows_base + (size_t)warps * ring * row_bytes) + warp * ring;
    // partial sums of the group's members, two sets (rows alternate between them)
    float2* s_part = reinterpret_cast<float2*>(reinterpret_cast<uint64_t*>(rows_base + (size_t)warps * ring * row_bytes) + warps * ring);
    const int nchunk = kIters > 0 ? kIters * 32 : (int)(seg_elems >> 4);  // 16-element chunks in this warp's share
    const int cbase = member * nchunk;                         // its first chunk's index in the row

    if (lane == 0) {
        for (int s = 0; s < ring; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&my_bars[s])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();

    // (a.row_end is resolved by the launcher: N, or N rounded up to 128 where the scale buffer's padding rows belong
    // to this call, or the end of the caller's row range)
    const int64_t total_rows = a.row_end;
    const int64_t span0 = a.row_begin + (int64_t)(blockIdx.x / a.ctas_per_span) * a.span_rows;
    const int64_t r0 = span0 + (int64_t)(blockIdx.x % a.ctas_per_span) * rows_per_cta;
    // (the last CTA also takes what lies behind the last span: the scale buffer's padding rows)
    const int64_t r1 = blockIdx.x + 1 == gridDim.x ? total_rows : min(min(r0 + rows_per_cta, span0 + a.span_rows), total_rows);
    const T* __restrict__ xg = static_cast<const T*>(a.x);

    auto issue = [&](int64_t r, int slot) {
        if (r < r1 && r < a.N && lane == 0) {
            const uint32_t bar = smem_u32(&my_bars[slot]);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(row_bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(my_rows + (size_t)slot * row_bytes)), "l"(xg + r * D + member * seg_elems), "r"(row_bytes), "r"(bar) : "memory");
        }
    };

    int64_t r_issue = r0 + grp;
    int64_t issued = 0;
    for (; issued < ring - 1; ++issued, r_issue += n_groups) issue(r_issue, (int)(issued % ring));

    const Nvfp4Ctx ctx = nvfp4_ctx(kMode == kOutNvfp4 ? __ldg(a.global_scale) : 1.0f);
    const float inv_d = 1.0f / (float)D;
    const T* __restrict__ scale_g = static_cast<const T*>(a.scale);
    const T* __restrict__ shift_g = static_cast<const T*>(a.shift);

    int64_t row = r0 + grp;
    int64_t i = 0;
    bool alive = true;
    for (int64_t seg = r0; seg < r1;) {
        // rows [seg, seg_end) share one scale row and one shift row
        int64_t seg_end = r1;
        if (cache_mod) {
            const int64_t lim = min(a.N, r1);
            if (seg < lim) {
                seg_end = lim;
                if (scale_g) seg_end = min(seg_end, (seg / a.scale_group + 1) * a.scale_group);
                if (shift_g) seg_end = min(seg_end, (seg / a.shift_group + 1) * a.shift_group);
                __syncthreads();  // the previous segment's readers are done with the cache
                const T* sc = scale_g ? scale_g + (seg / a.scale_group) * D : nullptr;
                const T* sh = shift_g ? shift_g + (seg / a.shift_group) * D : nullptr;
                for (int64_t j = threadIdx.x; j < D; j += blockDim.x) {
                    const float m = sc ? Elem<T>::to_f32(sc[j]) : (a.rms ? 1.0f : 0.0f);
                    const int pos = mod_pos((int)(j >> 4), (int)(j & 15));
                    s_mul[pos] = a.rms ? m : 1.0f + m;
                    s_add[pos] = sh ? Elem<T>::to_f32(sh[j]) : 0.0f;
                }
                __syncthreads();
            }
        }
        for (; row < seg_end && alive; row += n_groups, ++i) {
            // refill the slot consumed in the previous iteration
            issue(r_issue, (int)(issued % ring));
            ++issued;
            r_issue += n_groups;

            if (row >= a.N) {
                // rows that exist only as padding of the tiled scale buffer: zero their scale bytes
                if (kMode != kOutPlain && member == 0)
                    for (int64_t c4 = lane; c4 < (a.sf_cpad >> 2); c4 += 32)
                        *reinterpret_cast<uint32_t*>(a.sf + sf_offset(row, c4 * 4, a.sf_cpad)) = 0u;
                continue;
            }

            const int slot = (int)(i % ring);
            {
                const uint32_t bar = smem_u32(&my_bars[slot]), parity = (uint32_t)((i / ring) & 1);
                uint32_t done = 0;
                for (uint32_t spin = 0; spin < poll_limit && !done; ++spin)
                    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
                if (!__all_sync(0xffffffffu, done != 0)) {
                    if (lane == 0) atomicCAS(&g_norm_status, 0, 1);
                    alive = false;  // stop touching rows; still take part in the CTA barriers below
                    if (kGroup == 1) break;   // (a group leaves together at its barrier below)
                }
            }
            const T* xs = reinterpret_cast<const T*>(my_rows + (size_t)slot * row_bytes);

            // Statistics in one pass.  fp32 rows: shifted by the row's first element, so that a large common offset
            // does not cancel (a group's other members fetch it from global memory: it sits in the first member's
            // buffer).  16-bit rows: unshifted sums on the tensor cores; a row whose mean dwarfs its spread is
            // then summed again the shifted way (below).  Rows shared by a group of warps keep the shifted sums.
            float shift0 = 0.0f, sum1, sum2;
            auto shifted_sums = [&]() {
                shift0 = a.rms ? 0.0f : Elem<T>::to_f32((kGroup == 1 || member == 0) ? xs[0] : xg[row * D]);
                // two accumulator pairs, updated with sm_100's packed fp32 instructions (two IEEE operations each)
                float2 s1 = make_float2(0.0f, 0.0f), s2 = s1;
                const float2 nshift = make_float2(-shift0, -shift0);
#pragma unroll((sizeof(T) == 2 && kGroup == 1) ? 1 : (kIters > 0 ? kIters : 2))
                for (int c = lane; c < nchunk; c += 32) {
                    float f[16];
                    lds16<T, false>(xs + c * 16, lane, f);
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        const float2 d = __fadd2_rn(make_float2(f[j], f[j + 1]), nshift);
                        s1 = __fadd2_rn(s1, d);
                        s2 = __ffma2_rn(d, d, s2);
                    }
                }
                sum1 = warp_sum(s1.x + s1.y);
                sum2 = warp_sum(s2.x + s2.y);
            };
            if constexpr (sizeof(T) == 2 && kGroup == 1) {
                MmaStats st = {};
                const int rot = (lane >> 2) & 1;   // the order of a lane's two 16-byte reads (bank conflicts, see lds16)
#pragma unroll(kUnrollStats)
                for (int c0 = 0; c0 < nchunk; c0 += 32) {
                    const int c = c0 + lane;
                    uint4 u0 = make_uint4(0u, 0u, 0u, 0u), u1 = u0;   // (every lane takes part in the MMAs)
                    if (kIters > 0 || c < nchunk) {
                        const uint4* q = reinterpret_cast<const uint4*>(xs + c * 16);
                        u0 = q[rot];
                        u1 = q[rot ^ 1];
                    }
                    mma_stats_add<T>(st, u0, !a.rms);
                    mma_stats_add<T>(st, u1, !a.rms);
                }
                mma_stats_finish(st, lane, sum1, sum2);
            } else {
                shifted_sums();
            }
            if (kGroup > 1) {
                float2* part = s_part + (grp * 2 + (int)(i & 1)) * kGroup;
                if (lane == 0) part[member] = make_float2(sum1, sum2);
                __syncwarp();
                // the group's barrier: publishes the partial sums and ORs "my copy never arrived"
                uint32_t any_failed;
                asm volatile("{ .reg .pred p, q; setp.ne.b32 p, %1, 0; barrier.red.or.pred q, %2, %3, p; selp.u32 %0, 1, 0, q; }"
                             : "=r"(any_failed) : "r"(alive ? 0u : 1u), "r"(1 + grp), "r"(kGroup * 32) : "memory");
                if (any_failed) { alive = false; break; }
                sum1 = 0.0f; sum2 = 0.0f;
#pragma unroll
                for (int k = 0; k < kGroup; ++k) { const float2 v = part[k]; sum1 += v.x; sum2 += v.y; }
            }
            float m1 = sum1 * inv_d;   // mean - shift0
            float m2 = sum2 * inv_d;   // E[(x - shift0)^2]
            if (sizeof(T) == 2 && kGroup == 1 && !a.rms && (m2 - m1 * m1) * 256.0f < m2) {
                // |mean| > 16 standard deviations: E[x^2] - mean^2 has lost bits to cancellation
                shifted_sums();
                m1 = sum1 * inv_d;
                m2 = sum2 * inv_d;
            }
            const float mean = a.rms ? 0.0f : shift0 + m1;
            const float var = a.rms ? m2 : fmaxf(m2 - m1 * m1, 0.0f);
            const float rstd = rsqrtf(var + a.eps);
            const float nmr = -mean * rstd;
            const float2 rstd2 = make_float2(rstd, rstd), nmr2 = make_float2(nmr, nmr);

            const T* __restrict__ sc = (!cache_mod && scale_g) ? scale_g + (row / a.scale_group) * D : nullptr;
            const T* __restrict__ sh = (!cache_mod && shift_g) ? shift_g + (row / a.shift_group) * D : nullptr;

            // whole-warp steps: the MXFP8 block encoder shuffles between lane pairs
#pragma unroll(kUnrollOut)
            for (int c0 = 0; c0 < nchunk; c0 += 32) {
                const int c = c0 + lane;          // chunk within this warp's share
                const int cg = cbase + c;         // chunk within the row
                const bool ok = kIters > 0 || c < nchunk;
                const bool row_tail = kGroup == 1 || member == kGroup - 1;   // lanes past the share's end are past the row's end
                float y[16];
                if (kMode == kOutMxfp8) {
                    // its block encoder shuffles between lane pairs: lanes past the row's end take part with zeros
#pragma unroll
                    for (int j = 0; j < 16; ++j) y[j] = 0.0f;
                } else if (!ok) {
                    // scale columns that pad the row to a multiple of 4
                    if (kMode == kOutNvfp4 && row_tail && cg < a.sf_cpad) a.sf[sf_offset(row, cg, a.sf_cpad)] = 0;
                    continue;
                }
                // NVFP4 with cached modulation: lanes that read their high half first (lds16) keep that order
                // through the modulation and the block encoder (the block maximum does not care, the modulation is
                // read in the same order) and exchange the two words of codes at the end, instead of putting the
                // sixteen values back in order.
                const bool halves_swapped = kMode == kOutNvfp4 && sizeof(T) == 2 && cache_mod && ((lane >> 2) & 1);
                if (ok) {
                    float f[16];
                    lds16<T, kMode != kOutNvfp4>(xs + c * 16, lane, f);
                    if (cache_mod) {
                        const int mbase = mod_pos(cg, 0);
                        const int off_first = mbase + (halves_swapped ? 256 : 0);    // quads of f[0..7]
                        const int off_second = mbase + (halves_swapped ? 0 : 256);   // quads of f[8..15]
#pragma unroll
                        for (int j4 = 0; j4 < 4; ++j4) {
                            const int mo = (j4 < 2 ? off_first : off_second) + (j4 & 1) * 128;
                            const float4 mu = *reinterpret_cast<const float4*>(s_mul + mo);
                            const float4 ad = *reinterpret_cast<const float4*>(s_add + mo);
                            const float2 ya = __ffma2_rn(__ffma2_rn(make_float2(f[4 * j4 + 0], f[4 * j4 + 1]), rstd2, nmr2),
                                                         make_float2(mu.x, mu.y), make_float2(ad.x, ad.y));
                            const float2 yb = __ffma2_rn(__ffma2_rn(make_float2(f[4 * j4 + 2], f[4 * j4 + 3]), rstd2, nmr2),
                                                         make_float2(mu.z, mu.w), make_float2(ad.z, ad.w));
                            y[4 * j4 + 0] = ya.x; y[4 * j4 + 1] = ya.y; y[4 * j4 + 2] = yb.x; y[4 * j4 + 3] = yb.y;
                        }
                    } else {
                        if (kMode == kOutNvfp4 && sizeof(T) == 2 && ((lane >> 2) & 1)) {
                            // (the modulation comes from global memory in element order: put the halves back)
#pragma unroll
                            for (int j = 0; j < 8; ++j) { const float t = f[j]; f[j] = f[8 + j]; f[8 + j] = t; }
                        }
                        float m[16], b[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) { m[j] = a.rms ? 1.0f : 0.0f; b[j] = 0.0f; }
                        if (scale_g) load16<T>(sc + (int64_t)cg * 16, m);
                        if (shift_g) load16<T>(sh + (int64_t)cg * 16, b);
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            y[j] = fmaf(fmaf(f[j], rstd, nmr), a.rms ? m[j] : 1.0f + m[j], b[j]);
                    }
                }
                if (kMode == kOutPlain) {
                    if (ok) store16<T>(static_cast<T*>(a.out) + row * D + (int64_t)cg * 16, y);
                } else {
                    // the quantizers see the activation as it would have been stored
#pragma unroll
                    for (int j = 0; j < 16; j += 2) Elem<T>::round2(y[j], y[j + 1]);
                    if (kMode == kOutNvfp4) {
                        uint32_t s8;
                        uint2 packed = nvfp4_encode_block_straight(y, ctx, a.hi_first != 0, s8);
                        if (halves_swapped) packed = make_uint2(packed.y, packed.x);
                        *reinterpret_cast<uint2*>(static_cast<uint8_t*>(a.out) + row * (D >> 1) + (int64_t)cg * 8) = packed;
                        a.sf[sf_offset(row, cg, a.sf_cpad)] = (uint8_t)s8;
                    } else {
                        // 32-element block = this lane's chunk and its neighbour's (lane ^ 1)
                        uint32_t e;
                        float lo[8], hi[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) { lo[j] = y[j]; hi[j] = y[8 + j]; }
                        float amax = 0.0f;
#pragma unroll
                        for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(y[j]));
                        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                        const uint2 p0 = mxfp8_encode8(lo, amax, e), p1 = mxfp8_encode8(hi, amax, e);
                        if (ok) {
                            *reinterpret_cast<uint4*>(static_cast<uint8_t*>(a.out) + row * D + (int64_t)cg * 16) =
                                make_uint4(p0.x, p0.y, p1.x, p1.y);
                            if ((lane & 1) == 0) a.sf[sf_offset(row, cg >> 1, a.sf_cpad)] = (uint8_t)e;
                        } else if ((lane & 1) == 0 && row_tail && (cg >> 1) < a.sf_cpad) {
                            a.sf[sf_offset(row, cg >> 1, a.sf_cpad)] = 0;
                        }
                    }
                }
            }
            __syncwarp();  // every lane is done with this slot before it is refilled
        }
        seg = seg_end;
    }
    if (!alive) {
        // A wait ran out (or a group member's did).  The copies this warp issued for rows i .. issued-1 may still
        // be in flight: shared memory must not be released under them, so wait for each with the full limit.
        const int64_t lim = min(r1, a.N);
        for (int64_t j = i; j < issued; ++j) {
            if (r0 + grp + j * n_groups >= lim) break;
            const uint32_t bar = smem_u32(&my_bars[j % ring]), parity = (uint32_t)((j / ring) & 1);
            uint32_t done = 0;
            for (uint32_t spin = 0; spin < kRowWaitLimit && !done; ++spin)
                asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                             : "=r"(done) : "r"(bar), "r"(parity) : "memory");
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
    const size_t row_bytes = (size_t)a.D * sizeof(T);
    // the modulation cache pays when a modulation row serves many rows (AdaLN: one per batch entry)
    const bool has_mod = a.scale || a.shift;
    int cache_mod = has_mod && (!a.scale || a.scale_group >= 32) && (!a.shift || a.shift_group >= 32);
    if (g_norm_cache == 0) cache_mod = 0;
    // Warps per CTA, ring depth and whether to cache the modulation, from the shared-memory budget (225 KB of
    // the 227 a CTA can have; the barriers take the rest).  Throughput grows almost linearly with the warps
    // per SM up to 16 (each warp walks its rows serially), a second row buffer per warp adds a few percent,
    // and the modulation cache is worth about a quarter: so take the most warps whose rows fit once, give
    // them a second (third) buffer if there is room, and give up the cache where that doubles the warps
    // (rows of 16 KB and more).  g_norm_warps > 0 forces the warp count (up to 24, for tuning runs).
    // Rows too wide for 16 warps to stage one each (beside the modulation cache) are shared by 2 or 4
    // consecutive warps, each staging and processing an equal share of whole 32-element blocks: 16 warps per
    // SM stay in flight for rows up to 48 KB.  (Measured, 18432 rows: 12288 elements 386 -> 222 us with four
    // warps per row, 8192 elements 204 -> 147 us with two; 5120 elements fit 16 single warps and are faster so.)
    int group = 1;
    if (g_norm_group > 0) {
        group = g_norm_group;
    } else {
        const size_t need_cache = cache_mod ? (size_t)round_up(a.D, 512) * 8 : 0;
        while (group < 4 && 16 * (row_bytes / group) + need_cache > 225 * 1024) group *= 2;
        // Few rows per SM (at most one per warp): a row's latency, not throughput, sets the time, so two warps
        // share each row.  Measured on rows of 3072 elements: 512 rows 16.5 -> 8.8 us, 2304 rows 18.1 -> 13.4 us;
        // from 4096 rows on one warp per row is as fast or faster.
        const int64_t n_rows = (a.row_end > 0 ? a.row_end : a.N) - a.row_begin;
        if (group == 1 && n_rows <= 16 * 148 && a.D % 64 == 0 && a.D >= 1024) group = 2;
    }
    if (group != 1 && group != 2 && group != 4) CK_FAIL(CK_ERR_SHAPE, "adaln: warps per row must be 1, 2 or 4");
    while (group > 1 && a.D % (32 * group) != 0) group /= 2;   // every share must be whole 32-element blocks
    const size_t warp_bytes = row_bytes / group;   // what one warp stages of a row
    int warps = 0, ring = 1;
    size_t mod_bytes = 0;
    {
        const size_t cache_bytes = (size_t)round_up(a.D, 512) * 8;
        double best = 0.0;
        int best_cache = 0;
        for (int cache = cache_mod ? 1 : 0; cache >= 0; --cache) {
            const size_t mb = cache ? cache_bytes : 0;
            if (mb + row_bytes > 225 * 1024) continue;
            const size_t budget = 225 * 1024 - mb;
            int w = 0;
            if (g_norm_warps > 0) {
                w = g_norm_warps > 32 ? 32 : g_norm_warps;
                if (group > 1 && w > 16) w = 16;
                w -= w % group;
                if ((size_t)w * warp_bytes > budget) w = 0;
            } else {
                for (int cand : {16, 12, 8, 6, 4, 2, 1})   // (24 and 32 warps measured slower: option "norm_warps" only)
                    if (cand % group == 0 && (group == 1 || cand <= 16) && (size_t)cand * warp_bytes <= budget) { w = cand; break; }
            }
            if (w == 0) continue;
            const int r = (size_t)w * 3 * warp_bytes <= budget ? 3 : ((size_t)w * 2 * warp_bytes <= budget ? 2 : 1);
            const double score = w * (cache ? 1.0 : 0.75) * (r >= 2 ? 1.0 : 0.93);
            if (score > best) { best = score; warps = w; ring = r; best_cache = cache; mod_bytes = mb; }
        }
        if (warps == 0)
            CK_FAIL(CK_ERR_SHAPE, "adaln: a row of %lld bytes does not fit the staging ring", (long long)row_bytes);
        cache_mod = best_cache;
    }
    const size_t smem = mod_bytes + (size_t)warps * ring * warp_bytes + (size_t)warps * ring * 8 + (size_t)warps * 16;
    // three builds of the kernel: up to 16 warps with 128 registers per thread, up to 24 with 80, up to 32 with 64
    // rows of 3072 and 4096 elements (the common hidden sizes) get builds with the chunk count known at compile time,
    // rows of 3072 shared by two warps too (1152 rows: 9.1 -> 8.7 us)
    const int iters = (a.D == 3072) ? 6 : (a.D == 4096 ? 8 : 0);
    auto kern = group == 4 ? norm_stream_kernel<T, kMode, 512, 0, 4>
              : group == 2 ? (a.D == 3072 ? norm_stream_kernel<T, kMode, 512, 3, 2> : norm_stream_kernel<T, kMode, 512, 0, 2>)
              : warps > 24 ? (iters == 6 ? norm_stream_kernel<T, kMode, 1024, 6> : norm_stream_kernel<T, kMode, 1024, 0>)
              : warps > 16 ? (iters == 8 ? norm_stream_kernel<T, kMode, 768, 8> : (iters == 6 ? norm_stream_kernel<T, kMode, 768, 6> : norm_stream_kernel<T, kMode, 768, 0>))
                           : (iters == 6 ? norm_stream_kernel<T, kMode, 512, 6>
                                         : (iters == 8 ? norm_stream_kernel<T, kMode, 512, 8> : norm_stream_kernel<T, kMode, 512, 0>));
    const int attr_idx = group == 4 ? 5 : (group == 2 ? (a.D == 3072 ? 10 : 4) : (warps > 24 ? (iters == 6 ? 6 : 7) : (warps > 16 ? (iters == 8 ? 8 : (iters == 6 ? 9 : 3)) : (iters == 6 ? 1 : (iters == 8 ? 2 : 0)))));
    static bool attr_set[11][64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_set[attr_idx][dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) CK_FAIL((int)e, "adaln: cannot reserve shared memory: %s", cudaGetErrorString(e));
        if (dev >= 0 && dev < 64) attr_set[attr_idx][dev] = true;
    }
    // rows of this call: all of them (fused modes: plus the scale buffer's padding rows), or the caller's range
    // (the padding rows go with the range that ends at N)
    NormArgs ar = a;
    if (ar.row_end == 0) { ar.row_begin = 0; ar.row_end = a.N; }
    if (kMode != kOutPlain && ar.row_end == a.N) ar.row_end = round_up(a.N, 128);
    const int64_t rows = ar.row_end - ar.row_begin;
    if (rows <= 0) return CK_OK;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // one CTA per SM, each with a contiguous range of rows (at least one row per warp or group of warps)
    int64_t grid = ceil_div(rows, warps / group);
    if (grid > sms) grid = sms;
    int64_t rows_per_cta = ceil_div(rows, grid);
    grid = ceil_div(rows, rows_per_cta);
    ar.span_rows = rows;
    ar.ctas_per_span = (int)grid;
    // Cached modulation that changes every G rows: a CTA whose range straddled such a boundary would stop all its
    // warps there to refill the cache, and the whole launch waits for those few CTAs (measured: 4 x 4608 rows of
    // 3072 took 56.7 us against 48.5 us for 18432 rows under one modulation row).  Give every modulation group
    // its own share of the CTAs instead.
    {
        const int64_t G = a.scale && a.shift ? (a.scale_group == a.shift_group ? a.scale_group : 0)
                                             : (a.scale ? a.scale_group : (a.shift ? a.shift_group : 0));
        if (cache_mod && ar.row_begin == 0 && G > 0 && G < a.N && a.N % G == 0 && a.N / G <= sms / 2) {
            const int64_t n_spans = a.N / G;
            int64_t per_span = sms / n_spans;
            int64_t rpc = ceil_div(G, per_span);
            if (rpc < warps / group) rpc = warps / group;
            per_span = ceil_div(G, rpc);
            rows_per_cta = rpc;
            grid = n_spans * per_span;
            ar.span_rows = G;
            ar.ctas_per_span = (int)per_span;
        }
    }
    const uint32_t poll_limit = g_norm_poll_limit == 0 ? kRowWaitLimit : (g_norm_poll_limit < 0 ? 0u : (uint32_t)g_norm_poll_limit);
    kern<<<(unsigned)grid, warps * 32, smem, stream>>>(ar, ring, rows_per_cta, cache_mod, poll_limit);
    return launch_status("adaln");
}

bool warp_path_ok(const NormArgs& a) {
    return a.D % 16 == 0 && (size_t)a.D * 4 <= 48 * 1024 && aligned16(a.x) && (!a.scale || aligned16(a.scale)) &&
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
        CK_FAIL(CK_ERR_UNSUPPORTED, "%s: needs 16-byte aligned tensors and a row length that is a multiple of 8", what);
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

// launch_adaln_quantize_nvfp4_kernel restricted to rows [row_begin, row_end) of the N rows: codes and scale bytes of
// those rows only are written, at the positions the whole-tensor call writes them (a range that ends at N also
// writes the scale buffer's padding rows).  For sequence-parallel callers: each rank quantizes its rows of a shared
// activation.  Ranges whose bounds are multiples of 128 rows touch disjoint scale tiles.
extern "C" int launch_adaln_quantize_nvfp4_rows_kernel(const void* x, const void* scale, const void* shift,
                                                       const void* global_scale, void* output, void* block_scales,
                                                       int64_t N, int64_t D, int64_t scale_group, int64_t shift_group,
                                                       float eps, int dtype_code, bool hi_first, int norm_kind,
                                                       int64_t row_begin, int64_t row_end, cudaStream_t stream) {
    using namespace ck;
    if (norm_kind == 0 && (!scale || !shift)) CK_FAIL(CK_ERR_NULL, "adaln_quantize_nvfp4_rows: null modulation pointer");
    if (row_begin < 0 || row_end < row_begin || row_end > N)
        CK_FAIL(CK_ERR_SHAPE, "adaln_quantize_nvfp4_rows: rows %lld..%lld outside 0..%lld", (long long)row_begin, (long long)row_end, (long long)N);
    if (row_begin == row_end) return CK_OK;
    NormArgs a{x, scale, shift, output, static_cast<uint8_t*>(block_scales), static_cast<const float*>(global_scale),
               N, D, scale_group, shift_group, 0, eps, norm_kind != 0, hi_first ? 1 : 0, row_begin, row_end};
    if (!warp_path_ok(a)) CK_FAIL(CK_ERR_UNSUPPORTED, "adaln_quantize_nvfp4_rows: needs 16-byte aligned rows of a multiple of 16 elements");
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

// Reads and clears the device-side status word of the norm kernels (synchronises the device).
// 0 = no bounded wait on a row copy ran out since the last call.
extern "C" int ck_norm_device_status(void) {
    int v = 0, zero = 0;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) CK_FAIL((int)e, "norm status: %s", cudaGetErrorString(e));
    e = cudaMemcpyFromSymbol(&v, ck::g_norm_status, sizeof(int));
    if (e != cudaSuccess) CK_FAIL((int)e, "norm status: %s", cudaGetErrorString(e));
    cudaMemcpyToSymbol(ck::g_norm_status, &zero, sizeof(int));
    if (v != 0) CK_FAIL(CK_ERR_DEVICE_TIMEOUT, "norm kernel: a bounded wait on a row copy ran out");
    return CK_OK;
}
