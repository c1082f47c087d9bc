// Exchange step of the tensor-parallel stack: sum of the row-parallel GEMMs' partial results over the
// ranks, fused with the residual update that follows it, over NVLink peer memory.
//
//   x[r, c] <- bf16( x[r, c] + gate[c] * bf16( sum_i partial_i[r, c] ) )        on every rank
//
// i.e. all_reduce(sum) of the [rows, cols] partial outputs followed by addcmul(x, gate, y), in one
// kernel and without a collective library.  The reference has no multi-GPU code; this stands where a
// tensor-parallel port of it would call ncclAllReduce and an elementwise kernel.
//
// Every rank runs the same launch (same grid).  Rank r owns the r-th contiguous slice of the matrix:
//   1. start barrier  - block b tells block b of every peer "my partial is complete" (it is: the GEMM
//                       that wrote it precedes this kernel on the stream) and waits for theirs;
//   2. reduce         - 16-byte loads of the slice from all ranks' partial buffers (plain peer loads,
//                       no multicast), fp32 sum in rank order, one rounding to the 16-bit type, the
//                       residual update in fp32, one more rounding;
//   3. push           - the updated slice is stored into the residual buffer of every rank;
//   4. end barrier    - block b waits until block b of every peer has finished pushing, so that when
//                       the kernel completes on a rank its whole residual buffer is up to date.
// Since one rank computes each element, all ranks end with bit-identical residuals.
//
// Barrier flags live in a per-rank pad that the peers can write: start[block][source rank] and
// end[block][source rank] hold the epoch of the last call that signalled; the epoch itself is kept in the
// rank's own memory and advanced by the kernel, so a CUDA graph can replay the launch.  Every wait is
// bounded by wall-clock time (%globaltimer); on expiry the block records a status word and carries on
// without waiting (the result is then wrong, and ck_tp_device_status() says so).
#include "ck_common.cuh"

namespace ck {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxBlocks = 512;
constexpr int kThreads = 512;
constexpr unsigned long long kWaitNs = 4000000000ull;   // 4 s: far beyond any skew between ranks in a running job

__device__ int g_tp_status = 0;   // 0 ok; otherwise (phase << 16 | block) of the first wait that ran out

struct ExchangeParams {
    const uint4* partial[kMaxRanks];
    uint4* residual[kMaxRanks];
    uint32_t* pad[kMaxRanks];     // each rank's flag pad: start[kMaxBlocks][kMaxRanks], end[...], then epoch[kMaxBlocks]
    const uint4* mc_partial;      // multicast (NVLS) address of the partial buffers, or null
    uint4* mc_residual;           // multicast address of the residual buffers, or null
    const void* gate0;
    const void* gate1;
    int64_t split_vec;            // vectors (of 8 elements) before this index use gate0, the rest gate1
    int64_t total_vec;            // rows * cols / 8
    int vec_per_row;              // cols / 8
    int rank, world;
    int64_t slice_lo_vec, slice_hi_vec;   // this rank's slice in vectors (< 0: equal shares of total_vec)
    int local_only;               // 1: the updated slice stays in this rank's residual buffer, and there is no end barrier
};

__device__ __forceinline__ uint32_t* pad_start(uint32_t* pad, int block, int src) { return pad + (block * kMaxRanks + src); }
__device__ __forceinline__ uint32_t* pad_end(uint32_t* pad, int block, int src) { return pad + kMaxBlocks * kMaxRanks + (block * kMaxRanks + src); }
__device__ __forceinline__ uint32_t* pad_epoch(uint32_t* pad, int block) { return pad + 2 * kMaxBlocks * kMaxRanks + block; }
// (the gather kernel's own flags and epochs follow: gather_end[kMaxBlocks][kMaxRanks], gather_epoch[kMaxBlocks])
constexpr int kGatherPadOffset = 2 * kMaxBlocks * kMaxRanks + kMaxBlocks;
__device__ __forceinline__ uint32_t* pad_gather_end(uint32_t* pad, int block, int src) { return pad + kGatherPadOffset + (block * kMaxRanks + src); }
__device__ __forceinline__ uint32_t* pad_gather_epoch(uint32_t* pad, int block) { return pad + kGatherPadOffset + kMaxBlocks * kMaxRanks + block; }

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// 16-byte load that is served from L2 / the owning GPU, never from this SM's L1 (the data may have been
// rewritten by another GPU since the last call).
__device__ __forceinline__ uint4 ld_cg(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// NVLink-switch reduction: one load returns the sum over all ranks of the 8 values at this multicast address,
// accumulated in fp32 inside the switch and rounded once to the 16-bit type.
template <typename T>
__device__ __forceinline__ uint4 multimem_ld_reduce(const uint4* mc) {
    uint4 v;
    if (Elem<T>::code == CK_BF16)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    else
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
}
// One store that the switch delivers to every rank's copy of the buffer.
__device__ __forceinline__ void multimem_st(uint4* mc, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Threads 0 .. world-1 of the block: signal peer `threadIdx.x`, then wait for its signal.
__device__ __forceinline__ uint32_t* pad_flag(uint32_t* pad, int which, int block, int src) {
    return which == 0 ? pad_start(pad, block, src) : (which == 1 ? pad_end(pad, block, src) : pad_gather_end(pad, block, src));
}
// which: 0 = start flags, 1 = end flags, 2 = the gather kernel's flags
__device__ __forceinline__ void block_barrier(uint32_t* const* pads, int rank, int world, int which, uint32_t epoch) {
    __syncthreads();
    if ((int)threadIdx.x < world) {
        const int peer = threadIdx.x;
        const bool end_phase = which != 0;
        st_release_sys(pad_flag(pads[peer], which, blockIdx.x, rank), epoch);
        const uint32_t* mine = pad_flag(pads[rank], which, blockIdx.x, peer);
        const unsigned long long t0 = now_ns();
        uint32_t spins = 0;
        while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
            if ((++spins & 255u) == 0 && now_ns() - t0 > kWaitNs) {
                atomicCAS(&g_tp_status, 0, ((end_phase ? 2 : 1) << 16) | (int)blockIdx.x);
                (void)which;
                break;
            }
        }
    }
    __syncthreads();
}

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]);
template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
template <>
__device__ __forceinline__ void unpack8<__half>(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
}
template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    const __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// kWorld > 0: the rank count is known at compile time (2, 4, 8: the loops over ranks unroll and kUnroll is
// chosen so that a thread keeps (kWorld + 1) * kUnroll 16-byte loads in flight within ~100 registers);
// kWorld = 0: any rank count up to kMaxRanks.
template <typename T, int kWorld, int kUnroll>
__global__ void __launch_bounds__(kThreads)
tp_exchange_kernel(const ExchangeParams p) {
    __shared__ uint32_t s_epoch;
    uint32_t* my_pad = p.pad[p.rank];
    if (threadIdx.x == 0) s_epoch = *pad_epoch(my_pad, blockIdx.x) + 1u;
    __syncthreads();
    const uint32_t epoch = s_epoch;
    const int world = kWorld > 0 ? kWorld : p.world;
    constexpr int kRanks = kWorld > 0 ? kWorld : kMaxRanks;

    block_barrier(p.pad, p.rank, p.world, 0, epoch);   // every rank's partial result is complete

    // this rank's slice, and this block's part of it
    const int64_t lo = p.slice_lo_vec >= 0 ? p.slice_lo_vec : p.total_vec * p.rank / world;
    const int64_t hi = p.slice_lo_vec >= 0 ? p.slice_hi_vec : p.total_vec * (p.rank + 1) / world;
    const int64_t per_block = (hi - lo + gridDim.x - 1) / gridDim.x;
    const int64_t b0 = lo + per_block * blockIdx.x;
    const int64_t b1 = b0 + per_block < hi ? b0 + per_block : hi;
    for (int64_t base = b0 + threadIdx.x; base < b1; base += (int64_t)kThreads * kUnroll) {
        uint4 part[kUnroll][kRanks];
        uint4 xv[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t idx = base + (int64_t)u * kThreads;
            if (idx < b1) {
#pragma unroll
                for (int i = 0; i < kRanks; ++i)
                    if (i < world) part[u][i] = ld_cg(p.partial[i] + idx);
                xv[u] = ld_cg(p.residual[p.rank] + idx);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t idx = base + (int64_t)u * kThreads;
            if (idx >= b1) continue;
            float sum[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) sum[j] = 0.0f;
#pragma unroll
            for (int i = 0; i < kRanks; ++i) {
                if (i < world) {
                    float f[8];
                    unpack8<T>(part[u][i], f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) sum[j] += f[j];
                }
            }
            const int col_vec = (int)(idx % p.vec_per_row);
            const uint4* gate = reinterpret_cast<const uint4*>(idx < p.split_vec ? p.gate0 : p.gate1) + col_vec;
            float g[8], x[8];
            unpack8<T>(__ldg(gate), g);
            unpack8<T>(xv[u], x);
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                // y = the all-reduced GEMM output as it would have been stored; then x + gate * y, product and
                // sum rounded separately in fp32 (what an elementwise addcmul on 16-bit tensors computes)
                const float y0 = Elem<T>::round(sum[j]), y1 = Elem<T>::round(sum[j + 1]);
                w[j >> 1] = pack2<T>(__fadd_rn(x[j], __fmul_rn(g[j], y0)), __fadd_rn(x[j + 1], __fmul_rn(g[j + 1], y1)));
            }
            const uint4 out = make_uint4(w[0], w[1], w[2], w[3]);
            if (p.local_only) {
                p.residual[p.rank][idx] = out;
            } else {
#pragma unroll
                for (int i = 0; i < kRanks; ++i)
                    if (i < world) p.residual[i][idx] = out;
            }
        }
    }
    __threadfence_system();           // this thread's pushes are visible system-wide before the block signals
    if (!p.local_only) block_barrier(p.pad, p.rank, p.world, 1, epoch);    // every peer has finished pushing its slice into my residual buffer
    if (threadIdx.x == 0) *pad_epoch(my_pad, blockIdx.x) = epoch;
}

// The same exchange through the NVLink switch: the reduction happens in the switch (multimem.ld_reduce: this
// rank receives only its slice, already summed) and the updated slice is broadcast by the switch
// (multimem.st), so each GPU's links carry 1 / world of the matrix in each direction instead of
// (world - 1) / world.  The sum's accumulation order inside the switch is not specified; it is fp32 with one
// rounding, computed once per element by the slice's owner, so all ranks still end with identical bits.
template <typename T>
__global__ void __launch_bounds__(kThreads)
tp_exchange_multimem_kernel(const ExchangeParams p) {
    __shared__ uint32_t s_epoch;
    uint32_t* my_pad = p.pad[p.rank];
    if (threadIdx.x == 0) s_epoch = *pad_epoch(my_pad, blockIdx.x) + 1u;
    __syncthreads();
    const uint32_t epoch = s_epoch;
    block_barrier(p.pad, p.rank, p.world, 0, epoch);

    const int64_t lo = p.total_vec * p.rank / p.world, hi = p.total_vec * (p.rank + 1) / p.world;
    const int64_t per_block = (hi - lo + gridDim.x - 1) / gridDim.x;
    const int64_t b0 = lo + per_block * blockIdx.x;
    const int64_t b1 = b0 + per_block < hi ? b0 + per_block : hi;
    constexpr int kUnroll = 4;
    for (int64_t base = b0 + threadIdx.x; base < b1; base += (int64_t)kThreads * kUnroll) {
        uint4 yv[kUnroll], xv[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t idx = base + (int64_t)u * kThreads;
            if (idx < b1) {
                yv[u] = multimem_ld_reduce<T>(p.mc_partial + idx);
                xv[u] = ld_cg(p.residual[p.rank] + idx);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t idx = base + (int64_t)u * kThreads;
            if (idx >= b1) continue;
            const int col_vec = (int)(idx % p.vec_per_row);
            const uint4* gate = reinterpret_cast<const uint4*>(idx < p.split_vec ? p.gate0 : p.gate1) + col_vec;
            float g[8], x[8], y[8];
            unpack8<T>(__ldg(gate), g);
            unpack8<T>(xv[u], x);
            unpack8<T>(yv[u], y);
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 8; j += 2)
                w[j >> 1] = pack2<T>(__fadd_rn(x[j], __fmul_rn(g[j], y[j])), __fadd_rn(x[j + 1], __fmul_rn(g[j + 1], y[j + 1])));
            multimem_st(p.mc_residual + idx, make_uint4(w[0], w[1], w[2], w[3]));
        }
    }
    __threadfence_system();
    block_barrier(p.pad, p.rank, p.world, 1, epoch);
    if (threadIdx.x == 0) *pad_epoch(my_pad, blockIdx.x) = epoch;
}

// Reduce-my-rows with the peers' partial rows pulled by bulk copies (cp.async.bulk, no multicast) into a ring of
// shared-memory stages instead of by per-thread loads: one elected thread keeps (stages - 1) x world copies of
// kChunkBytes in flight, which fills the NVLink read path with far fewer outstanding instructions than 16-byte loads
// from every thread.  local_only form (sequence parallel): the result goes to this rank's residual rows only.
constexpr int kBulkThreads = 256;
constexpr int kChunkVecs = 256;                 // vectors per chunk: one per thread
constexpr int kChunkBytes = kChunkVecs * 16;    // 4 KB per source rank and chunk
constexpr int kBulkStages = 4;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

template <typename T>
__global__ void __launch_bounds__(kBulkThreads)
tp_reduce_rows_bulk_kernel(const ExchangeParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);                       // [kBulkStages]
    uint8_t* stage0 = smem + 128;
    const int world = p.world;
    const size_t stage_bytes = (size_t)world * kChunkBytes;
    __shared__ uint32_t s_epoch;
    uint32_t* my_pad = p.pad[p.rank];
    if (threadIdx.x == 0) {
        s_epoch = *pad_epoch(my_pad, blockIdx.x) + 1u;
        for (int s = 0; s < kBulkStages; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&bars[s])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    const uint32_t epoch = s_epoch;
    block_barrier(p.pad, p.rank, p.world, 0, epoch);   // every rank's partial result is complete

    const int64_t lo = p.slice_lo_vec, hi = p.slice_hi_vec;
    const int64_t per_block = ((hi - lo + gridDim.x - 1) / gridDim.x + kChunkVecs - 1) / kChunkVecs * kChunkVecs;
    const int64_t b0 = lo + per_block * blockIdx.x;
    const int64_t b1 = b0 + per_block < hi ? b0 + per_block : hi;
    const int64_t n_chunks = b1 > b0 ? (b1 - b0 + kChunkVecs - 1) / kChunkVecs : 0;

    auto issue = [&](int64_t j) {   // thread 0: all ranks' copies of chunk j into stage j % kBulkStages
        const int s = (int)(j % kBulkStages);
        const int64_t v0 = b0 + j * kChunkVecs;
        const uint32_t bytes = (uint32_t)((b1 - v0 < kChunkVecs ? b1 - v0 : kChunkVecs) * 16);
        const uint32_t bar = smem_addr(&bars[s]);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes * (uint32_t)world) : "memory");
        for (int i = 0; i < world; ++i)
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_addr(stage0 + s * stage_bytes + (size_t)i * kChunkBytes)), "l"(p.partial[i] + v0), "r"(bytes), "r"(bar)
                         : "memory");
    };
    if (threadIdx.x == 0)
        for (int64_t j = 0; j < kBulkStages - 1 && j < n_chunks; ++j) issue(j);

    bool alive = true;
    for (int64_t j = 0; j < n_chunks; ++j) {
        const int s = (int)(j % kBulkStages);
        const uint32_t bar = smem_addr(&bars[s]), parity = (uint32_t)((j / kBulkStages) & 1);
        const int64_t idx = b0 + j * kChunkVecs + threadIdx.x;
        uint4 xv = make_uint4(0u, 0u, 0u, 0u);
        if (idx < b1) xv = ld_cg(p.residual[p.rank] + idx);      // my residual rows are local: plain load, in flight during the wait
        if (alive) {
            const unsigned long long t0 = now_ns();
            uint32_t done = 0, spins = 0;
            while (!done) {
                asm volatile("{ .reg .pred q; mbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2; selp.u32 %0, 1, 0, q; }"
                             : "=r"(done) : "r"(bar), "r"(parity) : "memory");
                if (!done && (++spins & 63u) == 0 && now_ns() - t0 > kWaitNs) {
                    atomicCAS(&g_tp_status, 0, (3 << 16) | (int)blockIdx.x);
                    alive = false;
                    break;
                }
            }
        }
        if (idx < b1 && alive) {
            float sum[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) sum[k] = 0.0f;
            const uint4* st = reinterpret_cast<const uint4*>(stage0 + s * stage_bytes) + threadIdx.x;
            for (int i = 0; i < world; ++i) {
                float f[8];
                unpack8<T>(st[(size_t)i * kChunkVecs], f);
#pragma unroll
                for (int k = 0; k < 8; ++k) sum[k] += f[k];
            }
            const int col_vec = (int)(idx % p.vec_per_row);
            const uint4* gate = reinterpret_cast<const uint4*>(idx < p.split_vec ? p.gate0 : p.gate1) + col_vec;
            float g[8], x[8];
            unpack8<T>(__ldg(gate), g);
            unpack8<T>(xv, x);
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 8; k += 2) {
                const float y0 = Elem<T>::round(sum[k]), y1 = Elem<T>::round(sum[k + 1]);
                w[k >> 1] = pack2<T>(__fadd_rn(x[k], __fmul_rn(g[k], y0)), __fadd_rn(x[k + 1], __fmul_rn(g[k + 1], y1)));
            }
            p.residual[p.rank][idx] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        __syncthreads();   // everyone has read stage s: it can be refilled
        if (threadIdx.x == 0 && alive && j + kBulkStages - 1 < n_chunks) issue(j + kBulkStages - 1);
    }
    // (a block that gave up leaves its outstanding copies to land in shared memory it no longer reads; wait for them
    // before the block ends)
    if (!alive && threadIdx.x == 0) {
        const unsigned long long t0 = now_ns();
        while (now_ns() - t0 < 100000ull) { }
    }
    __syncthreads();
    if (threadIdx.x == 0) *pad_epoch(my_pad, blockIdx.x) = epoch;
}

template <typename T>
void launch_exchange(const ExchangeParams& p, int blocks, cudaStream_t stream) {
    if (p.local_only && p.world > 1 && g_tp_bulk) {
        const size_t smem = 128 + (size_t)kBulkStages * p.world * kChunkBytes;
        static bool attr_done = false;
        if (!attr_done) {   // enough for kMaxRanks sources per stage
            const cudaError_t e = cudaFuncSetAttribute(tp_reduce_rows_bulk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                       128 + kBulkStages * kMaxRanks * kChunkBytes);
            if (e != cudaSuccess) (void)cudaGetLastError();   // (the launch below then reports what is wrong)
            attr_done = true;
        }
        tp_reduce_rows_bulk_kernel<T><<<blocks, kBulkThreads, smem, stream>>>(p);
        return;
    }
    if (p.mc_partial != nullptr && p.world > 1) {
        tp_exchange_multimem_kernel<T><<<blocks, kThreads, 0, stream>>>(p);
        return;
    }
    switch (p.world) {
    case 1: tp_exchange_kernel<T, 1, 8><<<blocks, kThreads, 0, stream>>>(p); break;
    case 2: tp_exchange_kernel<T, 2, 6><<<blocks, kThreads, 0, stream>>>(p); break;
    case 4: tp_exchange_kernel<T, 4, 4><<<blocks, kThreads, 0, stream>>>(p); break;
    case 8: tp_exchange_kernel<T, 8, 2><<<blocks, kThreads, 0, stream>>>(p); break;
    default: tp_exchange_kernel<T, 0, 2><<<blocks, kThreads, 0, stream>>>(p); break;
    }
}

}  // namespace
}  // namespace ck

extern "C" int64_t ck_tp_pad_bytes(void) {
    // start + end flags and epochs of the exchange kernel, then the gather kernel's flags and epochs
    return (int64_t)sizeof(uint32_t) * (3 * ck::kMaxBlocks * ck::kMaxRanks + 2 * ck::kMaxBlocks);
}

static int exchange_impl(const void* const* partials, void* const* residuals, void* const* pads,
                         const void* mc_partial, void* mc_residual, int world,
                         int rank, const void* gate0, const void* gate1, int64_t split_row, int64_t rows,
                         int64_t cols, int dtype_code, int blocks, cudaStream_t stream, int64_t row_lo, int64_t row_hi,
                         int local_only) {
    using namespace ck;
    if (local_only && (row_lo < 0 || row_hi < row_lo || row_hi > rows))
        CK_FAIL(CK_ERR_SHAPE, "tp_reduce_rows: rows %lld..%lld outside 0..%lld", (long long)row_lo, (long long)row_hi, (long long)rows);
    if (!partials || !residuals || !pads || !gate0) CK_FAIL(CK_ERR_NULL, "tp_exchange: null pointer");
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
        CK_FAIL(CK_ERR_SHAPE, "tp_exchange: rank %d of %d (at most %d ranks)", rank, world, kMaxRanks);
    if (rows <= 0 || cols <= 0 || cols % 8 != 0 || split_row < 0)
        CK_FAIL(CK_ERR_SHAPE, "tp_exchange: bad shape rows=%lld cols=%lld (cols must be a multiple of 8)", (long long)rows, (long long)cols);
    if (dtype_code != CK_BF16 && dtype_code != CK_F16) CK_FAIL(CK_ERR_DTYPE, "tp_exchange: dtype code %d (bf16 or fp16)", dtype_code);
    ExchangeParams p{};
    for (int i = 0; i < world; ++i) {
        if (!partials[i] || !residuals[i] || !pads[i]) CK_FAIL(CK_ERR_NULL, "tp_exchange: null buffer of rank %d", i);
        if (!aligned16(partials[i]) || !aligned16(residuals[i]) || !aligned16(pads[i]))
            CK_FAIL(CK_ERR_ALIGN, "tp_exchange: buffers must be 16-byte aligned");
        p.partial[i] = static_cast<const uint4*>(partials[i]);
        p.residual[i] = static_cast<uint4*>(residuals[i]);
        p.pad[i] = static_cast<uint32_t*>(pads[i]);
    }
    if (!aligned16(gate0) || (gate1 && !aligned16(gate1))) CK_FAIL(CK_ERR_ALIGN, "tp_exchange: gates must be 16-byte aligned");
    if ((mc_partial == nullptr) != (mc_residual == nullptr)) CK_FAIL(CK_ERR_NULL, "tp_exchange: the two multicast addresses go together");
    if (mc_partial && (!aligned16(mc_partial) || !aligned16(mc_residual))) CK_FAIL(CK_ERR_ALIGN, "tp_exchange: multicast addresses must be 16-byte aligned");
    p.mc_partial = static_cast<const uint4*>(mc_partial);
    p.mc_residual = static_cast<uint4*>(mc_residual);
    p.gate0 = gate0;
    p.gate1 = gate1 ? gate1 : gate0;
    p.vec_per_row = (int)(cols / 8);
    p.total_vec = rows * (cols / 8);
    p.split_vec = (split_row < rows ? split_row : rows) * (cols / 8);
    if (!gate1) p.split_vec = p.total_vec;
    p.rank = rank;
    p.world = world;
    p.local_only = local_only;
    p.slice_lo_vec = local_only ? row_lo * (cols / 8) : -1;
    p.slice_hi_vec = local_only ? row_hi * (cols / 8) : -1;
    if (local_only) { p.mc_partial = nullptr; p.mc_residual = nullptr; }
    if (blocks <= 0) blocks = 148;   // one per SM: 114 registers x 512 threads leave room for one block per SM
    if (blocks > kMaxBlocks) blocks = kMaxBlocks;
    if (dtype_code == CK_BF16) launch_exchange<__nv_bfloat16>(p, blocks, stream);
    else launch_exchange<__half>(p, blocks, stream);
    return launch_status("tp_exchange");
}

namespace ck {
namespace {

// All-gather by pushing: every rank copies up to two byte ranges of its own buffer to the same offsets of every
// peer's buffer (16-byte stores), then waits until all peers have done the same.  Used for the quantized
// activation of the sequence-parallel stack (codes and scale tiles of the rank's rows) and for the residual
// stream at the end of a forward.  Flags and epochs of its own, so it can follow the reduction kernel freely.
struct GatherParams {
    uint4* buf[kMaxRanks];
    uint32_t* pad[kMaxRanks];
    int64_t lo[2], hi[2];    // ranges in 16-byte vectors (hi <= lo: empty)
    int rank, world;
};

__global__ void __launch_bounds__(kThreads)
tp_gather_kernel(const GatherParams p) {
    __shared__ uint32_t s_epoch;
    uint32_t* my_pad = p.pad[p.rank];
    if (threadIdx.x == 0) s_epoch = *pad_gather_epoch(my_pad, blockIdx.x) + 1u;
    __syncthreads();
    const uint32_t epoch = s_epoch;
    const uint4* src = p.buf[p.rank];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int64_t n = p.hi[r] - p.lo[r];
        if (n <= 0) continue;
        const int64_t per_block = (n + gridDim.x - 1) / gridDim.x;
        const int64_t b0 = p.lo[r] + per_block * blockIdx.x;
        const int64_t b1 = b0 + per_block < p.hi[r] ? b0 + per_block : p.hi[r];
        constexpr int kUnroll = 4;
        for (int64_t base = b0 + threadIdx.x; base < b1; base += (int64_t)kThreads * kUnroll) {
            uint4 v[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int64_t idx = base + (int64_t)u * kThreads;
                if (idx < b1) v[u] = ld_cg(src + idx);
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int64_t idx = base + (int64_t)u * kThreads;
                if (idx >= b1) continue;
                for (int i = 0; i < p.world; ++i)
                    if (i != p.rank) p.buf[i][idx] = v[u];
            }
        }
    }
    __threadfence_system();
    block_barrier(p.pad, p.rank, p.world, 2, epoch);   // every peer's ranges have landed in my buffer
    if (threadIdx.x == 0) *pad_gather_epoch(my_pad, blockIdx.x) = epoch;
}

}  // namespace
}  // namespace ck

extern "C" int launch_tp_gather_kernel(void* const* bufs, void* const* pads, int world, int rank, int64_t lo0, int64_t hi0,
                                       int64_t lo1, int64_t hi1, int blocks, cudaStream_t stream) {
    using namespace ck;
    if (!bufs || !pads) CK_FAIL(CK_ERR_NULL, "tp_gather: null pointer");
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
        CK_FAIL(CK_ERR_SHAPE, "tp_gather: rank %d of %d (at most %d ranks)", rank, world, kMaxRanks);
    if ((lo0 | hi0 | lo1 | hi1) & 15) CK_FAIL(CK_ERR_ALIGN, "tp_gather: range bounds must be multiples of 16 bytes");
    if (lo0 < 0 || lo1 < 0) CK_FAIL(CK_ERR_SHAPE, "tp_gather: negative offset");
    GatherParams p{};
    for (int i = 0; i < world; ++i) {
        if (!bufs[i] || !pads[i]) CK_FAIL(CK_ERR_NULL, "tp_gather: null buffer of rank %d", i);
        if (!aligned16(bufs[i]) || !aligned16(pads[i])) CK_FAIL(CK_ERR_ALIGN, "tp_gather: buffers must be 16-byte aligned");
        p.buf[i] = static_cast<uint4*>(bufs[i]);
        p.pad[i] = static_cast<uint32_t*>(pads[i]);
    }
    p.lo[0] = lo0 / 16; p.hi[0] = hi0 / 16; p.lo[1] = lo1 / 16; p.hi[1] = hi1 / 16;
    p.rank = rank;
    p.world = world;
    if (blocks <= 0) blocks = 148;
    if (blocks > kMaxBlocks) blocks = kMaxBlocks;
    tp_gather_kernel<<<blocks, kThreads, 0, stream>>>(p);
    return launch_status("tp_gather");
}

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant for a single rank.
//
// Some hosts of this library cannot allocate device memory when they call it: an inference runtime that
// hands out one fixed arena at start-up and forbids cudaMalloc afterwards, or a plugin running inside
// someone else's stream-ordered pipeline where an allocation would synchronise the device.  The exchange
// kernel needs a flag pad besides its inputs and outputs; this entry point keeps that pad in a
// file-scope device array instead of taking it from the caller, for the one-rank case (no peers to map
// it for): residual <- residual + gate * partial.
//
// Limits and rules:
//   - the pad serves at most kMaxBlocks (512) blocks: a larger `blocks` is refused (CK_ERR_SHAPE);
//     it occupies 34 816 bytes on every GPU that loads the library, until the process exits;
//   - the first call on a device looks the array's device address up (cudaGetSymbolAddress, with that
//     device current) and remembers it; make that first call outside any stream capture;
//   - all calls on a device share the pad, which keeps the epochs the previous call left: nothing needs
//     clearing (the kernel only ever compares against "the epoch I am about to write"), but two calls
//     that overlap on the GPU (different streams) race on it -- keep them on one stream;
//   - nothing here calls cudaMalloc, cudaFree or any allocating routine.
static __device__ __align__(256) uint32_t g_noalloc_pad[2 * ck::kMaxBlocks * ck::kMaxRanks + ck::kMaxBlocks];

extern "C" int launch_tp_exchange_noalloc_kernel(const void* partial, void* residual, const void* gate0, const void* gate1,
                                                 int64_t split_row, int64_t rows, int64_t cols, int dtype_code, int blocks,
                                                 cudaStream_t stream) {
    using namespace ck;
    if (blocks > kMaxBlocks)
        CK_FAIL(CK_ERR_SHAPE, "tp_exchange_noalloc: %d blocks asked for, the built-in flag pad serves at most %d", blocks, kMaxBlocks);
    // In host code the array's name is only a handle: the kernel needs its device address, per device.
    static uint32_t* pad_of_device[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) CK_FAIL((int)e, "tp_exchange_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) CK_FAIL(CK_ERR_UNSUPPORTED, "tp_exchange_noalloc: device index %d out of range", dev);
    if (pad_of_device[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_pad);
        if (e != cudaSuccess || p == nullptr)
            CK_FAIL(e != cudaSuccess ? (int)e : CK_ERR_UNSUPPORTED, "tp_exchange_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        pad_of_device[dev] = static_cast<uint32_t*>(p);
    }
    const void* partials[1] = {partial};
    void* residuals[1] = {residual};
    void* pads[1] = {pad_of_device[dev]};
    return launch_tp_exchange_kernel(partials, residuals, pads, nullptr, nullptr, 1, 0, gate0, gate1, split_row, rows, cols,
                                     dtype_code, blocks, stream);
}

extern "C" int launch_tp_exchange_kernel(const void* const* partials, void* const* residuals, void* const* pads,
                                         const void* mc_partial, void* mc_residual, int world,
                                         int rank, const void* gate0, const void* gate1, int64_t split_row, int64_t rows,
                                         int64_t cols, int dtype_code, int blocks, cudaStream_t stream) {
    return exchange_impl(partials, residuals, pads, mc_partial, mc_residual, world, rank, gate0, gate1, split_row, rows, cols,
                         dtype_code, blocks, stream, 0, 0, 0);
}

// Sequence-parallel form of the exchange: this rank sums rows [row_lo, row_hi) of all ranks' partial results and
// updates those rows of its OWN residual buffer only (nothing is pushed, no end barrier); the ranks' row ranges
// partition the matrix.  launch_tp_gather_kernel later distributes whatever the ranks derive from their rows.
extern "C" int launch_tp_reduce_rows_kernel(const void* const* partials, void* const* residuals, void* const* pads, int world,
                                            int rank, const void* gate0, const void* gate1, int64_t split_row, int64_t rows,
                                            int64_t cols, int64_t row_lo, int64_t row_hi, int dtype_code, int blocks,
                                            cudaStream_t stream) {
    return exchange_impl(partials, residuals, pads, nullptr, nullptr, world, rank, gate0, gate1, split_row, rows, cols,
                         dtype_code, blocks, stream, row_lo, row_hi, 1);
}

// Reads and clears the exchange kernel's status word (synchronises the device): 0, or
// CK_ERR_DEVICE_TIMEOUT when a wait for a peer ran out since the last call.
extern "C" int ck_tp_device_status(void) {
    int v = 0, zero = 0;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) CK_FAIL((int)e, "tp status: %s", cudaGetErrorString(e));
    e = cudaMemcpyFromSymbol(&v, ck::g_tp_status, sizeof(int));
    if (e != cudaSuccess) CK_FAIL((int)e, "tp status: %s", cudaGetErrorString(e));
    cudaMemcpyToSymbol(ck::g_tp_status, &zero, sizeof(int));
    if (v != 0) CK_FAIL(CK_ERR_DEVICE_TIMEOUT, "tp exchange kernel: the %s barrier of block %d timed out waiting for a peer",
                        (v >> 16) == 1 ? "start" : "end", v & 0xffff);
    return CK_OK;
}
