// Block-scaled GEMMs for sm_100a: NVFP4 (E2M1 data, E4M3 scale per 16) and MXFP8
// (E4M3 data, E8M0 scale per 32), written directly on tcgen05 / TMEM / TMA.
//
//   D[M,N] = alpha * sum_k (A[m,k] * SFA[m,k/B]) * (W[n,k] * SFW[n,k/B]) + bias[n]
//
// A is [M,K] and W is [N,K], both K-contiguous ("TN"); the scale factors arrive in
// the 128x4 tiled layout written by the quantizers (ck_common.cuh: sf_offset), one
// 512-byte tile per 128 rows x 4 scale columns.  Semantics follow
// comfy_kitchen/backends/eager/quantization.py:224-248 (NVFP4) and :369-404
// (MXFP8); the reference's CUDA backend forwards NVFP4 to a library GEMM
// (backends/cuda/ops/cublas_gemm_nvfp4.cu:64-340) and has no MXFP8 kernel.
//
// Kernel structure: persistent clusters of two CTAs (one per SM of a pair), 736
// threads each.  A pair works on a 256 x 256 output tile with tcgen05.mma
// .cta_group::2: CTA r of the pair holds rows 128r..128r+127 of the A tile, rows
// 128r..128r+127 of the W tile (i.e. half of N) and, in TMEM, the 128 x 256 fp32
// accumulator of its own rows.  Per CTA:
//   warp 0       TMA producer: per k-tile one 128x128B box of A, one 128x128B box of
//                W (both SWIZZLE_128B) and the scale tiles (its A rows' tile, both W
//                tiles) into a 5-stage shared-memory ring.
//   warp 1, 22   in the leader CTA (rank 0) the two MMA issuers, taking the k-tiles in
//                turn: four tcgen05.mma.kind::{mxf4nvf4,mxf8f6f4}.block_scale per
//                k-tile (256x256xK64 for FP4, xK32 for FP8); tcgen05.commit (multicast
//                to both CTAs) releases the stage and, per tile, publishes the
//                accumulator.  In both CTAs warp 1 allocates and frees TMEM.
//   warps 2-17   epilogue: each warp reads its 32 TMEM lanes x 64 columns into
//                registers, hands the accumulator back, then applies alpha and bias
//                (optionally the residual update), converts and writes through a
//                swizzled staging buffer with TMA stores (optionally into the buffers
//                of other ranks), overlapping the next tile's main loop.
// Two ways of getting the scale tiles from shared memory into TMEM (template flag kCp):
//   tcgen05.cp (default): every copy of both CTAs signals the LEADER's barrier
//                (cp.async.bulk.tensor ... .cta_group::2, no multicast); the MMA issuer
//                waits for that one barrier and issues tcgen05.cp.cta_group::2 for the
//                stage's scale tiles right in front of its MMAs; the scale buffer in
//                TMEM is indexed by the stage.  Warps 18-21 have no work.
//   movers:      warps 18-21 copy shared memory -> registers -> TMEM (tcgen05.st), one
//                warp per 32-lane quarter, into a ring of three scale buffers, and tell
//                the leader's issuers when a k-tile's scales (and, transitively, its
//                operands) are in place.
// Why this shape: measured on B200, one block-scaled MMA with 128 rows per CTA keeps
// the issuing thread ~140 clocks whether N is 64 or 256, so only N = 256 reaches the
// tensor cores' rate (hence also two issuing warps); with one CTA per tile that costs
// 96 KB of shared-memory traffic per k-tile, and pairing the CTAs halves the W traffic
// of each SM.  The 256-column accumulator leaves no room for a second one beside the
// scale buffers, hence the register-buffered epilogue.
//
// Every wait on an mbarrier in this file is bounded: on expiry the CTA records a
// status word, stops issuing work, drains its own copies and frees its TMEM before
// returning.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>
#include <unordered_map>

#include "ck_common.cuh"

namespace ck {
namespace {

constexpr int BM = 128;            // rows per CTA (256 per pair)
constexpr int BN = 256;            // columns per pair tile; each CTA stages 128 of the W rows
#ifndef CK_GEMM_STAGES
#define CK_GEMM_STAGES 5
#endif
constexpr int kStages = CK_GEMM_STAGES;
constexpr int kFirstEpiWarp = 2, kEpiWarps = 16;  // four warps per TMEM lane quarter, 64 columns each
constexpr int kFirstMoverWarp = kFirstEpiWarp + kEpiWarps;
constexpr int kSecondMmaWarp = kFirstMoverWarp + 4;   // issues the odd k-tiles; warp 1 the even ones
constexpr int kThreads = 32 * (kSecondMmaWarp + 1);
constexpr int kSfBufs = 3;
constexpr int kKbPerTile = 4;  // MMAs per k-tile

constexpr int kSmemA = BM * 128;            // 16 KB
constexpr int kSmemB = (BN / 2) * 128;      // 16 KB
constexpr int kSmemSfA = 4 * 512;           // up to four 512-byte tiles (NVFP4) for this CTA's 128 rows
constexpr int kSmemSfB = 2 * 4 * 512;       // two row tiles x four: all 256 columns
constexpr int kStageBytes = kSmemA + kSmemB + kSmemSfA + kSmemSfB;   // 38 KB
constexpr int kSmemOut = kEpiWarps * 2048;   // per-epilogue-warp staging: 32 rows x 64 bytes, 64-byte swizzle
constexpr int kSmemBytes = kStages * kStageBytes + kSmemOut + 256 /*barriers*/ + 1024 /*alignment slack*/;
static_assert(kStageBytes % 1024 == 0, "operand tiles need 1024-byte alignment");
static_assert(kSmemBytes <= 232448, "exceeds the 227 KB of shared memory a CTA can have");

constexpr uint32_t kTmemCols = 512;
// accumulator in columns 0..255; scale buffer b: A scales 16 columns at 256 + 48 b, W scales 32 columns after them
constexpr uint32_t kTmemAcc = 0;
__device__ __forceinline__ uint32_t tmem_sfa_col(uint32_t b) { return 256u + 48u * b; }
__device__ __forceinline__ uint32_t tmem_sfb_col(uint32_t b) { return 272u + 48u * b; }


constexpr uint32_t kSpinLimit = 1u << 22;   // polls of mbarrier.try_wait before giving up (a fraction of a second)

__device__ int g_gemm_status = 0;           // 0 ok; otherwise (code << 16 | CTA) of the first failure

enum : int { kTimeoutFull = 1, kTimeoutEmpty = 2, kTimeoutTmemFull = 3, kTimeoutTmemEmpty = 4, kTimeoutSfFull = 5 };

// ------------------------------------------------------------------ PTX wrappers

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// All threads of both CTAs.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Arrive on the same barrier in CTA `rank` of the cluster (which may be this CTA).
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t* bar, uint32_t rank) {
    asm volatile(
        "{ .reg .b32 ra; mapa.shared::cluster.u32 ra, %0, %1;\n"
        "mbarrier.arrive.shared::cluster.b64 _, [ra]; }"
        ::"r"(smem_u32(bar)), "r"(rank) : "memory");
}
// Plain (CTA-scope) waits also serve the barriers that the peer CTA's warps arrive on: what those arrivals
// publish is TMEM content and TMA-written shared memory, ordered by the tcgen05 fences around them, not
// generic-proxy data.  (A cluster-scope release/acquire pair here measured ~1000 clocks per arrival.)
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Non-blocking look at a barrier phase (try_wait may suspend the thread for a while when the phase is
// still pending; this never does).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait, called by all 32 lanes of a warp.  Returns false (to every lane alike)
// when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
    // Phase already complete (seen by every lane): skip try_wait, which costs ~150 clocks even then.
    if (__all_sync(0xffffffffu, mbar_test_wait(bar, parity))) return true;
    bool done = false;
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) { done = true; break; }
        if ((i & 1023u) == 1023u && *abort_flag) break;
    }
    if (!done && !*abort_flag) {
        *abort_flag = 1;
        atomicCAS(&g_gemm_status, 0, (code << 16) | (int)(blockIdx.x & 0xffff));
    }
    return __all_sync(0xffffffffu, done);
}

// One lane of a converged warp, chosen by the hardware.  Code that wraps a single asm statement in
// `if (elect_one())` stays warp-uniform, so its operands can live in uniform registers.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{ .reg .pred p; elect.sync _|p, 0xffffffff; selp.u32 %0, 1, 0, p; }" : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}
// Address of the same shared-memory location in CTA `rank` of the cluster (shared::cluster window).
__device__ __forceinline__ uint32_t cluster_addr(const void* p, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(p)), "r"(rank));
    return a;
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar_cluster_addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(bar_cluster_addr), "r"(bytes) : "memory");
}
// Tile load whose completion is signalled on a barrier that may live in the peer CTA of the pair (no multicast:
// the data still lands in the executing CTA's shared memory only).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Shared -> global tile store (clipped at the tensor's edges), tracked by the issuing thread's bulk groups.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(c0), "r"(c1) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// The tcgen05 issue wrappers below are called by all 32 lanes of the issuing warp with identical
// arguments; one elected lane executes the instruction.
// Arrives (once the MMAs issued so far have completed) on the barrier at this shared-memory offset in
// both CTAs of the pair.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    if (elect_one())
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
// Shared-memory descriptors are built from a 32-bit low word (start address >> 4, plus the
// leading-offset field for the swizzled form) and a constant high word:
//   operand tiles: K-major, 128-byte rows, 128-byte swizzle, 8-row groups 1024 bytes apart
//                  -> hi = SBO 64 | version 1 (bit 46) | layout SWIZZLE_128B (bits 61-63)
constexpr uint32_t kDescHiOperand = 64u | (1u << 14) | (2u << 29);
constexpr uint32_t kDescLoLbo1 = 1u << 16;

//   scale tiles: 32 rows x 16 bytes, no swizzle, 8-row groups 128 bytes apart -> hi = SBO 8 | version 1
constexpr uint32_t kDescHiScale = 8u | (1u << 14);
// One 512-byte scale tile, shared memory -> TMEM columns [taddr, taddr + 4), replicated into the four 32-lane
// quarters, in both CTAs of the pair (each from its own shared memory at the same offset).
__device__ __forceinline__ void tc_cp_scale_pair(uint32_t taddr, uint32_t desc_lo) {
    if (elect_one())
    asm volatile(
        "{ .reg .b64 d; mov.b64 d, {%1, %2};\n"
        "tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], d; }"
        ::"r"(taddr), "r"(desc_lo), "n"(kDescHiScale) : "memory");
}

template <bool kFp4>
__device__ __forceinline__ void tc_mma(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate,
                                       uint32_t sfa, uint32_t sfb) {
    if (!elect_one()) return;
    if (kFp4) {
        asm volatile(
            "{ .reg .pred p; .reg .b64 da, db; setp.ne.b32 p, %4, 0;\n"
            "mov.b64 da, {%1, %7}; mov.b64 db, {%2, %7};\n"
            "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], da, db, %3, [%5], [%6], p; }"
            ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb), "n"(kDescHiOperand) : "memory");
    } else {
        asm volatile(
            "{ .reg .pred p; .reg .b64 da, db; setp.ne.b32 p, %4, 0;\n"
            "mov.b64 da, {%1, %7}; mov.b64 db, {%2, %7};\n"
            "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], da, db, %3, [%5], [%6], p; }"
            ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb), "n"(kDescHiOperand) : "memory");
    }
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Register -> TMEM stores: thread i of the warp writes lane (32 * (warp % 4) + i), consecutive columns.
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tc_st8(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void tc_st4(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

struct GemmParams {
    const uint8_t* sfa;
    const uint8_t* sfb;
    const void* bias;
    const float* alpha;   // device scalar or null (1.0)
    int M, N, K;          // K in elements
    int sf_tiles_k;       // 512-byte scale tiles along K (= padded scale columns / 4)
    int sf_row_tiles_a;   // 128-row scale tiles of A
    int sf_row_tiles_b;   // 128-row scale tiles of W
    int out_code, bias_code;
    int tiles_m, tiles_n; // pair tiles (256 x 256)
    // fused residual update (16-bit outputs only): D = residual + gate[n] * round(alpha * acc + bias); both null = off
    const void* residual; // [M, N] in the output dtype, row pitch N (may be D itself)
    const void* gate;     // [N] in the output dtype
};

// Scattered output (tensor-parallel reduce-scatter fused into the epilogue, kEpi = 2): output row r of this GEMM is
// row row_offset + r of a matrix whose rows [bounds[d], bounds[d+1]) belong to rank d; its tile rows go to rank d's
// buffer through m[d], rows counted from bounds[d].
struct OutMaps {
    CUtensorMap m[8];
    int world, row_offset;
    int bounds[9];
};

// Tile order: bands of kGroupM tile rows, walked column by column inside a band, so that the ~74 tiles in
// flight at any time cover a compact block of the output (about kGroupM x 18 tiles) and re-use the same few A and
// W tiles from L2 while the much larger output streams through it.  Band heights of 2 to 4 measured alike and
// 2-4 % ahead of 8 on the K = 3072 shapes (timed in one process, L2 flushed before every launch); 1 (row-major)
// loses a quarter on narrow outputs with long K.
#ifndef CK_GEMM_GROUP_M
#define CK_GEMM_GROUP_M 4
#endif
__device__ __forceinline__ void tile_coords(int tile, const GemmParams& p, int& tm, int& tn) {
    constexpr int kGroupM = CK_GEMM_GROUP_M;
    const int per_band = kGroupM * p.tiles_n;
    const int band = tile / per_band, in_band = tile - band * per_band;
    const int first = band * kGroupM;
    const int rows = min(kGroupM, p.tiles_m - first);
    tn = in_band / rows;
    tm = first + (in_band - tn * rows);
}

template <typename T16>
__device__ __forceinline__ uint32_t pack_pair(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);   // .x = a in the low half
    return *reinterpret_cast<const uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack_pair<__half>(float a, float b) {
    const __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// kCp = false: scale movers (warps 18-21) as described at the top of the file.
// kCp = true:  no movers.  The scale tiles arrive through tensor maps (map_sfa, map_sfb) like the operands, every
//              copy of both CTAs signals the LEADER's full[] barrier (cp.async.bulk.tensor with .cta_group::2, no
//              multicast), and the MMA issuer itself moves the stage's scale tiles into TMEM with tcgen05.cp
//              (.cta_group::2: one instruction copies in both CTAs, each from its own shared memory) right before
//              the stage's MMAs; the scale buffer in TMEM is indexed by the stage, so it is free when the stage is.
template <bool kFp4, int kEpi, bool kCp>   // kEpi: 0 plain output, 1 fused residual update, 2 output scattered over ranks
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_blockscaled_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_sfa,
                        const __grid_constant__ CUtensorMap map_sfb, const __grid_constant__ OutMaps omaps,
                        const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled tiles (the same offset in both CTAs of the pair)
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stage_base = smem;
    uint8_t* s_out = smem + kStages * kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_out + kSmemOut);
    uint64_t* full = bars;                    // [kStages]  this CTA's TMA copies landed -> its scale movers
    uint64_t* empty = bars + kStages;         // [kStages]  movers have read the scales + the pair's MMAs of the k-tile are
                                              //            done -> TMA producer (stage free), movers (scale buffer free)
    uint64_t* sf_full = empty + kStages;      // [kSfBufs]  (leader's) both CTAs' scales in TMEM -> MMA issuer
    uint64_t* tmem_full = sf_full + kSfBufs;  //            accumulator complete -> epilogue
    uint64_t* tmem_empty = tmem_full + 1;     //            (leader's) both CTAs' accumulators copied out -> MMA issuer
    uint64_t* tile_open = tmem_empty + 1;     //            first MMA of a tile issued -> the second MMA issuer
    uint64_t* drain = tile_open + 1;          // [2]        an MMA issuer that gave up: its MMAs in flight are done
    uint32_t* s_tmem_base = reinterpret_cast<uint32_t*>(drain + 2);
    volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem_base + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();              // 0 = leader
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    constexpr int kElemsPerTile = kFp4 ? 256 : 128;       // K elements per k-tile (128 bytes per row)
    constexpr int kMmaK = kFp4 ? 64 : 32;
    constexpr int kSfTilesPerStage = kFp4 ? 4 : 1;        // 512-byte tiles per 128 rows per k-tile
    const int k_tiles = (p.K + kElemsPerTile - 1) / kElemsPerTile;
    const int num_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], kCp ? 2 : 1); mbar_init(&empty[s], kCp ? 1 : 5); }
        for (int b = 0; b < kSfBufs; ++b) mbar_init(&sf_full[b], 8);
        mbar_init(tmem_full, 2);   // one commit per tile from each MMA issuer
        mbar_init(tile_open, 1);
        mbar_init(&drain[0], 1);
        mbar_init(&drain[1], 1);
        mbar_init(tmem_empty, 2 * kEpiWarps);
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();   // barriers of both CTAs initialised, TMEM of both allocated
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        uint32_t it = 0;  // k-tiles issued so far (ring position)
        bool ok = true;
        const size_t sf_row_pitch = (size_t)p.sf_tiles_k * 512;
        for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
            int tm, tn;
            tile_coords(tile, p, tm, tn);
            const int row_tile_a = tm * 2 + (int)rank;     // this CTA's 128 rows of A
            const bool have_a = row_tile_a < p.sf_row_tiles_a;
            const int row_tile_b = tn * 2;                 // first of the two 128-row scale tiles of the W tile
            const int b_tiles = (row_tile_b + 1 < p.sf_row_tiles_b) ? 2 : 1;
            const uint8_t* sfa_src = p.sfa + (size_t)row_tile_a * sf_row_pitch;
            const uint8_t* sfb_src = p.sfb + (size_t)row_tile_b * sf_row_pitch;
            for (int kt = 0; kt < k_tiles && ok; ++kt, ++it) {
                const int s = it % kStages;
                const uint32_t round = it / kStages;
                if (round > 0) ok = mbar_wait(&empty[s], (round - 1) & 1, s_abort, kTimeoutEmpty);
                if (!ok) break;
                // operands are computed by the whole warp; one elected lane issues the copies
                uint8_t* st = stage_base + s * kStageBytes;
                int n_sf = p.sf_tiles_k - kt * kSfTilesPerStage;  // scale tiles valid in this k-tile (the last may be short)
                if (n_sf > kSfTilesPerStage) n_sf = kSfTilesPerStage;
                const uint32_t sf_bytes = (uint32_t)n_sf * 512u;
                const size_t sf_off = (size_t)kt * (kSfTilesPerStage * 512);
                const uint32_t tx_bytes = kSmemA + kSmemB + sf_bytes * ((have_a ? 1 : 0) + b_tiles);
                if constexpr (kCp) {
                    // every box is transferred whole (zero-filled outside the tensor): a fixed byte count per stage
                    constexpr uint32_t kSfBox = kSfTilesPerStage * 512u;
                    const uint32_t lead_full = cluster_addr(&full[s], 0);
                    if (elect_one()) {
                        mbar_expect_tx_cluster(lead_full, kSmemA + kSmemB + 3u * kSfBox);
                        tma_load_2d_pair(st, &map_a, kt * 128, tm * 256 + (int)rank * BM, lead_full);
                        tma_load_2d_pair(st + kSmemA, &map_b, kt * 128, tn * BN + (int)rank * (BN / 2), lead_full);
                        tma_load_2d_pair(st + kSmemA + kSmemB, &map_sfa, kt * kSfTilesPerStage * 64, row_tile_a, lead_full);
                        tma_load_2d_pair(st + kSmemA + kSmemB + kSmemSfA, &map_sfb, kt * kSfTilesPerStage * 64, row_tile_b, lead_full);
                    }
                } else
                if (elect_one()) {
                    mbar_expect_tx(&full[s], tx_bytes);
                    tma_load_2d(st, &map_a, kt * 128, tm * 256 + (int)rank * BM, &full[s]);
                    tma_load_2d(st + kSmemA, &map_b, kt * 128, tn * BN + (int)rank * (BN / 2), &full[s]);
                    if (have_a) bulk_load(st + kSmemA + kSmemB, sfa_src + sf_off, sf_bytes, &full[s]);
                    bulk_load(st + kSmemA + kSmemB + kSmemSfA, sfb_src + sf_off, sf_bytes, &full[s]);
                    if (b_tiles == 2)
                        bulk_load(st + kSmemA + kSmemB + kSmemSfA + kSmemSfB / 2, sfb_src + sf_row_pitch + sf_off,
                                  sf_bytes, &full[s]);
                }
                __syncwarp();
            }
        }
        // drain: every copy this warp issued must have landed before the CTA may exit.  (kCp: completion is
        // signalled in the leader only; a finished kernel has consumed every stage, and a CTA that gave up waits
        // long enough below for copies in flight to land.)
        if (kCp && !ok) __nanosleep(50000);
        const uint32_t first = it > (uint32_t)kStages ? it - kStages : 0;
        for (uint32_t j = (kCp && rank != 0) ? it : first; j < it; ++j) {
            const int s = j % kStages;
            (void)mbar_wait(&full[s], (j / kStages) & 1, s_abort, kTimeoutFull);
        }
    } else if (kCp && warp >= kFirstMoverWarp && warp < kSecondMmaWarp) {
        // (these warps have no work in this variant)
    } else if (warp >= kFirstMoverWarp && warp < kSecondMmaWarp) {
        // ------------------------------------------------------------ scale movers (smem -> registers -> TMEM)
        // A 512-byte scale tile is 32 rows x 16 bytes: row i holds, for the four 32-row groups g of a
        // 128-row tile, the scale bytes of row 32g + i.  The MMA wants it in TMEM as 32 lanes x 4 columns
        // (column g), the same in each 32-lane quarter.  Each mover warp owns one quarter: lane i reads row
        // i with one 128-bit load per tile and stores its words to TMEM lane i.  k-tile `it` uses scale
        // buffer it % 3, last read by the MMAs of k-tile it - 3, whose completion empty[] reports.
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        uint32_t it = 0;
        bool ok = true;
        for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
            for (int kt = 0; kt < k_tiles && ok; ++kt, ++it) {
                const int s = it % kStages;
                const uint32_t b = it % kSfBufs;
                ok = mbar_wait(&full[s], (it / kStages) & 1, s_abort, kTimeoutFull);
                if (!ok) break;
                const uint8_t* sfa_s = stage_base + s * kStageBytes + kSmemA + kSmemB + lane * 16;
                const uint8_t* sfb_s = sfa_s + kSmemSfA;
                constexpr int kNa = kFp4 ? 16 : 4, kNb = kFp4 ? 32 : 8;   // words per lane: A scales, W scales
                uint32_t ra[kNa], rb[kNb];
                {
#pragma unroll
                    for (int t = 0; t < kSfTilesPerStage; ++t) {  // k-block t: A columns 4t.., W columns 8t.. (first, then second row tile)
                        const uint4 v = *reinterpret_cast<const uint4*>(sfa_s + t * 512);
                        ra[4 * t] = v.x; ra[4 * t + 1] = v.y; ra[4 * t + 2] = v.z; ra[4 * t + 3] = v.w;
                        const uint4 v0 = *reinterpret_cast<const uint4*>(sfb_s + t * 512);
                        const uint4 v1 = *reinterpret_cast<const uint4*>(sfb_s + kSmemSfB / 2 + t * 512);
                        rb[8 * t + 0] = v0.x; rb[8 * t + 1] = v0.y; rb[8 * t + 2] = v0.z; rb[8 * t + 3] = v0.w;
                        rb[8 * t + 4] = v1.x; rb[8 * t + 5] = v1.y; rb[8 * t + 6] = v1.z; rb[8 * t + 7] = v1.w;
                    }
                    // make sure the loads have returned before the stage's scale area is handed back
                    asm volatile("" ::"r"(ra[0]), "r"(rb[0]), "r"(rb[4]) : "memory");
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
                if (it >= (uint32_t)kSfBufs) {
                    const uint32_t prev = it - kSfBufs;
                    ok = mbar_wait(&empty[prev % kStages], (prev / kStages) & 1, s_abort, kTimeoutEmpty);
                    if (!ok) break;
                }
                tc_fence_after();
                const uint32_t t_sfa = tmem_base + lane_base + tmem_sfa_col(b);
                const uint32_t t_sfb = tmem_base + lane_base + tmem_sfb_col(b);
                if constexpr (kFp4) {
                    tc_st16(t_sfa, ra);
                    tc_st16(t_sfb, rb);
                    tc_st16(t_sfb + 16, rb + 16);
                } else {
                    tc_st4(t_sfa, ra);
                    tc_st8(t_sfb, rb);
                }
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(&sf_full[b], 0);   // the leader's barrier
            }
        }
    } else if (warp == 1 || warp == kSecondMmaWarp) {
        // ------------------------------------------------------------ MMA issuers (leader CTA only)
        // Issuing one block-scaled MMA keeps a thread ~100 clocks and the bookkeeping of a k-tile (barrier
        // look-ahead, commit) another ~150, while the tensor cores need 128 clocks per MMA: a single issuer
        // cannot keep them fed.  Two warps therefore take the k-tiles in turn (warp 1 the even ones).  The
        // accumulation order does not matter except for the first MMA of a tile, which overwrites: the second
        // issuer waits (tile_open) until the first has issued it.  A commit covers the committing thread's own
        // MMAs, so each issuer releases the stages it consumed and both commit to tmem_full.
        const uint32_t which = warp == 1 ? 0u : 1u;
        if (rank == 0) {
        const uint32_t idesc_base = (kFp4 ? ((1u << 7) | (1u << 10)) : 0u) | ((uint32_t)(BN >> 3) << 17) |
                                    (kFp4 ? 0u : (1u << 23)) | ((uint32_t)((2 * BM) >> 4) << 24);
        const uint32_t smem16 = (smem_u32(stage_base) & 0x3ffffu) >> 4;
        const bool tail_full = (p.K % kElemsPerTile) == 0;
        uint32_t it = 0, local_tile = 0;
        bool ok = true, ready = false;
        for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local_tile) {
            ready = false;
            if (local_tile > 0) ok = mbar_wait(tmem_empty, (local_tile - 1) & 1, s_abort, kTimeoutTmemEmpty);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + kTmemAcc;
            if (which == 1 && k_tiles > 1) {   // the overwriting MMA must be in the pipe before any of mine
                ok = mbar_wait(tile_open, local_tile & 1, s_abort, kTimeoutTmemEmpty);
                if (!ok) break;
            }
            for (int kt = 0; kt < k_tiles && ok; ++kt, ++it) {
                if ((uint32_t)(kt & 1) != which) continue;
                const int s = it % kStages;
                const uint32_t sb = kCp ? (uint32_t)s : it % kSfBufs;
                // The movers of both CTAs publish sf_full only after they saw their full[s], so this one wait
                // covers the operands too.  `ready` is an early look taken while the previous k-tile was issued.
                // (kCp: full[s] here in the leader collects the copies of both CTAs.)
                if (!__all_sync(0xffffffffu, ready))
                    ok = kCp ? mbar_wait(&full[s], (it / kStages) & 1, s_abort, kTimeoutFull)
                             : mbar_wait(&sf_full[sb], (it / kSfBufs) & 1, s_abort, kTimeoutSfFull);
                if (!ok) break;
                tc_fence_after();
                // every descriptor of this stage is "stage start >> 4" plus a constant (the same in both CTAs)
                const uint32_t st16 = smem16 + (uint32_t)s * (kStageBytes >> 4);
                const uint32_t a_lo = st16 | kDescLoLbo1, b_lo = (st16 + (kSmemA >> 4)) | kDescLoLbo1;
                const uint32_t t_sfa = tmem_base + tmem_sfa_col(sb), t_sfb = tmem_base + tmem_sfb_col(sb);
                int n_kb = kKbPerTile;
                if (kt + 1 == k_tiles && !tail_full) n_kb = (p.K - kt * kElemsPerTile + kMmaK - 1) / kMmaK;
                if constexpr (kCp) {
                    // this stage's scale tiles: shared memory -> TMEM, in both CTAs, ahead of the MMAs in the same pipe
                    const uint32_t sfa16 = (st16 + ((kSmemA + kSmemB) >> 4)) | kDescLoLbo1;
                    const uint32_t sfb16 = (st16 + ((kSmemA + kSmemB + kSmemSfA) >> 4)) | kDescLoLbo1;
#pragma unroll
                    for (int t = 0; t < kSfTilesPerStage; ++t) {
                        tc_cp_scale_pair(t_sfa + 4 * t, sfa16 + t * 32);
                        tc_cp_scale_pair(t_sfb + 8 * t, sfb16 + t * 32);
                        tc_cp_scale_pair(t_sfb + 8 * t + 4, sfb16 + kSfTilesPerStage * 32 + t * 32);
                    }
                }
#pragma unroll
                for (int kb = 0; kb < kKbPerTile; ++kb) {
                    if (kb < n_kb) {
                        // 32 bytes along K per MMA inside the 128-byte swizzled row
                        uint32_t idesc = idesc_base, sfa = t_sfa, sfb = t_sfb;
                        if (kFp4) { sfa += 4 * kb; sfb += 8 * kb; }
                        else { idesc |= ((uint32_t)kb << 29) | ((uint32_t)kb << 4); }
                        tc_mma<kFp4>(d_tmem, a_lo + 2 * kb, b_lo + 2 * kb, idesc, (kt > 0 || kb > 0) ? 1u : 0u, sfa, sfb);
                        if (kt == 0 && kb == 0 && lane == 0) mbar_arrive(tile_open);   // which == 0 here
                    }
                    // the pipe is busy with these for a while: look at my next k-tile's barrier now
                    if (kb == 1) ready = kt + 2 < k_tiles &&
                                         (kCp ? mbar_test_wait(&full[(it + 2) % kStages], ((it + 2) / kStages) & 1)
                                              : mbar_test_wait(&sf_full[(it + 2) % kSfBufs], ((it + 2) / kSfBufs) & 1));
                }
                tc_commit_pair(&empty[s]);                      // stage and scale buffer reusable once these MMAs are done
            }
            // the accumulator is complete when both issuers' MMAs are (an issuer that had no k-tile in this tile
            // commits nothing and arrives at once)
            if (ok) tc_commit_pair(tmem_full);
        }
        if (!ok) {
            // Gave up on a wait: the MMAs already issued still read both CTAs' stages and write both accumulators.
            // Wait (bounded) until they are done before this CTA goes on to the final cluster barrier.
            tc_commit_pair(&drain[which]);
            (void)mbar_wait(&drain[which], 0, s_abort, kTimeoutTmemFull);
        }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..17)
        // Lane i of a warp owns TMEM lane 32q + i, i.e. one output row, and 64 of its columns.  The warp copies
        // them to registers and hands the accumulator back at once; alpha, bias, the conversion and the store
        // overlap the next tile's MMAs.  Results leave through shared memory, 64 bytes per row at a time: the
        // lane writes 16-byte pieces placed with the 64-byte swizzle, which keeps the writes conflict-free, and
        // a TMA store moves the 32 x 64-byte chunk to global memory, clipped at the matrix edges.  Lane 0 issues the warp's stores and waits for the previous one to have read the
        // staging buffer before it is overwritten.
        const int e = warp - kFirstEpiWarp;
        const int q = warp & 3;    // TMEM lanes 32q .. 32q+31 belong to this warp
        const int part = e >> 2;   // which 64 columns of the tile
        uint8_t* stg = s_out + e * 2048;
        const float alpha = p.alpha ? __ldg(p.alpha) : 1.0f;
        uint32_t local_tile = 0;
        bool ok = true;
        for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local_tile) {
            int tm, tn;
            tile_coords(tile, p, tm, tn);
            const int n0 = tn * BN + part * 64;
            // bias for these 64 columns: lane l keeps columns l and l + 32, the others fetch them with shuffles
            float bias_reg[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                float b = 0.0f;
                const int n = n0 + k * 32 + lane;
                if (p.bias && n < p.N) {
                    if (p.bias_code == CK_F32) b = static_cast<const float*>(p.bias)[n];
                    else if (p.bias_code == CK_F16) b = __half2float(static_cast<const __half*>(p.bias)[n]);
                    else b = __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[n]);
                }
                bias_reg[k] = b;
            }
            auto bias_at = [&](int col) { return __shfl_sync(0xffffffffu, bias_reg[col >> 5], col & 31); };
            // fused residual update: gate for these 64 columns, kept like the bias
            constexpr bool fuse_res = kEpi == 1;
            float gate_reg[2] = {0.0f, 0.0f};
            if (fuse_res) {
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const int n = n0 + k * 32 + lane;
                    if (n < p.N)
                        gate_reg[k] = p.out_code == CK_F16 ? __half2float(static_cast<const __half*>(p.gate)[n])
                                                           : __bfloat162float(static_cast<const __nv_bfloat16*>(p.gate)[n]);
                }
            }
            auto gate_at = [&](int col) { return __shfl_sync(0xffffffffu, gate_reg[col >> 5], col & 31); };
            ok = mbar_wait(tmem_full, local_tile & 1, s_abort, kTimeoutTmemFull);
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + kTmemAcc + ((uint32_t)(q * 32) << 16) + (uint32_t)(part * 64);
            const int row0 = tm * 256 + (int)rank * BM + q * 32;   // first of this warp's 32 rows
            uint32_t r[2][32];
            tc_ld32(acc, r[0]);
            tc_ld32(acc + 32, r[1]);
            tc_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tmem_empty, 0);
            const bool store_ok = row0 < p.M;
            // a staging chunk is 32 rows x 64 bytes: 32 columns of a 16-bit output, 16 of an fp32 one
            const int n_chunks = p.out_code == CK_F32 ? 4 : 2;
            const int chunk_cols = p.out_code == CK_F32 ? 16 : 32;
            uint8_t* my_row = stg + lane * 64;
            const int sw = (lane >> 1) & 3;   // 64-byte swizzle: 16-byte piece index ^ ((row / 2) % 4)
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
                if (ch < n_chunks) {
                    // the residual values this lane's row needs for the chunk (its 32 columns = 64 bytes), fetched
                    // before the staging buffer is waited for
                    uint4 xres[4];
                    if (fuse_res) {
                        const int64_t row = row0 + lane;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int col = n0 + ch * 32 + 8 * j;
                            xres[j] = make_uint4(0u, 0u, 0u, 0u);
                            if (row < p.M && col < p.N)
                                xres[j] = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.residual) + row * p.N + col);
                        }
                    }
                    if (lane == 0) bulk_wait_read_all();
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 4; ++j) {   // one 16-byte piece: 8 columns (16-bit) or 4 (fp32)
                        uint32_t w[4];
                        if (p.out_code != CK_F32) {
                            const uint32_t xw[4] = {xres[j].x, xres[j].y, xres[j].z, xres[j].w};
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int c = 32 * (ch & 1) + 8 * j + 2 * i;
                                float a = fmaf(__uint_as_float(r[c >> 5][c & 31]), alpha, bias_at(c));
                                float b = fmaf(__uint_as_float(r[c >> 5][(c & 31) + 1]), alpha, bias_at(c + 1));
                                if (fuse_res) {
                                    // y rounded as it would have been stored, then x + gate * y with the product and the
                                    // sum rounded separately (an elementwise addcmul on the stored tensors)
                                    float x0, x1;
                                    if (p.out_code == CK_BF16) {
                                        a = __bfloat162float(__float2bfloat16_rn(a)); b = __bfloat162float(__float2bfloat16_rn(b));
                                        x0 = __uint_as_float(xw[i] << 16); x1 = __uint_as_float(xw[i] & 0xffff0000u);
                                    } else {
                                        a = __half2float(__float2half_rn(a)); b = __half2float(__float2half_rn(b));
                                        const float2 xf = __half22float2(*reinterpret_cast<const __half2*>(&xw[i]));
                                        x0 = xf.x; x1 = xf.y;
                                    }
                                    a = __fadd_rn(x0, __fmul_rn(gate_at(c), a));
                                    b = __fadd_rn(x1, __fmul_rn(gate_at(c + 1), b));
                                }
                                w[i] = p.out_code == CK_BF16 ? pack_pair<__nv_bfloat16>(a, b) : pack_pair<__half>(a, b);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int c = 16 * ch + 4 * j + i;
                                w[i] = __float_as_uint(fmaf(__uint_as_float(r[c >> 5][c & 31]), alpha, bias_at(c)));
                            }
                        }
                        *reinterpret_cast<uint4*>(my_row + ((j ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                    fence_async_smem();
                    __syncwarp();
                    const int col = n0 + ch * chunk_cols;
                    if (lane == 0 && store_ok && col < p.N) {
                        if constexpr (kEpi == 2) {
                            // the 32 rows of this chunk belong to one rank (bounds are multiples of 128): its buffer, its row count
                            const int grow = omaps.row_offset + row0;
                            int d = 0;
                            while (d + 1 < omaps.world && grow >= omaps.bounds[d + 1]) ++d;
                            tma_store_2d(&omaps.m[d], stg, col, grow - omaps.bounds[d]);
                        } else {
                            tma_store_2d(&map_out, stg, col, row0);
                        }
                    }
                }
            }
        }
        if (lane == 0) bulk_wait_all();   // the staging buffer must outlive the stores that read it
        __syncwarp();
    }

    // Neither CTA may leave (or free its TMEM) while the other can still signal its barriers, read its
    // shared memory or write its TMEM through a paired MMA.
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------ host side

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(sym);
    });
    return fn;
}

// [rows, row_bytes] byte matrix, box = 128 bytes x box_rows, 128-byte swizzle, zero fill outside.
int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t row_bytes, int box_rows) {
    EncodeFn enc = get_encode();
    if (!enc) CK_FAIL(CK_ERR_UNSUPPORTED, "scaled_mm: cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) CK_FAIL(CK_ERR_UNSUPPORTED, "scaled_mm: cuTensorMapEncodeTiled failed with %d", (int)r);
    return CK_OK;
}

// Output [rows, cols] of 2- or 4-byte elements, box = 64 bytes x 32 rows, 64-byte swizzle (the layout the
// epilogue writes into its staging buffers).
int make_output_map(CUtensorMap* map, void* base, int64_t rows, int64_t cols, int elem_bytes) {
    EncodeFn enc = get_encode();
    if (!enc) CK_FAIL(CK_ERR_UNSUPPORTED, "scaled_mm: cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(cols * elem_bytes)};
    cuuint32_t box[2] = {(cuuint32_t)(64 / elem_bytes), 32u};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = enc(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, base, dims,
                     strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                     CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) CK_FAIL(CK_ERR_UNSUPPORTED, "scaled_mm: cuTensorMapEncodeTiled (output) failed with %d", (int)r);
    return CK_OK;
}

// Encoded tensor maps are a pure function of (base, rows, row length, box, element size); a model calls the
// GEMM with the same few weights and activation buffers over and over, so the three driver calls per launch
// are replaced by a lookup.  (ck_set_option("gemm_map_cache", 0) turns the cache off.)
struct MapKey {
    const void* base; int64_t rows, cols; int kind;   // kind: box rows for operands, -(element bytes) for outputs
    bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && cols == o.cols && kind == o.kind; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
        h ^= (uint64_t)k.rows * 0xC2B2AE3D27D4EB4Full + ((uint64_t)k.cols << 7) + (uint64_t)(k.kind + 64);
        return (size_t)(h ^ (h >> 29));
    }
};
// Tiled scale buffer as a 2-D tensor: one row per 128-row scale tile row, tiles_k * 512 bytes long (64-bit
// elements, so that a box can span four 512-byte tiles); box = box_tiles tiles x box_rows tile rows, no swizzle.
int make_scale_map(CUtensorMap* map, const void* base, int64_t row_tiles, int64_t tiles_k, int box_tiles, int box_rows) {
    EncodeFn enc = get_encode();
    if (!enc) CK_FAIL(CK_ERR_UNSUPPORTED, "scaled_mm: cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)tiles_k * 64u, (cuuint64_t)row_tiles};
    cuuint64_t strides[1] = {(cuuint64_t)tiles_k * 512u};
    cuuint32_t box[2] = {(cuuint32_t)box_tiles * 64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) CK_FAIL(CK_ERR_UNSUPPORTED, "scaled_mm: cuTensorMapEncodeTiled (scales) failed with %d", (int)r);
    return CK_OK;
}

int cached_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int kind) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{base, rows, cols, kind};
    if (g_gemm_map_cache) {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *map = it->second; return CK_OK; }
    }
    // kind: 1 .. 999 operand (box rows), -2 / -4 output (element bytes), 1000 + 10 * box_tiles + box_rows scales
    const int rc = kind >= 1000 ? make_scale_map(map, base, rows, cols, (kind - 1000) / 10, (kind - 1000) % 10)
                 : kind > 0     ? make_operand_map(map, base, rows, cols, kind)
                                : make_output_map(map, const_cast<void*>(base), rows, cols, -kind);
    if (rc == CK_OK && g_gemm_map_cache) {
        std::lock_guard<std::mutex> lock(mu);
        if (cache.size() >= 8192) cache.clear();   // bounded: a long-running process with ever-new buffers starts over
        cache.emplace(key, *map);
    }
    return rc;
}

int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        cached[dev] = n > 0 ? n : 148;
    }
    return cached[dev];
}

template <bool kFp4, int kEpi = 0>
int launch_gemm(const void* a, const void* sfa, const void* b, const void* sfb, void* d, const void* bias,
                int bias_code, int64_t M, int64_t N, int64_t K, const float* alpha, int out_code, cudaStream_t stream,
                const void* residual = nullptr, const void* gate = nullptr, void* const* scatter_dests = nullptr,
                const int64_t* scatter_bounds = nullptr, int scatter_world = 0, int64_t scatter_row_offset = 0) {
    const char* what = kFp4 ? "scaled_mm_nvfp4" : "scaled_mm_mxfp8";
    if (scatter_world < 0 || scatter_world > 8) CK_FAIL(CK_ERR_SHAPE, "%s: scatter over %d ranks (at most 8)", what, scatter_world);
    if (scatter_world > 0) {
        if (!scatter_dests || !scatter_bounds) CK_FAIL(CK_ERR_NULL, "%s: scatter needs destinations and bounds", what);
        if (out_code == CK_F32 || residual) CK_FAIL(CK_ERR_UNSUPPORTED, "%s: scattered output is 16-bit and without residual", what);
        d = scatter_dests[0];   // (only checked for alignment below)
    }
    if ((residual != nullptr) != (gate != nullptr)) CK_FAIL(CK_ERR_NULL, "%s: residual and gate go together", what);
    if (residual && out_code == CK_F32) CK_FAIL(CK_ERR_DTYPE, "%s: the fused residual update needs a 16-bit output", what);
    if (residual && (!aligned16(residual) || !aligned16(gate))) CK_FAIL(CK_ERR_ALIGN, "%s: residual and gate must be 16-byte aligned", what);
    if (!a || !sfa || !b || !sfb || !d) CK_FAIL(CK_ERR_NULL, "%s: null pointer", what);
    if (M <= 0 || N <= 0 || K <= 0 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX)
        CK_FAIL(CK_ERR_SHAPE, "%s: bad shape M=%lld N=%lld K=%lld", what, (long long)M, (long long)N, (long long)K);
    if (K % 32 != 0 || N % 8 != 0)
        CK_FAIL(CK_ERR_SHAPE, "%s: K (%lld) must be a multiple of 32 and N (%lld) a multiple of 8", what, (long long)K, (long long)N);
    if (out_code != CK_F32 && out_code != CK_F16 && out_code != CK_BF16)
        CK_FAIL(CK_ERR_DTYPE, "%s: unsupported output dtype code %d", what, out_code);
    if (bias && bias_code != CK_F32 && bias_code != CK_F16 && bias_code != CK_BF16)
        CK_FAIL(CK_ERR_DTYPE, "%s: unsupported bias dtype code %d", what, bias_code);
    const int64_t row_bytes = kFp4 ? K / 2 : K;
    if (!aligned16(a) || !aligned16(b) || !aligned16(sfa) || !aligned16(sfb) || !aligned16(d) || row_bytes % 16 != 0)
        CK_FAIL(CK_ERR_ALIGN, "%s: operands, scales and output must be 16-byte aligned (row pitch too)", what);

    // Which pipeline: 1 = scale movers, 2 = tcgen05.cp by the MMA issuer (ck_set_option("gemm_tile", ...); 0 = default).
    // Default: the tcgen05.cp pipeline (measured 1-3 % faster for NVFP4, 2-13 % for MXFP8, never slower by more than
    // the run-to-run spread); ck_set_option("gemm_tile", 1) selects the scale movers.  Both pipelines use two
    // MMA-issuing warps whose k-tiles may reach the tensor pipe in either order: NVFP4 results repeat bit for bit in
    // every test, MXFP8 sums can differ in the last fp32 bit from launch to launch with either pipeline.
    const bool use_cp = g_gemm_tile != 1;
    auto kern = use_cp ? gemm_blockscaled_kernel<kFp4, kEpi, true> : gemm_blockscaled_kernel<kFp4, kEpi, false>;
    // per device and variant: shared-memory opt-in, and how many CTA pairs can be resident at once
    static int max_pairs[2][64] = {};   // (one table per instantiation of this function)
    int dev = 0;
    cudaGetDevice(&dev);
    int pairs_cap = (dev >= 0 && dev < 64) ? max_pairs[use_cp][dev] : 0;
    if (pairs_cap == 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) CK_FAIL((int)e, "%s: cannot reserve %d bytes of shared memory: %s", what, kSmemBytes, cudaGetErrorString(e));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * (unsigned)(sm_count() / 2));
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kSmemBytes;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
        if (e != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = sm_count() / 2;
        }
        pairs_cap = n < sm_count() / 2 ? n : sm_count() / 2;
        if (dev >= 0 && dev < 64) max_pairs[use_cp][dev] = pairs_cap;
    }

    CUtensorMap map_a, map_b, map_out;
    if (int rc = cached_map(&map_a, a, M, row_bytes, BM)) return rc;
    if (int rc = cached_map(&map_b, b, N, row_bytes, BN / 2)) return rc;
    if (scatter_world == 0)
        if (int rc = cached_map(&map_out, d, M, N, out_code == CK_F32 ? -4 : -2)) return rc;
    OutMaps omaps;
    if (scatter_world > 0) {
        map_out = map_a;   // (placeholder: the scattered epilogue does not read it)
        for (int i = 0; i < scatter_world; ++i) {
            const int64_t lo = scatter_bounds[i], hi = scatter_bounds[i + 1];
            if (lo < 0 || hi < lo || lo % 128 != 0 || (hi % 128 != 0 && i + 1 < scatter_world) || lo > INT32_MAX || hi > INT32_MAX)
                CK_FAIL(CK_ERR_SHAPE, "%s: scatter bounds must ascend in multiples of 128 rows", what);
            if (!scatter_dests[i] || !aligned16(scatter_dests[i])) CK_FAIL(CK_ERR_ALIGN, "%s: scatter destination %d", what, i);
            omaps.m[i] = map_a;
            if (hi > lo)
                if (int rc = cached_map(&omaps.m[i], scatter_dests[i], hi - lo, N, -2)) return rc;
        }
        for (int i = scatter_world; i < 8; ++i) omaps.m[i] = map_a;
        if (M % 32 != 0) CK_FAIL(CK_ERR_SHAPE, "%s: scattered output needs M (%lld) to be a multiple of 32 rows", what, (long long)M);
        if (scatter_row_offset < 0 || scatter_row_offset % 32 != 0 || scatter_row_offset + M > scatter_bounds[scatter_world])
            CK_FAIL(CK_ERR_SHAPE, "%s: scatter row offset %lld (multiple of 32, rows within the bounds)", what, (long long)scatter_row_offset);
    } else {
        for (int i = 0; i < 8; ++i) omaps.m[i] = map_a;
    }

    GemmParams p{};
    p.sfa = static_cast<const uint8_t*>(sfa);
    p.sfb = static_cast<const uint8_t*>(sfb);
    p.bias = bias;
    p.alpha = alpha;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    const int64_t blk = kFp4 ? 16 : 32;
    p.sf_tiles_k = (int)(round_up(K / blk, 4) / 4);
    p.sf_row_tiles_a = (int)ceil_div(M, 128);
    p.sf_row_tiles_b = (int)ceil_div(N, 128);
    p.out_code = out_code;
    p.bias_code = bias_code;
    p.tiles_m = (int)ceil_div(M, 2 * BM);
    p.tiles_n = (int)ceil_div(N, BN);
    p.residual = residual;
    p.gate = gate;
    omaps.world = scatter_world;
    omaps.row_offset = (int)scatter_row_offset;
    for (int i = 0; i < 9; ++i) omaps.bounds[i] = (scatter_world > 0 && i <= scatter_world) ? (int)scatter_bounds[i] : 0;
    const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
    const int grid = 2 * (int)(tiles < pairs_cap ? tiles : pairs_cap);   // clusters of two CTAs
    CUtensorMap map_sfa = map_a, map_sfb = map_a;   // (placeholders for the mover variant, which does not read them)
    if (use_cp) {
        const int box_tiles = kFp4 ? 4 : 1;
        if (int rc = cached_map(&map_sfa, sfa, p.sf_row_tiles_a, p.sf_tiles_k, 1000 + 10 * box_tiles + 1)) return rc;
        if (int rc = cached_map(&map_sfb, sfb, p.sf_row_tiles_b, p.sf_tiles_k, 1000 + 10 * box_tiles + 2)) return rc;
    }
    kern<<<grid, kThreads, kSmemBytes, stream>>>(map_a, map_b, map_out, map_sfa, map_sfb, omaps, p);
    return launch_status(what);
}

}  // namespace
}  // namespace ck

// D[M,N] = alpha * (A . W^T) + bias, NVFP4 operands.  A: [M, K/2] bytes, W: [N, K/2] bytes,
// scales tiled E4M3, alpha: device fp32 scalar (null = 1), bias: [N] or null.
extern "C" int launch_scaled_mm_nvfp4_kernel(const void* A, const void* A_scale, const void* B, const void* B_scale,
                                             void* D, const void* bias, int bias_dtype_code, int64_t M, int64_t N,
                                             int64_t K, const float* alpha_device_ptr, int out_dtype_code,
                                             cudaStream_t stream) {
    return ck::launch_gemm<true>(A, A_scale, B, B_scale, D, bias, bias_dtype_code, M, N, K, alpha_device_ptr,
                                 out_dtype_code, stream);
}

// launch_scaled_mm_nvfp4_kernel followed by  D = residual + gate[n] * D  (an elementwise addcmul on the stored
// 16-bit tensors), in the GEMM's epilogue.  residual: [M, N] in the output dtype, may be D itself (in place);
// gate: [N] in the output dtype.  No counterpart in the reference.
extern "C" int launch_scaled_mm_nvfp4_residual_kernel(const void* A, const void* A_scale, const void* B, const void* B_scale,
                                                      void* D, const void* bias, int bias_dtype_code, const void* residual,
                                                      const void* gate, int64_t M, int64_t N, int64_t K,
                                                      const float* alpha_device_ptr, int out_dtype_code, cudaStream_t stream) {
    if (!residual || !gate) CK_FAIL(CK_ERR_NULL, "scaled_mm_nvfp4_residual: null residual or gate");
    return ck::launch_gemm<true, 1>(A, A_scale, B, B_scale, D, bias, bias_dtype_code, M, N, K, alpha_device_ptr,
                                       out_dtype_code, stream, residual, gate);
}

// launch_scaled_mm_nvfp4_kernel with the output scattered by rows over the ranks of a tensor-parallel group (the
// reduce-scatter of a row-parallel GEMM fused into its epilogue: each output tile row goes straight into the
// buffer of the rank that will sum it, over NVLink, while the main loop carries on).  Output row r is row
// row_offset + r of the group's [bounds[world], N] matrix; rows [bounds[d], bounds[d+1]) are written to dests[d]
// (a [bounds[d+1] - bounds[d], N] buffer in rank d's memory, mapped into this process), counted from bounds[d].
// dests, bounds: host arrays (world pointers, world + 1 row numbers in multiples of 128 except the last).
// 16-bit outputs.  No counterpart in the reference (it has no multi-GPU code).
extern "C" int launch_scaled_mm_nvfp4_scatter_kernel(const void* A, const void* A_scale, const void* B, const void* B_scale,
                                                     void* const* dests, const int64_t* bounds, int world, int64_t row_offset,
                                                     const void* bias, int bias_dtype_code, int64_t M, int64_t N, int64_t K,
                                                     const float* alpha_device_ptr, int out_dtype_code, cudaStream_t stream) {
    if (world < 1) CK_FAIL(CK_ERR_SHAPE, "scaled_mm_nvfp4_scatter: world must be at least 1");
    return ck::launch_gemm<true, 2>(A, A_scale, B, B_scale, nullptr, bias, bias_dtype_code, M, N, K, alpha_device_ptr,
                                    out_dtype_code, stream, nullptr, nullptr, dests, bounds, world, row_offset);
}

// Same contraction, MXFP8 operands: A: [M, K] E4M3, W: [N, K] E4M3, scales tiled E8M0.
extern "C" int launch_scaled_mm_mxfp8_kernel(const void* A, const void* A_scale, const void* B, const void* B_scale,
                                             void* D, const void* bias, int bias_dtype_code, int64_t M, int64_t N,
                                             int64_t K, int out_dtype_code, cudaStream_t stream) {
    return ck::launch_gemm<false>(A, A_scale, B, B_scale, D, bias, bias_dtype_code, M, N, K, nullptr, out_dtype_code,
                                  stream);
}

// Argument order and meaning of the reference's entry point (weights first; bias has the
// output's dtype; workspace unused; accumulate must be false).
extern "C" int launch_cublas_gemm_blockwise_fp4_kernel(const void* B_ptr, const void* B_decode_scale_ptr,
                                                       const void* A_ptr, const void* A_decode_scale_ptr, void* D_ptr,
                                                       const void* bias_ptr, int64_t M, int64_t N, int64_t K,
                                                       const float* alpha_device_ptr, int out_dtype_code,
                                                       void* workspace_ptr, bool accumulate, cudaStream_t stream) {
    (void)workspace_ptr;
    if (accumulate) CK_FAIL(CK_ERR_UNSUPPORTED, "cublas_gemm_blockwise_fp4: accumulate=true is not supported");
    return ck::launch_gemm<true>(A_ptr, A_decode_scale_ptr, B_ptr, B_decode_scale_ptr, D_ptr, bias_ptr, out_dtype_code,
                                 M, N, K, alpha_device_ptr, out_dtype_code, stream);
}


// Reads and clears the device-side status word of the GEMM kernels (synchronises the device).
// 0 = no bounded wait ran out since the last call, CK_ERR_DEVICE_TIMEOUT otherwise.
extern "C" int ck_gemm_device_status(void) {
    int v = 0, zero = 0;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) CK_FAIL((int)e, "gemm status: %s", cudaGetErrorString(e));
    e = cudaMemcpyFromSymbol(&v, ck::g_gemm_status, sizeof(int));
    if (e != cudaSuccess) CK_FAIL((int)e, "gemm status: %s", cudaGetErrorString(e));
    cudaMemcpyToSymbol(ck::g_gemm_status, &zero, sizeof(int));
    if (v != 0) CK_FAIL(CK_ERR_DEVICE_TIMEOUT, "gemm kernel: bounded wait %d ran out in CTA %d", v >> 16, v & 0xffff);
    return CK_OK;
}
