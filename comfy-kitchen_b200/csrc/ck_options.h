// Names accepted by ck_set_option() beyond the public "nvfp4_exact_div" (see
// include/comfy_kitchen_b200.h).  These are the launchers' tuning knobs and one test hook; they are
// process-wide ints read at launch time.
//
//   "norm_warps"          n > 0 forces the warps per CTA of the norm kernels (0: the launcher chooses)
//   "norm_cache"          0 keeps the norm kernels from caching the modulation rows in shared
//                         memory (-1: the launcher chooses)
//   "norm_group"          1, 2 or 4 warps share a row (0: the launcher chooses); more than one changes
//                         the summation order of the row statistics, so a result may move by one
//                         rounding step of the output type, while the fused outputs stay equal to
//                         "norm kernel -> quantizer"
//   "norm_poll_limit"     polls of a row copy's mbarrier before a norm kernel's consumer gives the row
//                         up and records a time-out (0: default, 2^22).  The warp still waits with the
//                         default limit for its outstanding copies before it leaves.  Test hook: a
//                         negative value means no poll at all, so the time-out path runs on every
//                         row, deterministically and without any fault.
//   "rope_threads_per_sm" n > 0: threads per SM the RoPE launcher aims for when it splits the walk
//                         over the broadcast dimension (0: default)
//   "qk_heads_per_warp"   n > 0: heads of a token that one warp of the QK-norm + RoPE kernel walks (0: default, one)
//   "gelu_table_min"      the gather quantizer tabulates GELU per CTA from n activated elements on
//                         (default 8 Mi; negative: never; same bytes either way)
//   "gemm_tile"           GEMM pipeline: 0 or 2 = scales moved by tcgen05.cp (default); 1 = scale-mover warps; 2 = tcgen05.cp from
//                         the MMA issuer, copies of both CTAs signalling the leader's barrier.  Same MMAs either way;
//                         with either one MXFP8 sums can differ in the last fp32 bit between launches (two issuing
//                         warps), NVFP4 results repeat bit for bit
//   "gemm_map_cache"      0 disables the cache of encoded tensor maps (1: default)
//   "tp_bulk"             1: launch_tp_reduce_rows_kernel pulls the peers' rows with bulk copies through shared memory
//                         (0: 16-byte peer loads from every thread)
#pragma once

namespace ck {
extern int g_nvfp4_exact_div;
extern int g_norm_warps;
extern int g_norm_cache;
extern int g_norm_group;
extern int g_norm_poll_limit;
extern int g_rope_threads_per_sm;
extern int g_gelu_table_min;
extern int g_gemm_tile;
extern int g_gemm_map_cache;
extern int g_tp_bulk;
extern int g_qk_heads_per_warp;
}  // namespace ck
