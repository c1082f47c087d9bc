// Library-level entry points of the C ABI: error text, version, device check.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "ck_common.cuh"

namespace ck {
namespace {
thread_local char g_error[512] = "";
}

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}
}  // namespace ck

extern "C" const char* ck_last_error(void) { return ck::g_error; }

extern "C" int ck_abi_version(void) { return 1; }

namespace ck {
int g_nvfp4_exact_div = 0, g_norm_warps = 0, g_norm_cache = -1, g_norm_group = 0, g_norm_poll_limit = 0;
int g_rope_threads_per_sm = 0, g_gelu_table_min = 8 << 20, g_gemm_tile = 0, g_gemm_map_cache = 1, g_tp_bulk = 0, g_qk_heads_per_warp = 0;
}

// Library options: the public one is described in the C header, the tuning knobs in ck_options.h.
extern "C" int ck_set_option(const char* name, int value) {
    static const struct { const char* name; int* slot; } table[] = {
        {"norm_warps", &ck::g_norm_warps},   {"norm_cache", &ck::g_norm_cache},
        {"norm_group", &ck::g_norm_group},   {"norm_poll_limit", &ck::g_norm_poll_limit},
        {"rope_threads_per_sm", &ck::g_rope_threads_per_sm}, {"gelu_table_min", &ck::g_gelu_table_min},
        {"gemm_tile", &ck::g_gemm_tile},     {"gemm_map_cache", &ck::g_gemm_map_cache},
        {"tp_bulk", &ck::g_tp_bulk},         {"qk_heads_per_warp", &ck::g_qk_heads_per_warp},
    };
    if (name && !strcmp(name, "nvfp4_exact_div")) { ck::g_nvfp4_exact_div = value ? 1 : 0; return CK_OK; }
    if (name)
        for (const auto& t : table)
            if (!strcmp(name, t.name)) { *t.slot = value; return CK_OK; }
    CK_FAIL(CK_ERR_UNSUPPORTED, "ck_set_option: unknown option '%s'", name ? name : "(null)");
}

// 0 when the current device can run this library (compute capability 10.x), else a status.
extern "C" int ck_check_device(void) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) CK_FAIL((int)e, "cudaGetDevice: %s", cudaGetErrorString(e));
    int major = 0, minor = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (major != 10) CK_FAIL(CK_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", dev, major, minor);
    return CK_OK;
}
