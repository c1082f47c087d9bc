// Library-level entry points of the C ABI: error text, version, device check.
#include <cstdarg>
#include <cstdio>

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
