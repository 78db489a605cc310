// Error channel shared by all entry points (see common.cuh).
#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>

static thread_local char g_error[512] = "";

void gi_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int gi_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        gi_set_error("%s: %s", what, cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

extern "C" const char* gi_last_error(void) { return g_error; }

#include <stdlib.h>
#include <string.h>
// GARLIC_B200_PDL=0 or =1 in the environment decides for the whole process; otherwise the caller's last
// gi_set_pdl() does (off until then).
static int g_pdl_requested = 0;
bool gi_pdl_enabled() {
    static int from_env = -2;
    if (from_env == -2) {
        const char* v = getenv("GARLIC_B200_PDL");
        from_env = (v && strcmp(v, "1") == 0) ? 1 : (v && strcmp(v, "0") == 0) ? 0 : -1;
    }
    return from_env >= 0 ? from_env == 1 : g_pdl_requested == 1;
}
extern "C" void gi_set_pdl(int on) { g_pdl_requested = on ? 1 : 0; }

// Compute capability of the current device as major*10+minor, or a negative CUDA error.
extern "C" int gi_device_arch(void) {
    int dev = 0, major = 0, minor = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (e != cudaSuccess) {
        gi_set_error("gi_device_arch: %s", cudaGetErrorString(e));
        return -(int)e;
    }
    return major * 10 + minor;
}

#include <mutex>
#include <vector>
namespace {
struct SmemRecord { const void* kernel; int device; size_t bytes; };
std::mutex g_smem_mutex;
std::vector<SmemRecord> g_smem_done;
}
int gi_reserve_smem(const void* kernel, size_t bytes, const char* who) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { gi_set_error("%s: %s", who, cudaGetErrorString(e)); return (int)e; }
    std::lock_guard<std::mutex> lock(g_smem_mutex);
    for (const SmemRecord& r : g_smem_done)
        if (r.kernel == kernel && r.device == dev && r.bytes >= bytes) return 0;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) {
        gi_set_error("%s: cannot reserve %zu bytes of shared memory: %s", who, bytes, cudaGetErrorString(e));
        return (int)e;
    }
    g_smem_done.push_back({kernel, dev, bytes});
    return 0;
}
