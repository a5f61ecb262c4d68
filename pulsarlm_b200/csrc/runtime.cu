// Error reporting and version of the kernel library.
#include "common.cuh"

#include <cstdarg>

namespace {
thread_local char last_error[1024] = "";
int overlap_enabled = 1;
}

int pl_overlap_enabled() { return overlap_enabled; }

// Switches programmatic dependent launch of the library's kernels on (default) or
// off; returns the previous setting.
PL_API int pl_set_overlap(int enabled) {
    const int before = overlap_enabled;
    overlap_enabled = enabled != 0;
    return before;
}

int pl_fail(int code, const char* format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(last_error, sizeof(last_error), format, args);
    va_end(args);
    return code;
}

PL_API const char* pl_last_error() { return last_error; }

// Bumped when an entry point's signature changes; the Python side checks it so a
// stale build is rebuilt instead of being called with the wrong arguments.
PL_API int pl_abi_version() { return 21; }

// Compute capability of the current device as major * 10 + minor, or -1.
PL_API int pl_device_arch() {
    int device = 0, major = 0, minor = 0;
    if (cudaGetDevice(&device) != cudaSuccess) {
        return -1;
    }
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess ||
        cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device) != cudaSuccess) {
        return -1;
    }
    return major * 10 + minor;
}
