#include "common.cuh"

#include <mutex>

namespace macko {

char *last_error_buffer()
{
    static thread_local char buf[512] = "";
    return buf;
}

int fail(int status, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buffer(), 512, fmt, ap);
    va_end(ap);
    return status;
}

int current_device_info(const DeviceInfo **out)
{
    static DeviceInfo infos[kMaxDevices];
    static std::mutex mu;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(MACKO_ERR_CUDA, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    DeviceInfo &d = infos[dev];
    if (!d.valid) {
        e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
        d.valid = true;
    }
    *out = &d;
    return MACKO_OK;
}

}  // namespace macko

extern "C" {

int macko_version(void) { return MACKO_B200_VERSION; }

const char *macko_status_string(int status)
{
    switch (status) {
        case MACKO_OK: return "ok";
        case MACKO_ERR_INVALID_ARGUMENT: return "invalid argument";
        case MACKO_ERR_MISALIGNED: return "misaligned buffer";
        case MACKO_ERR_SIZE_OVERFLOW: return "size overflow";
        case MACKO_ERR_CUDA: return "CUDA error";
        case MACKO_ERR_WORKSPACE: return "workspace too small";
        default: return "unknown status";
    }
}

const char *macko_last_error(void) { return macko::last_error_buffer(); }
}
