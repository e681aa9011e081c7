// Status plumbing and device queries behind the C ABI.
#include <mutex>

#include "common.cuh"

namespace tb200 {

namespace {
thread_local cudaError_t g_last_cuda = cudaSuccess;
}

int cuda_failed(cudaError_t e) {
    g_last_cuda = e;
    // Leave the runtime's sticky "last error" clear so that one failed launch
    // configuration does not poison the caller's later cudaGetLastError().
    cudaGetLastError();
    return TB200_ERR_CUDA;
}

int current_device(DeviceInfo *out) {
    static std::mutex lock;
    static DeviceInfo known[64];
    int dev = 0;
    TB200_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return TB200_ERR_DEVICE;
    std::lock_guard<std::mutex> hold(lock);
    DeviceInfo &d = known[dev];
    if (d.device != dev) {
        int sms = 0, major = 0, minor = 0, smem = 0;
        TB200_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        TB200_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        TB200_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
        TB200_CUDA(cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        d.sms = sms;
        d.cc_major = major;
        d.cc_minor = minor;
        d.smem_optin = static_cast<size_t>(smem);
        d.device = dev;
    }
    *out = d;
    return d.cc_major == 10 ? TB200_OK : TB200_ERR_DEVICE;
}

}  // namespace tb200

extern "C" int tb200_version(void) { return 100; }

extern "C" const char *tb200_strerror(int status) {
    switch (status) {
        case TB200_OK: return "ok";
        case TB200_ERR_NULL: return "a required pointer is null";
        case TB200_ERR_SHAPE: return "an extent or stride is out of range";
        case TB200_ERR_DTYPE: return "unknown or unsupported element type";
        case TB200_ERR_ALIGN: return "a pointer is not aligned to its element type";
        case TB200_ERR_WORKSPACE: return "workspace missing, too small or not 16-byte aligned";
        case TB200_ERR_CUDA: return "a CUDA call failed (see tb200_last_cuda_error)";
        case TB200_ERR_UNSUPPORTED: return "no kernel for this request";
        case TB200_ERR_DEVICE: return "the current device is not compute capability 10.x";
        default: return "unknown status";
    }
}

extern "C" const char *tb200_last_cuda_error(void) { return cudaGetErrorString(tb200::g_last_cuda); }

extern "C" int tb200_sm_count(void) {
    tb200::DeviceInfo d;
    int st = tb200::current_device(&d);
    return st == TB200_OK ? d.sms : st;
}

// The tensor-core kernel families and the row kernels fed through shared memory each keep one error word; a caller that launches several kinds
// polls them all at a synchronisation point through this one call.
extern "C" int tb200_device_errors(void) {
    const int product = tb200_device_error();
    if (product < 0) return product;
    const int forward = tb200_attention_device_error();
    if (forward < 0) return forward;
    const int backward = tb200_attention_bwd_device_error();
    if (backward < 0) return backward;
    const int rows = tb200_rows_device_error();
    if (rows < 0) return rows;
    const int scans = tb200_deltanet_device_error();
    if (scans < 0) return scans;
    return (product & 0xff) | ((forward & 0xff) << 8) | ((backward & 0xff) << 16) | ((rows & 0xf) << 24) | ((scans & 0x7) << 28);
}
