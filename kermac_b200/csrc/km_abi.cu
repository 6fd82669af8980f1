// Error reporting, version queries and device checks of the kermac_b200 C-ABI.
#include <cstring>
#include <mutex>

#include "km_host.h"

namespace km {

static thread_local char g_last_error[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_status(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return 0;
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
    return static_cast<int>(e);
}

namespace {
struct DeviceInfo {
    int known = 0;
    int major = 0;
    int sms   = 0;
};
DeviceInfo g_devices[64];
std::mutex g_device_mutex;

const DeviceInfo* current_device_info() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_device_mutex);
    DeviceInfo& d = g_devices[dev];
    if (!d.known) {
        if (cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return nullptr;
        if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
        d.known = 1;
    }
    return &d;
}
}  // namespace

int require_sm100() {
    const DeviceInfo* d = current_device_info();
    if (!d) return fail(KM_ERR_NOT_SM100, "no usable CUDA device is current");
    if (d->major != 10)
        return fail(KM_ERR_NOT_SM100, "kermac_b200 kernels are built for sm_100a only; current device is sm_%d", d->major * 10);
    return 0;
}

int sm_count() {
    const DeviceInfo* d = current_device_info();
    return d ? d->sms : 148;
}

}  // namespace km

extern "C" {

const char* kermac_b200_last_error(void) { return km::g_last_error; }

int kermac_b200_copy_2d_async(void* dst, int64_t dst_pitch_bytes, const void* src, int64_t src_pitch_bytes,
                              int64_t row_bytes, int64_t rows, int32_t direction, void* stream) {
    using namespace km;
    if (row_bytes < 0 || rows < 0) return fail(KM_ERR_BAD_SHAPE, "row_bytes and rows must be >= 0");
    if (row_bytes == 0 || rows == 0) return 0;
    if (!dst || !src) return fail(KM_ERR_NULL_POINTER, "dst and src must not be NULL");
    if (dst_pitch_bytes < row_bytes || src_pitch_bytes < row_bytes)
        return fail(KM_ERR_BAD_STRIDE, "a pitch is smaller than the row it spans");
    if (direction != 0 && direction != 1) return fail(KM_ERR_BAD_ENUM, "direction must be 0 (to device) or 1 (to host)");
    return cuda_status(cudaMemcpy2DAsync(dst, (size_t)dst_pitch_bytes, src, (size_t)src_pitch_bytes, (size_t)row_bytes,
                                         (size_t)rows, direction == 0 ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost,
                                         static_cast<cudaStream_t>(stream)),
                       "cudaMemcpy2DAsync");
}

int kermac_b200_abi_version(void) { return KERMAC_B200_ABI_VERSION; }

#define KM_STR2(x) #x
#define KM_STR(x) KM_STR2(x)
const char* kermac_b200_build_id(void) {
    return "kermac_b200 abi " KM_STR(KERMAC_B200_ABI_VERSION) " sm_100a " __DATE__ " " __TIME__;
}

}  // extern "C"
