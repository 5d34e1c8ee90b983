// Library runtime of libhkb200: error messages, per-device scratch and status word.
#include "common.cuh"

#include <mutex>
#include <string>

namespace hkb {

static thread_local std::string g_err;

int set_error(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}

namespace {
constexpr int kMaxDev = 64;
struct DeviceState {
    int sms = 0;
    void* scratch[SCRATCH_SLOTS] = {};
    size_t scratch_bytes[SCRATCH_SLOTS] = {};
    uint32_t* status = nullptr;
};
DeviceState g_dev[kMaxDev];
std::mutex g_mu;

int current_device(int* dev) {
    HKB_CUDA(cudaGetDevice(dev));
    HKB_REQUIRE(*dev >= 0 && *dev < kMaxDev, HKB_ERR_CUDA, "device index %d out of range", *dev);
    return HKB_OK;
}
}  // namespace

int sm_count() {
    int dev = 0;
    if (current_device(&dev) != HKB_OK) return 0;
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_dev[dev].sms == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        g_dev[dev].sms = n;
    }
    return g_dev[dev].sms;
}

int scratch_get(ScratchSlot slot, size_t bytes, void** out) {
    int dev = 0;
    int rc = current_device(&dev);
    if (rc != HKB_OK) return rc;
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& d = g_dev[dev];
    if (d.scratch_bytes[slot] < bytes) {
        // Growing frees the old block; earlier launches that still use it are ordered before
        // the free by the implicit synchronisation of cudaFree.
        if (d.scratch[slot]) HKB_CUDA(cudaFree(d.scratch[slot]));
        d.scratch[slot] = nullptr;
        d.scratch_bytes[slot] = 0;
        size_t want = (bytes + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
        HKB_CUDA(cudaMalloc(&d.scratch[slot], want));
        d.scratch_bytes[slot] = want;
    }
    *out = d.scratch[slot];
    return HKB_OK;
}

int status_word(uint32_t** out) {
    int dev = 0;
    int rc = current_device(&dev);
    if (rc != HKB_OK) return rc;
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& d = g_dev[dev];
    if (!d.status) {
        HKB_CUDA(cudaMalloc(&d.status, 256));
        HKB_CUDA(cudaMemset(d.status, 0, 256));
    }
    *out = d.status;
    return HKB_OK;
}

}  // namespace hkb

extern "C" {

int hkb_version(void) { return 100; }

const char* hkb_last_error(void) { return hkb::g_err.c_str(); }

int hkb_release(void) {
    using namespace hkb;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess) {
        cudaGetLastError();
        return HKB_OK;  // nothing can have been allocated without a device
    }
    int prev = 0;
    HKB_CUDA(cudaGetDevice(&prev));
    std::lock_guard<std::mutex> lk(g_mu);
    for (int d = 0; d < ndev && d < kMaxDev; ++d) {
        DeviceState& s = g_dev[d];
        bool any = s.status != nullptr;
        for (int i = 0; i < SCRATCH_SLOTS; ++i) any = any || s.scratch[i];
        if (!any) continue;
        HKB_CUDA(cudaSetDevice(d));
        for (int i = 0; i < SCRATCH_SLOTS; ++i) {
            if (s.scratch[i]) HKB_CUDA(cudaFree(s.scratch[i]));
            s.scratch[i] = nullptr;
            s.scratch_bytes[i] = 0;
        }
        if (s.status) HKB_CUDA(cudaFree(s.status));
        s.status = nullptr;
    }
    HKB_CUDA(cudaSetDevice(prev));
    return HKB_OK;
}

int hkb_check_status(void* stream) {
    using namespace hkb;
    uint32_t* w = nullptr;
    int rc = status_word(&w);
    if (rc != HKB_OK) return rc;
    uint32_t host = 0;
    HKB_CUDA(cudaMemcpyAsync(&host, w, sizeof host, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    HKB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (host != 0) {
        cudaMemsetAsync(w, 0, sizeof host, (cudaStream_t)stream);
        return set_error(HKB_ERR_TIMEOUT, "a kernel abandoned a bounded wait (status 0x%08x)", host);
    }
    return HKB_OK;
}

}  // extern "C"
