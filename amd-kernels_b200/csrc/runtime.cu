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
struct StreamScratch {
    cudaStream_t stream = nullptr;
    bool used = false;
    uint64_t last_use = 0;
    void* block[SCRATCH_SLOTS] = {};
    size_t bytes[SCRATCH_SLOTS] = {};
};
struct DeviceState {
    int sms = 0;
    StreamScratch scratch[kScratchStreams];
    uint64_t clock = 0;
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

int scratch_get(ScratchSlot slot, cudaStream_t stream, size_t bytes, void** out) {
    int dev = 0;
    int rc = current_device(&dev);
    if (rc != HKB_OK) return rc;
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& d = g_dev[dev];
    // the entry of this stream, else a free one, else the least recently used one
    StreamScratch* e = nullptr;
    for (auto& c : d.scratch)
        if (c.used && c.stream == stream) { e = &c; break; }
    if (!e)
        for (auto& c : d.scratch)
            if (!c.used) { e = &c; break; }
    if (!e) {
        e = &d.scratch[0];
        for (auto& c : d.scratch)
            if (c.last_use < e->last_use) e = &c;
        // Another stream's launches may still read these blocks: cudaFree waits for the device.
        for (int i = 0; i < SCRATCH_SLOTS; ++i) {
            if (e->block[i]) HKB_CUDA(cudaFree(e->block[i]));
            e->block[i] = nullptr;
            e->bytes[i] = 0;
        }
    }
    e->used = true;
    e->stream = stream;
    e->last_use = ++d.clock;
    if (e->bytes[slot] < bytes) {
        // Growing frees the old block; earlier launches that still use it are ordered before
        // the free by the implicit synchronisation of cudaFree.
        if (e->block[slot]) HKB_CUDA(cudaFree(e->block[slot]));
        e->block[slot] = nullptr;
        e->bytes[slot] = 0;
        size_t want = (bytes + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
        HKB_CUDA(cudaMalloc(&e->block[slot], want));
        e->bytes[slot] = want;
    }
    *out = e->block[slot];
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

static thread_local const char* g_last_kernel = "";
void note_kernel(const char* name) { g_last_kernel = name; }

}  // namespace hkb

extern "C" {

int hkb_version(void) { return 200; }

const char* hkb_last_kernel(void) { return hkb::g_last_kernel; }

const char* hkb_last_error(void) { return hkb::g_err.c_str(); }

int hkb_shard_bounds(int64_t N, int64_t world_size, int64_t rank, int64_t* n0, int64_t* n1) {
    using namespace hkb;
    HKB_REQUIRE(n0 && n1, HKB_ERR_BAD_ARG, "shard_bounds: null pointer");
    HKB_REQUIRE(N > 0 && N % 128 == 0, HKB_ERR_BAD_SHAPE, "shard_bounds: N=%lld must be a positive multiple of 128", (long long)N);
    HKB_REQUIRE(world_size >= 1 && rank >= 0 && rank < world_size, HKB_ERR_BAD_ARG, "shard_bounds: rank %lld outside a world of %lld",
                (long long)rank, (long long)world_size);
    const int64_t blocks = N / 128, base = blocks / world_size, extra = blocks % world_size;
    const int64_t b0 = rank * base + (rank < extra ? rank : extra);
    *n0 = b0 * 128;
    *n1 = (b0 + base + (rank < extra ? 1 : 0)) * 128;
    return HKB_OK;
}

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
        for (auto& c : s.scratch) any = any || c.used;
        if (!any) continue;
        HKB_CUDA(cudaSetDevice(d));
        for (auto& c : s.scratch) {
            for (int i = 0; i < SCRATCH_SLOTS; ++i)
                if (c.block[i]) HKB_CUDA(cudaFree(c.block[i]));
            c = StreamScratch{};
        }
        if (s.status) HKB_CUDA(cudaFree(s.status));
        s.status = nullptr;
    }
    HKB_CUDA(cudaSetDevice(prev));
    return HKB_OK;
}

int hkb_check_status(void* stream) {
    using namespace hkb;
    // Two words can hold a failure: the allocated one of the ordinary entry points and the one built
    // into the library image that the allocation-free entry point uses.  Neither is created here:
    // a word that no launch has used yet cannot hold anything.
    int dev = 0;
    int rc = current_device(&dev);
    if (rc != HKB_OK) return rc;
    uint32_t* words[2];
    {
        std::lock_guard<std::mutex> lk(g_mu);
        words[0] = g_dev[dev].status;
    }
    words[1] = static_status_peek();
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t host[2] = {0, 0};
    for (int i = 0; i < 2; ++i)
        if (words[i]) HKB_CUDA(cudaMemcpyAsync(&host[i], words[i], sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    HKB_CUDA(cudaStreamSynchronize(st));
    if (host[0] | host[1]) {
        for (int i = 0; i < 2; ++i)
            if (host[i]) cudaMemsetAsync(words[i], 0, sizeof(uint32_t), st);
        return set_error(HKB_ERR_TIMEOUT, "a kernel abandoned a bounded wait (status 0x%08x%s)", host[0] | host[1],
                         host[1] ? ", allocation-free entry point" : "");
    }
    return HKB_OK;
}

}  // extern "C"
