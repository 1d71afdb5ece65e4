// Error reporting, device status word and device properties for the C ABI.
#include "common.cuh"

#include <mutex>
#include <vector>

namespace dq {

std::string& last_error() {
    static thread_local std::string msg;
    return msg;
}

int fail(int code, const char* file, int line, const char* cond, const char* fmt, ...) {
    // Same text as the reference's throwCheckError (csrc/util.h:143-152).
    char head[1024];
    const char* base = file;
    for (const char* p = file; *p; ++p)
        if (*p == '/') base = p + 1;
    snprintf(head, sizeof(head), "[ASSERT FAILED] %s:%d  Condition: %s", base, line, cond);
    std::string msg(head);
    if (fmt != nullptr && fmt[0] != '\0') {
        char info[1024];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(info, sizeof(info), fmt, ap);
        va_end(ap);
        msg += "  Info: ";
        msg += info;
    }
    last_error() = msg;
    return code;
}

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_mu;
int* g_status_host[kMaxDevices] = {nullptr};
int* g_status_dev[kMaxDevices] = {nullptr};
int g_sm_count[kMaxDevices] = {0};
}  // namespace

static bool ensure_status(int dev) {
    if (g_status_host[dev] != nullptr) return true;
    int* h = nullptr;
    // Pinned, mapped host memory: no device allocation is made by this library.
    if (cudaHostAlloc(reinterpret_cast<void**>(&h), 64, cudaHostAllocMapped) != cudaSuccess) return false;
    *h = 0;
    int* d = nullptr;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&d), h, 0) != cudaSuccess) return false;
    g_status_host[dev] = h;
    g_status_dev[dev] = d;
    return true;
}

int* device_status_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        fail(DQMOE_ERR_CUDA, __FILE__, __LINE__, "cudaGetDevice", "no current CUDA device");
        return nullptr;
    }
    std::lock_guard<std::mutex> lk(g_mu);
    if (!ensure_status(dev)) {
        fail(DQMOE_ERR_CUDA, __FILE__, __LINE__, "cudaHostAlloc", "cannot map the device status word");
        return nullptr;
    }
    return g_status_dev[dev];
}

volatile int* host_status_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!ensure_status(dev)) return nullptr;
    return g_status_host[dev];
}

int sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    if (g_sm_count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        g_sm_count[dev] = n;
    }
    return g_sm_count[dev];
}

}  // namespace dq

extern "C" {

const char* dqmoe_last_error(void) { return dq::last_error().c_str(); }

int dqmoe_abi_version(void) { return DQMOE_ABI_VERSION; }

int dqmoe_device_status(int* code) {
    DQ_CHECK(code != nullptr);
    volatile int* h = dq::host_status_word();
    if (h == nullptr) return dq::fail(DQMOE_ERR_CUDA, __FILE__, __LINE__, "host_status_word", "no status word");
    DQ_CUDA(cudaDeviceSynchronize());
    *code = *h;
    *h = 0;
    return DQMOE_OK;
}

}  // extern "C"
