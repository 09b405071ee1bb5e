// Library-level state: per-thread error text, per-device status words, SM count.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace b200 {

namespace {
thread_local char g_last_error[512] = "";

constexpr int kMaxDevices = 64;
std::mutex g_mu;
int* g_status_words[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};
}  // namespace

namespace {
thread_local bool g_pdl = false;
}
namespace {
thread_local uint64_t g_launches = 0;
}
uint64_t kernel_launch_count() { return g_launches; }
void note_kernel_launch() { ++g_launches; }
bool pdl_launches_enabled() { return g_pdl; }
void set_pdl_launches(bool on) { g_pdl = on; }

void set_last_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

int* device_status_words(int* err) {
    *err = B200_OK;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_last_error("cudaGetDevice failed or device index out of range");
        *err = B200_ERR_CUDA;
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_status_words[dev]) {
        int* p = nullptr;
        if (cudaMalloc(&p, 16 * sizeof(int)) != cudaSuccess ||
            cudaMemset(p, 0, 16 * sizeof(int)) != cudaSuccess) {
            set_last_error("allocating the device status words failed: %s",
                           cudaGetErrorString(cudaGetLastError()));
            *err = B200_ERR_CUDA;
            return nullptr;
        }
        g_status_words[dev] = p;
    }
    return g_status_words[dev];
}

int sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    if (g_sm_count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        g_sm_count[dev] = n;
    }
    return g_sm_count[dev];
}

}  // namespace b200

extern "C" {

const char* b200_last_error(void) { return b200::g_last_error; }

int b200_abi_version(void) { return 1; }

int b200_read_device_status(int32_t out[2], b200_stream_t stream) {
    B200_CHECK_ARG(out != nullptr, "out must not be NULL");
    int err = B200_OK;
    int* words = b200::device_status_words(&err);
    if (err != B200_OK) return err;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    B200_CHECK_CUDA(cudaStreamSynchronize(s));
    int host[2] = {0, 0};
    B200_CHECK_CUDA(cudaMemcpy(host, words, sizeof(host), cudaMemcpyDeviceToHost));
    out[0] = host[0];
    out[1] = host[1];
    if (host[0] != 0 || host[1] != 0) B200_CHECK_CUDA(cudaMemset(words, 0, sizeof(host)));
    return B200_OK;
}

}  // extern "C"
