// Per-device runtime state shared by the kernels: the status word and cached device properties.
#include "neox_b200.h"
#include <mutex>

namespace {
constexpr int MAX_DEV = 64;
int* g_status[MAX_DEV] = {nullptr};
int g_sms[MAX_DEV] = {0};
std::mutex g_mu;
}  // namespace

int* neox_status_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return nullptr;
    std::lock_guard<std::mutex> g(g_mu);
    if (!g_status[dev]) {
        int* p = nullptr;
        if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
        cudaMemset(p, 0, 256);
        g_status[dev] = p;
    }
    return g_status[dev];
}

int neox_sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return 1;
    if (!g_sms[dev]) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        g_sms[dev] = n > 0 ? n : 1;
    }
    return g_sms[dev];
}

extern "C" int neox_read_status() {
    int* p = neox_status_word();
    if (!p) return -1;
    int v = 0;
    if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
    if (v) cudaMemset(p, 0, sizeof(int));
    return v;
}

extern "C" int neox_sm_count_c() { return neox_sm_count(); }
