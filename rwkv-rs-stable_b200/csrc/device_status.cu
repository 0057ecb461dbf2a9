// Per-device status word that kernels set instead of trapping (expired bounded
// wait, out-of-range index), and the cached device properties the launchers use.
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>

#include "kernels.h"

namespace rwkv7 {

__device__ int g_device_status_word = 0;

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_mu;
int *g_status_ptr[kMaxDevices] = {};
std::atomic<int64_t> g_launches{0};
}  // namespace

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }

// The symbol's address differs per device and must be resolved with that device
// current; callers hold a DeviceGuard.
int device_status_ptr(int device, int **out) {
    if (device < 0 || device >= kMaxDevices) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_status_ptr[device] == nullptr) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_device_status_word);
        if (e != cudaSuccess) return (int)e;
        g_status_ptr[device] = static_cast<int *>(p);
    }
    *out = g_status_ptr[device];
    return 0;
}

}  // namespace rwkv7
