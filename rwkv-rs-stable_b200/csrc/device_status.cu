// Per-device status word that kernels set instead of trapping (expired bounded
// wait, out-of-range index), and the cached device properties the launchers use.
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>

#include "kernels.h"
#include "sm100_umma.cuh"

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

// Exercises the error path every kernel in this library takes when a bounded wait expires:
// one thread waits, for at most `max_polls` polls, on an mbarrier that nothing will ever arrive
// on, then records the time-out in the status word and returns.  The wait cannot hang (it is
// the same bounded loop the kernels use) and nothing faults; the context stays usable.
__global__ void bounded_wait_selftest_kernel(int *status, unsigned max_polls) {
    __shared__ __align__(8) uint64_t bar;
    sm100::mbar_init(&bar, 1);
    sm100::mbar_fence_init();
    if (!sm100::mbar_wait(&bar, 0, max_polls)) atomicExch(status, (int)kDevTimeout);
}

int launch_bounded_wait_selftest(int device, unsigned max_polls, cudaStream_t stream) {
    int *status = nullptr;
    if (int e = device_status_ptr(device, &status)) return e;
    bounded_wait_selftest_kernel<<<1, 1, 0, stream>>>(status, max_polls);
    count_launch();
    return (int)cudaGetLastError();
}

}  // namespace rwkv7
