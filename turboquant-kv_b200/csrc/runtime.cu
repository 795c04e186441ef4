// runtime.cu -- process-wide state of libtqb200: last-error text, launch counter, device facts.
#include "common.cuh"

namespace tqb {

std::atomic<int64_t> g_launches{0};

char* last_error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

int sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace tqb

extern "C" {

int tqb_abi_version(void) { return 2; }

const char* tqb_last_error(void) { return tqb::last_error_buffer(); }

int64_t tqb_launch_count(void) { return tqb::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
