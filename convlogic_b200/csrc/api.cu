// Library-wide entry points: version, status text, last CUDA error of the calling thread.
#include "clb_common.cuh"

#include <atomic>

static thread_local int g_last_cuda_error = 0;
static std::atomic<long long> g_launches{0};
namespace clb_host {
void set_last_cuda_error(int e) { g_last_cuda_error = e; }
void count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
} // namespace clb_host

extern "C" long long clb_kernel_launches(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int clb_version(void) { return 100; }

extern "C" int clb_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" const char *clb_status_string(int status)
{
    switch (status) {
    case CLB_OK: return "ok";
    case CLB_ERR_ARG: return "invalid argument (null pointer, bad enum value or negative size)";
    case CLB_ERR_SHAPE: return "shape is inconsistent or outside what the kernels support";
    case CLB_ERR_LAUNCH: return "CUDA launch failed";
    case CLB_ERR_SCRATCH: return "scratch buffer missing or too small";
    case CLB_ERR_ODD_OUTPUT:
        return "Output height and width after convolution must be divisible by 2 for 2x2 max pooling";
    case CLB_ERR_TOO_LARGE: return "size exceeds a fixed maximum of this entry point";
    default: return "unknown status";
    }
}
