// Library-wide entry points: version, status text, last CUDA error of the calling thread.
#include "clb_common.cuh"

#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

static thread_local int g_last_cuda_error = 0;
static std::atomic<long long> g_launches{0};
namespace clb_host {
void set_last_cuda_error(int e) { g_last_cuda_error = e; }
void count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
} // namespace clb_host

// ---- launch tracing: CUDA events around the launches that CLB_TRACED marks -------------------------
namespace {
struct TraceRec {
    const char *name;
    cudaEvent_t e0, e1;
};
std::atomic<int> g_trace_on{0};
std::mutex g_trace_mutex;
std::vector<TraceRec> g_trace;
void trace_drop_locked()
{
    for (TraceRec &r : g_trace) {
        if (r.e0) cudaEventDestroy(r.e0);
        if (r.e1) cudaEventDestroy(r.e1);
    }
    g_trace.clear();
}
} // namespace

namespace clb_host {
bool trace_enabled() { return g_trace_on.load(std::memory_order_relaxed) != 0; }
int trace_begin(const char *name, cudaStream_t st)
{
    TraceRec r{name, nullptr, nullptr};
    if (cudaEventCreate(&r.e0) != cudaSuccess || cudaEventCreate(&r.e1) != cudaSuccess) {
        cudaGetLastError();
        if (r.e0) cudaEventDestroy(r.e0);
        return -1;
    }
    cudaEventRecord(r.e0, st);
    std::lock_guard<std::mutex> lock(g_trace_mutex);
    g_trace.push_back(r);
    return (int)g_trace.size() - 1;
}
void trace_end(int slot, cudaStream_t st)
{
    std::lock_guard<std::mutex> lock(g_trace_mutex);
    if (slot >= 0 && slot < (int)g_trace.size()) cudaEventRecord(g_trace[slot].e1, st);
}
} // namespace clb_host

// ---- tuning knobs and per-device facts ---------------------------------------------------------------
namespace {
std::atomic<long long> g_tapgrad_slice_bytes{0};
std::atomic<long long> g_plane_kernels{1};
std::atomic<long long> g_slab_mux{0};
std::atomic<int> g_sm_count[64];
} // namespace

namespace clb_host {
long long tune_get(int key)
{
    if (key == CLB_TUNE_TAPGRAD_SLICE_BYTES) return g_tapgrad_slice_bytes.load(std::memory_order_relaxed);
    if (key == CLB_TUNE_PLANE_KERNELS) return g_plane_kernels.load(std::memory_order_relaxed);
    if (key == CLB_TUNE_SLAB_MUX) return g_slab_mux.load(std::memory_order_relaxed);
    return -1;
}
int sm_count()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        return 148;
    }
    int n = g_sm_count[dev].load(std::memory_order_relaxed);
    if (n <= 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = 148; // B200; also what a query without a device (size planning on the host) assumes
        }
        g_sm_count[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}
namespace {
struct SmemEntry {
    const void *kernel;
    int dev, bytes;
};
std::mutex g_smem_mu;
SmemEntry g_smem[256];
int g_smem_n = 0;
} // namespace
cudaError_t ensure_dynamic_smem_ptr(const void *kernel, int bytes)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return cudaGetLastError();
    std::lock_guard<std::mutex> lock(g_smem_mu);
    SmemEntry *slot = nullptr;
    for (int i = 0; i < g_smem_n; ++i)
        if (g_smem[i].kernel == kernel && g_smem[i].dev == dev) {
            if (g_smem[i].bytes >= bytes) return cudaSuccess;
            slot = &g_smem[i];
            break;
        }
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    if (!slot && g_smem_n < 256) slot = &g_smem[g_smem_n++]; // a full table only costs the repeated driver call
    if (slot) *slot = SmemEntry{kernel, dev, bytes};
    return cudaSuccess;
}
} // namespace clb_host

extern "C" int clb_tune(int key, long long value)
{
    if (key == CLB_TUNE_TAPGRAD_SLICE_BYTES && value >= 0) {
        g_tapgrad_slice_bytes.store(value, std::memory_order_relaxed);
        return CLB_OK;
    }
    if (key == CLB_TUNE_SLAB_MUX && (value == 0 || value == 1)) {
        g_slab_mux.store(value, std::memory_order_relaxed);
        return CLB_OK;
    }
    if (key == CLB_TUNE_PLANE_KERNELS && (value == 0 || value == 1)) {
        g_plane_kernels.store(value, std::memory_order_relaxed);
        return CLB_OK;
    }
    return CLB_ERR_ARG;
}
extern "C" long long clb_tune_get(int key) { return clb_host::tune_get(key); }

extern "C" int clb_trace(int on)
{
    std::lock_guard<std::mutex> lock(g_trace_mutex);
    trace_drop_locked();
    g_trace_on.store(on ? 1 : 0, std::memory_order_relaxed);
    return CLB_OK;
}

extern "C" long long clb_trace_report(char *buf, size_t cap)
{
    std::lock_guard<std::mutex> lock(g_trace_mutex);
    struct Row {
        const char *name;
        long long launches;
        double ms;
    };
    std::vector<Row> rows;
    for (TraceRec &r : g_trace) {
        float ms = 0.f;
        if (cudaEventSynchronize(r.e1) != cudaSuccess || cudaEventElapsedTime(&ms, r.e0, r.e1) != cudaSuccess) {
            cudaGetLastError();
            continue;
        }
        size_t i = 0;
        for (; i < rows.size(); ++i)
            if (rows[i].name == r.name || std::strcmp(rows[i].name, r.name) == 0) break;
        if (i == rows.size()) rows.push_back(Row{r.name, 0, 0.0});
        rows[i].launches += 1;
        rows[i].ms += ms;
    }
    std::string out;
    char line[256];
    for (const Row &r : rows) {
        std::snprintf(line, sizeof line, "%s\t%lld\t%.6f\n", r.name, r.launches, r.ms);
        out += line;
    }
    trace_drop_locked();
    if (buf && cap > 0) {
        const size_t n = out.size() < cap - 1 ? out.size() : cap - 1;
        std::memcpy(buf, out.data(), n);
        buf[n] = 0;
    }
    return (long long)out.size() + 1;
}

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
