// Shared device/host helpers of the convlogic_b200 kernels (sm_100a).
//
// Gate algebra.  Each of the 16 two-input gates is multilinear on [0,1]^2:
//     op_i(a, b) = K[0][i]*ab + K[1][i]*a + K[2][i]*b + K[3][i]
// (the reference keeps the same table as `coefs_T`, src/convlogic/cuda/full_convlogic_kernel.cu:692-696),
// so a mixture  sum_i w_i op_i(a, b)  collapses to four coefficients per gate,
//     y = k1 + ka*a + kb*b + kab*ab,   (ka, kb, kab, k1) = K w,
// which costs three FMAs per gate instead of the reference's 15-term sum, and the gradient w.r.t.
// the mixture is  K^T (sum gy*ab, sum gy*a, sum gy*b, sum gy).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/convlogic_b200.h"

namespace clb {

// K[r][i] for rows r = 0..3 = (ab, a, b, 1), derived from gate i's truth table
// (id bit 3 = f(0,0), bit 2 = f(0,1), bit 1 = f(1,0), bit 0 = f(1,1)) by multilinear interpolation.
// Pure arithmetic, so fully unrolled loops fold it to constants.
__host__ __device__ constexpr int kcoef(int r, int i)
{
    return r == 3   ? ((i >> 3) & 1)
           : r == 1 ? (((i >> 1) & 1) - ((i >> 3) & 1))
           : r == 2 ? (((i >> 2) & 1) - ((i >> 3) & 1))
                    : ((i & 1) - ((i >> 1) & 1) - ((i >> 2) & 1) + ((i >> 3) & 1));
}

template <typename T> struct Gate {
    T k1, ka, kb, kab;
};

template <typename T> __device__ __forceinline__ T fma_t(T a, T b, T c);
template <> __device__ __forceinline__ float fma_t<float>(float a, float b, float c) { return fmaf(a, b, c); }
template <> __device__ __forceinline__ double fma_t<double>(double a, double b, double c) { return fma(a, b, c); }

template <typename T> __device__ __forceinline__ T gate_eval(const Gate<T> &g, T a, T b)
{
    return fma_t<T>(a, fma_t<T>(g.kab, b, g.ka), fma_t<T>(g.kb, b, g.k1));
}
template <typename T> __device__ __forceinline__ T gate_da(const Gate<T> &g, T b) { return fma_t<T>(g.kab, b, g.ka); }
template <typename T> __device__ __forceinline__ T gate_db(const Gate<T> &g, T a) { return fma_t<T>(g.kab, a, g.kb); }

// Mixture over the 16 gates from the 16 stored values of one gate, according to wmode.
template <typename T> __device__ __forceinline__ void gate_mixture(const T *__restrict__ w16, int wmode, T p[16])
{
#pragma unroll
    for (int i = 0; i < 16; ++i) p[i] = w16[i];
    if (wmode == CLB_W_SOFTMAX) {
        T m = p[0];
#pragma unroll
        for (int i = 1; i < 16; ++i) m = p[i] > m ? p[i] : m;
        T s = T(0);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            p[i] = exp(p[i] - m);
            s += p[i];
        }
        T inv = T(1) / s;
#pragma unroll
        for (int i = 0; i < 16; ++i) p[i] *= inv;
    } else if (wmode == CLB_W_ARGMAX) {
        int best = 0;
        T m = p[0];
#pragma unroll
        for (int i = 1; i < 16; ++i)
            if (p[i] > m) {
                m = p[i];
                best = i;
            }
#pragma unroll
        for (int i = 0; i < 16; ++i) p[i] = (i == best) ? T(1) : T(0);
    }
}

template <typename T> __device__ __forceinline__ Gate<T> gate_from_mixture(const T p[16])
{
    Gate<T> g;
    g.kab = g.ka = g.kb = g.k1 = T(0);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        g.kab += T(kcoef(0, i)) * p[i];
        g.ka += T(kcoef(1, i)) * p[i];
        g.kb += T(kcoef(2, i)) * p[i];
        g.k1 += T(kcoef(3, i)) * p[i];
    }
    return g;
}

template <typename T> __device__ __forceinline__ Gate<T> gate_load(const T *__restrict__ w16, int wmode)
{
    T p[16];
    gate_mixture<T>(w16, wmode, p);
    return gate_from_mixture<T>(p);
}

// Basis sums (sum gy*ab, sum gy*a, sum gy*b, sum gy) -> 16 gradients of one gate.
// CLB_W_PROB / CLB_W_ARGMAX: gradient w.r.t. the mixture.  CLB_W_SOFTMAX: w.r.t. the logits.
template <typename T>
__device__ __forceinline__ void gate_grad_store(const T s[4], const T *__restrict__ w16, int wmode, T *__restrict__ out16)
{
    T g[16];
#pragma unroll
    for (int i = 0; i < 16; ++i)
        g[i] = T(kcoef(0, i)) * s[0] + T(kcoef(1, i)) * s[1] + T(kcoef(2, i)) * s[2] + T(kcoef(3, i)) * s[3];
    if (wmode == CLB_W_SOFTMAX) {
        T p[16];
        gate_mixture<T>(w16, CLB_W_SOFTMAX, p);
        T dot = T(0);
#pragma unroll
        for (int i = 0; i < 16; ++i) dot += p[i] * g[i];
#pragma unroll
        for (int i = 0; i < 16; ++i) g[i] = p[i] * (g[i] - dot);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) out16[i] = g[i];
}

struct Tap {
    int ch, dy, dx; // channel, row/col offset already reduced by the padding
};
__device__ __forceinline__ Tap unpack_tap(int32_t word, int ph, int pw)
{
    Tap t;
    t.ch = (word >> 16) & 0xFFFF;
    t.dy = ((word >> 8) & 0xFF) - ph;
    t.dx = (word & 0xFF) - pw;
    return t;
}

template <typename T> __device__ __forceinline__ T warp_sum(T v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

} // namespace clb

// ---- host side ----------------------------------------------------------------------------------
namespace clb_host {
void set_last_cuda_error(int e);
void count_launches(int n);
// Call after launching `n` kernels: reports a refused launch, else adds n to the library's counter.
inline int check_launch(int n = 1)
{
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        set_last_cuda_error((int)e);
        cudaGetLastError(); // clear the sticky-less launch error so later calls start clean
        return CLB_ERR_LAUNCH;
    }
    count_launches(n);
    return CLB_OK;
}
long long tune_get(int key); // clb_tune's current value
int sm_count();              // multiprocessors of the current device, asked once per device
// Raises a kernel's dynamic shared-memory limit to `bytes`; the driver is asked once per (kernel, device), later
// calls with the same or a smaller size are a table look-up.
cudaError_t ensure_dynamic_smem_ptr(const void *kernel, int bytes);
template <typename K> inline cudaError_t ensure_dynamic_smem(K kernel, int bytes)
{
    return ensure_dynamic_smem_ptr(reinterpret_cast<const void *>(kernel), bytes);
}
// Launch tracing (clb_trace / clb_trace_report): while it is on, a traced launch is bracketed by two CUDA
// events on its stream; off, the cost is one relaxed atomic load.
bool trace_enabled();
int trace_begin(const char *name, cudaStream_t st);
void trace_end(int slot, cudaStream_t st);
struct TraceScope {
    int slot;
    cudaStream_t st;
    TraceScope(const char *name, cudaStream_t s) : slot(trace_enabled() ? trace_begin(name, s) : -1), st(s) {}
    ~TraceScope()
    {
        if (slot >= 0) trace_end(slot, st);
    }
};
// CLB_TRACED("kernel name", stream, kernel<<<grid, block, smem, stream>>>(args...));
#define CLB_TRACED(name, st, ...)                                                                                       \
    do {                                                                                                                \
        clb_host::TraceScope clb_trace_scope_(name, st);                                                                \
        __VA_ARGS__;                                                                                                    \
    } while (0)
inline int conv_out(int in, int pad, int k, int stride) { return (in + 2 * pad - k) / stride + 1; }
inline bool conv_args_ok(int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw)
{
    return N >= 0 && Ci > 0 && H > 0 && W > 0 && C >= 0 && sh > 0 && sw > 0 && ph >= 0 && pw >= 0 && kh > 0 && kw > 0 &&
           kh <= 256 && kw <= 256 && Ci <= 65536;
}
} // namespace clb_host
