// TreeLogicLayer kernels: one pairwise gate level on the trailing dimension.
//   x, gx [N,C,HW,2X]   y, gy [N,C,HW,X]   w, gw [C,X,16]
// A block works on one channel c (its X gates are block-uniform, in shared memory); thread <->
// (position, p) with p fastest, so x is read as contiguous pairs and y written contiguously.
// The gate gradient uses the same deterministic two-stage reduction as the conv kernels.
#include "clb_common.cuh"

namespace clb {

constexpr int kTreeMaxX = 256;

template <typename T>
__device__ __forceinline__ void load_tree_gates(Gate<T> *sg, const T *__restrict__ w, int c, int X, int wmode)
{
    for (int p = threadIdx.x; p < X; p += blockDim.x) sg[p] = gate_load<T>(w + ((size_t)c * X + p) * 16, wmode);
}

// MODE 0: forward; MODE 1: backward w.r.t. x.   grid (chunks, C, N)
template <typename T, int MODE>
__global__ void __launch_bounds__(256) tree_map_kernel(const T *__restrict__ x, const T *__restrict__ w, const T *__restrict__ gy,
                                                       T *__restrict__ out, int C, int HW, int X, int wmode)
{
    __shared__ Gate<T> sg[kTreeMaxX];
    const int c = blockIdx.y, n = blockIdx.z;
    load_tree_gates<T>(sg, w, c, X, wmode);
    __syncthreads();
    const size_t base = ((size_t)n * C + c) * HW * X; // offset in units of gates
    const long long total = (long long)HW * X;
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < total; j += (long long)gridDim.x * blockDim.x) {
        const int p = (int)(j % X);
        const T a = x[(base + j) * 2], b = x[(base + j) * 2 + 1];
        if (MODE == 0) {
            out[base + j] = gate_eval<T>(sg[p], a, b);
        } else {
            const T g = gy[base + j];
            out[(base + j) * 2] = g * gate_da<T>(sg[p], b);
            out[(base + j) * 2 + 1] = g * gate_db<T>(sg[p], a);
        }
    }
}

// grid (parts, C).  blockDim is a multiple of X' = the largest divisor layout: thread t owns gate p = t % X.
template <typename T>
__global__ void __launch_bounds__(256) tree_bwd_w_kernel(const T *__restrict__ x, const T *__restrict__ gy, T *__restrict__ partial,
                                                         int N, int C, int HW, int X, int threads_used)
{
    __shared__ T red[256][4];
    const int c = blockIdx.y, t = threadIdx.x;
    const int p = t % X, lane_pos = t / X, pos_stride = threads_used / X;
    T acc[4] = {T(0), T(0), T(0), T(0)};
    const long long total = (long long)N * HW; // positions of this channel over the batch
    const long long per = (total + gridDim.x - 1) / gridDim.x;
    const long long lo = per * blockIdx.x, hi = min(total, lo + per);
    if (t < threads_used) {
        for (long long q = lo + lane_pos; q < hi; q += pos_stride) {
            const int n = (int)(q / HW), pos = (int)(q % HW);
            const size_t e = (((size_t)n * C + c) * HW + pos) * X + p;
            const T a = x[e * 2], b = x[e * 2 + 1], g = gy[e];
            acc[0] = fma_t<T>(g, a * b, acc[0]);
            acc[1] = fma_t<T>(g, a, acc[1]);
            acc[2] = fma_t<T>(g, b, acc[2]);
            acc[3] += g;
        }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) red[t][k] = acc[k];
    __syncthreads();
    if (t < X) {
        T s[4] = {T(0), T(0), T(0), T(0)};
        for (int u = t; u < threads_used; u += X) {
#pragma unroll
            for (int k = 0; k < 4; ++k) s[k] += red[u][k];
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) partial[(((size_t)blockIdx.x * C + c) * X + t) * 4 + k] = s[k];
    }
}

template <typename T>
__global__ void tree_grad_finalize_kernel(const T *__restrict__ partial, const T *__restrict__ w, T *__restrict__ gw, int parts,
                                          long long ngates, int wmode)
{
    const long long gi = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gi >= ngates) return;
    T sums[4] = {T(0), T(0), T(0), T(0)};
    for (int p = 0; p < parts; ++p) {
#pragma unroll
        for (int k = 0; k < 4; ++k) sums[k] += partial[((size_t)p * ngates + gi) * 4 + k];
    }
    gate_grad_store<T>(sums, w + gi * 16, wmode, gw + gi * 16);
}

} // namespace clb

using namespace clb;
using namespace clb_host;

static bool tree_args_ok(int N, int C, int HW, int X) { return N >= 0 && C >= 0 && HW >= 0 && X >= 1; }

template <int MODE>
static int launch_tree_map(const void *x, const void *w, const void *gy, void *out, int N, int C, int HW, int X, int wmode,
                           int dtype, void *stream)
{
    if (!tree_args_ok(N, C, HW, X) || !x || !w || !out || (MODE == 1 && !gy) || wmode < 0 || wmode > 2) return CLB_ERR_ARG;
    if (X > kTreeMaxX || C > 65535 || N > 65535) return CLB_ERR_SHAPE;
    if (N == 0 || C == 0 || HW == 0) return CLB_OK;
    long long chunks = ((long long)HW * X + 255) / 256;
    if (chunks > 64) chunks = 64;
    dim3 grid((unsigned)chunks, C, N);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == CLB_F32)
        CLB_TRACED("tree_map_kernel", st, tree_map_kernel<float, MODE><<<grid, 256, 0, st>>>((const float *)x, (const float *)w, (const float *)gy, (float *)out, C, HW, X, wmode));
    else if (dtype == CLB_F64)
        CLB_TRACED("tree_map_kernel", st, tree_map_kernel<double, MODE><<<grid, 256, 0, st>>>((const double *)x, (const double *)w, (const double *)gy, (double *)out, C, HW, X, wmode));
    else
        return CLB_ERR_ARG;
    return check_launch();
}

extern "C" int clb_tree_fwd(const void *x, const void *w, void *y, int N, int C, int HW, int X, int wmode, int dtype, void *stream)
{
    return launch_tree_map<0>(x, w, nullptr, y, N, C, HW, X, wmode, dtype, stream);
}
extern "C" int clb_tree_bwd_x(const void *gy, const void *x, const void *w, void *gx, int N, int C, int HW, int X, int wmode,
                              int dtype, void *stream)
{
    return launch_tree_map<1>(x, w, gy, gx, N, C, HW, X, wmode, dtype, stream);
}

static int tree_parts(long long positions, int C)
{
    long long parts = ((long long)sm_count() * 8 + C - 1) / (C > 0 ? C : 1);
    long long most = positions / 1024;
    if (parts > most) parts = most;
    if (parts < 1) parts = 1;
    if (parts > 1024) parts = 1024;
    return (int)parts;
}

extern "C" size_t clb_tree_bwd_w_scratch_bytes(int N, int C, int HW, int X, int dtype)
{
    return (size_t)tree_parts((long long)N * HW, C) * (size_t)C * X * 4 * (dtype == CLB_F64 ? 8 : 4);
}

extern "C" int clb_tree_bwd_w(const void *gy, const void *x, const void *w, void *gw, void *scratch, size_t scratch_bytes, int N,
                              int C, int HW, int X, int wmode, int dtype, void *stream)
{
    if (!tree_args_ok(N, C, HW, X) || !x || !w || !gy || !gw || wmode < 0 || wmode > 2) return CLB_ERR_ARG;
    if (dtype != CLB_F32 && dtype != CLB_F64) return CLB_ERR_ARG;
    if (X > kTreeMaxX || C > 65535) return CLB_ERR_SHAPE;
    if (C == 0) return CLB_OK;
    const int parts = tree_parts((long long)N * HW, C);
    if (!scratch || scratch_bytes < clb_tree_bwd_w_scratch_bytes(N, C, HW, X, dtype)) return CLB_ERR_SCRATCH;
    const int threads_used = (256 / X) * X;
    dim3 grid(parts, C);
    const long long ngates = (long long)C * X;
    const int fb = (int)((ngates + 127) / 128);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == CLB_F32) {
        CLB_TRACED("tree_bwd_w_kernel", st, tree_bwd_w_kernel<float><<<grid, 256, 0, st>>>((const float *)x, (const float *)gy, (float *)scratch, N, C, HW, X, threads_used));
        CLB_TRACED("tree_grad_finalize_kernel", st, tree_grad_finalize_kernel<float><<<fb, 128, 0, st>>>((const float *)scratch, (const float *)w, (float *)gw, parts, ngates, wmode));
    } else {
        CLB_TRACED("tree_bwd_w_kernel", st, tree_bwd_w_kernel<double><<<grid, 256, 0, st>>>((const double *)x, (const double *)gy, (double *)scratch, N, C, HW, X, threads_used));
        CLB_TRACED("tree_grad_finalize_kernel", st, tree_grad_finalize_kernel<double><<<fb, 128, 0, st>>>((const double *)scratch, (const double *)w, (double *)gw, parts, ngates, wmode));
    }
    return check_launch(2);
}
