// Flat LogicLayer kernels on feature-major activations: x [in,B], y [out,B], batch contiguous.
//
// The work is HBM-bound (two gathered input rows and one output row per neuron, three FMAs per
// element), so the layout of the loop is chosen for memory: one warp owns one neuron (forward, gate
// gradient) or one input feature (input gradient) and sweeps the batch with 128-bit accesses, every
// row access being a fully coalesced 512-byte segment per warp.  The 16 gate values of a neuron are
// read once per warp: 16 lanes load one value each and the soft-max / 4-coefficient reduction runs on
// shuffles inside the half-warp, two neurons at a time.
//
// Input gradient: segmented reduction over the consumer lists (CSR), no atomics, fixed order.
// A neuron whose two inputs are the same feature is listed twice in a row; the first entry takes the
// derivative w.r.t. its first input and the second w.r.t. its second input, so the sum is the true
// derivative (the reference kernel, src/difflogic/cuda/difflogic_kernel.cu:196-226, applies the
// first-input derivative twice in that case; its CPU path gives the sum used here).
#include "clb_common.cuh"

#include <cmath>

namespace clb {

// Each half-warp reduces the 16 values of one neuron: the lane handles value (lane & 15) of neuron
// `j` (the same j in all 16 lanes of a half-warp; the two halves may name unrelated neurons).
// Returns that neuron's gate in every lane of the half-warp, plus the lane's mixture value p.
// Neurons outside [0, out_dim) give zeros.
template <typename T>
__device__ __forceinline__ Gate<T> half_warp_gate(const T *__restrict__ w, long long j, long long out_dim, int wmode, int lane, T &p)
{
    const int i = lane & 15;
    T v = (j >= 0 && j < out_dim) ? w[j * 16 + i] : T(0);
    if (wmode == CLB_W_SOFTMAX) {
        T m = v;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            const T u = __shfl_xor_sync(0xffffffffu, m, o);
            m = u > m ? u : m;
        }
        v = exp(v - m);
        T s = v;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        v = v / s;
    } else if (wmode == CLB_W_ARGMAX) {
        // first maximum: compare (value, -index) pairs
        T m = v;
        int bi = i;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            const T um = __shfl_xor_sync(0xffffffffu, m, o);
            const int ui = __shfl_xor_sync(0xffffffffu, bi, o);
            if (um > m || (um == m && ui < bi)) {
                m = um;
                bi = ui;
            }
        }
        v = (i == bi) ? T(1) : T(0);
    }
    p = v;
    Gate<T> g;
    g.kab = T(kcoef(0, i)) * v;
    g.ka = T(kcoef(1, i)) * v;
    g.kb = T(kcoef(2, i)) * v;
    g.k1 = T(kcoef(3, i)) * v;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
        g.kab += __shfl_xor_sync(0xffffffffu, g.kab, o);
        g.ka += __shfl_xor_sync(0xffffffffu, g.ka, o);
        g.kb += __shfl_xor_sync(0xffffffffu, g.kb, o);
        g.k1 += __shfl_xor_sync(0xffffffffu, g.k1, o);
    }
    return g;
}

template <typename T> __device__ __forceinline__ Gate<T> gate_from_lane(const Gate<T> &g, int src)
{
    Gate<T> r;
    r.kab = __shfl_sync(0xffffffffu, g.kab, src);
    r.ka = __shfl_sync(0xffffffffu, g.ka, src);
    r.kb = __shfl_sync(0xffffffffu, g.kb, src);
    r.k1 = __shfl_sync(0xffffffffu, g.k1, src);
    return r;
}

template <typename T, int V> struct Vec;
template <> struct Vec<float, 4> { using type = float4; };
template <> struct Vec<float, 1> { using type = float; };
template <> struct Vec<double, 1> { using type = double; };
template <> struct Vec<double, 2> { using type = double2; };

template <typename T, int V> __device__ __forceinline__ void vload(const T *p, T (&r)[V])
{
    using VT = typename Vec<T, V>::type;
    const VT v = __ldg(reinterpret_cast<const VT *>(p));
    const T *e = reinterpret_cast<const T *>(&v);
#pragma unroll
    for (int k = 0; k < V; ++k) r[k] = e[k];
}
template <typename T, int V> __device__ __forceinline__ void vstore(T *p, const T (&r)[V])
{
    using VT = typename Vec<T, V>::type;
    VT v;
    T *e = reinterpret_cast<T *>(&v);
#pragma unroll
    for (int k = 0; k < V; ++k) e[k] = r[k];
    *reinterpret_cast<VT *>(p) = v;
}

// ---------------------------------------------------------------------------------------- forward
template <typename T, int V>
__global__ void __launch_bounds__(256) logic_fwd_kernel(const T *__restrict__ x, const int64_t *__restrict__ ia,
                                                        const int64_t *__restrict__ ib, const T *__restrict__ w, T *__restrict__ y,
                                                        long long out_dim, long long B, int wmode)
{
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long j0 = warp * 2; j0 < out_dim; j0 += nwarps * 2) {
        T p;
        const Gate<T> gh = half_warp_gate<T>(w, j0 + (lane >> 4), out_dim, wmode, lane, p);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const long long j = j0 + h;
            if (j >= out_dim) break;
            const Gate<T> g = gate_from_lane<T>(gh, h * 16);
            const T *xa = x + ia[j] * B, *xb = x + ib[j] * B;
            T *yo = y + j * B;
            for (long long b0 = (long long)lane * V; b0 < B; b0 += 32 * V) {
                T a[V], b[V], r[V];
                vload<T, V>(xa + b0, a);
                vload<T, V>(xb + b0, b);
#pragma unroll
                for (int k = 0; k < V; ++k) r[k] = gate_eval<T>(g, a[k], b[k]);
                vstore<T, V>(yo + b0, r);
            }
        }
    }
}

// ------------------------------------------------------------------------------------ gate grads
template <typename T, int V>
__global__ void __launch_bounds__(256) logic_bwd_w_kernel(const T *__restrict__ x, const int64_t *__restrict__ ia,
                                                          const int64_t *__restrict__ ib, const T *__restrict__ w,
                                                          const T *__restrict__ gy, T *__restrict__ gw, long long out_dim, long long B,
                                                          int wmode)
{
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long j0 = warp * 2; j0 < out_dim; j0 += nwarps * 2) {
        T s[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const long long j = j0 + h;
            T acc[4] = {T(0), T(0), T(0), T(0)};
            if (j < out_dim) {
                const T *xa = x + ia[j] * B, *xb = x + ib[j] * B, *g = gy + j * B;
                for (long long b0 = (long long)lane * V; b0 < B; b0 += 32 * V) {
                    T a[V], b[V], d[V];
                    vload<T, V>(xa + b0, a);
                    vload<T, V>(xb + b0, b);
                    vload<T, V>(g + b0, d);
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        acc[0] = fma_t<T>(d[k], a[k] * b[k], acc[0]);
                        acc[1] = fma_t<T>(d[k], a[k], acc[1]);
                        acc[2] = fma_t<T>(d[k], b[k], acc[2]);
                        acc[3] += d[k];
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) s[h][k] = warp_sum<T>(acc[k]);
        }
        // lane l writes gradient (l & 15) of neuron j0 + (l >> 4)
        const int h = lane >> 4, i = lane & 15;
        const long long j = j0 + h;
        T sh4[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) sh4[k] = h ? s[1][k] : s[0][k];
        T gi = T(kcoef(0, i)) * sh4[0] + T(kcoef(1, i)) * sh4[1] + T(kcoef(2, i)) * sh4[2] + T(kcoef(3, i)) * sh4[3];
        if (wmode == CLB_W_SOFTMAX) {
            T p;
            (void)half_warp_gate<T>(w, j, out_dim, CLB_W_SOFTMAX, lane, p);
            T dot = p * gi;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            gi = p * (gi - dot);
        }
        if (j < out_dim) gw[j * 16 + i] = gi;
    }
}

// ----------------------------------------------------------------------------------- input grads
// gx[f] = sum over the consumers j of feature f (CSR lists built at construction) of  gy[j] * d op_j / d x_f.
// A warp owns a unit = (FPU consecutive features, batch split); the consumer entries of consecutive features are
// one contiguous range of the CSR list, so the warp walks that range 32 entries at a time whatever the fan-out:
// lane l reads entry e0+l, finds the feature it belongs to (a 5-step search over the 32 list starts held by the
// lanes), reads the consumer's two input indices and 16 logits, takes the soft-max and keeps the two coefficients
// (k0, kab) of  d op / d x_f = k0 + kab * other.  The entries are then handed round by shuffles while all lanes
// stream each entry's two rows (gy[j] and the other operand's x row), U entries' loads in flight at a time; the
// running sum is stored and reset whenever the feature changes (features without consumers get zeros).  FPU is 1
// for wide fan-outs (one feature per warp) and up to 32 when a feature has one or two consumers, where a per-feature
// chain of dependent loads would otherwise dominate.  Entries are added in list order: no dependence on scheduling.
template <typename T, int V, int SLOTS>
__global__ void __launch_bounds__(256) logic_bwd_x_kernel(const T *__restrict__ x, const int64_t *__restrict__ ia,
                                                          const int64_t *__restrict__ ib, const T *__restrict__ w,
                                                          const T *__restrict__ gy, T *__restrict__ gx,
                                                          const int64_t *__restrict__ start, const int64_t *__restrict__ cons,
                                                          long long in_dim, long long out_dim, long long B, int wmode,
                                                          int batch_splits, int fpu)
{
    constexpr int U = 8 / SLOTS; // entries whose rows are loaded before the first is added
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    // a split is a multiple of 32*V elements
    const long long span = ((B + (long long)batch_splits * 32 * V - 1) / ((long long)batch_splits * 32 * V)) * 32 * V;
    const long long funits = (in_dim + fpu - 1) / fpu;
    for (long long unit = warp; unit < funits * batch_splits; unit += nwarps) {
        const long long f0 = (unit / batch_splits) * fpu, f1 = min(in_dim, f0 + fpu);
        const long long blo = (unit % batch_splits) * span, bhi = min(B, blo + span);
        const long long my_start = start[min(f0 + lane, f1)]; // lanes past the unit hold its end
        const long long lo = __shfl_sync(0xffffffffu, my_start, 0), hi = start[f1];
        for (long long bb = blo; bb < bhi; bb += (long long)SLOTS * 32 * V) {
            T acc[SLOTS][V];
#pragma unroll
            for (int q = 0; q < SLOTS; ++q)
#pragma unroll
                for (int k = 0; k < V; ++k) acc[q][k] = T(0);
            long long cur_f = f0; // the feature `acc` belongs to
            auto flush_to = [&](long long f_next) {
                while (cur_f < f_next) {
#pragma unroll
                    for (int q = 0; q < SLOTS; ++q) {
                        const long long b0 = bb + ((long long)q * 32 + lane) * V;
                        if (b0 < bhi) vstore<T, V>(gx + cur_f * B + b0, acc[q]);
#pragma unroll
                        for (int k = 0; k < V; ++k) acc[q][k] = T(0);
                    }
                    ++cur_f;
                }
            };
            for (long long c0 = lo; c0 < hi; c0 += 32) {
                const long long e = c0 + lane;
                int my_j = 0, my_other = 0, my_f = 0;
                T my_k0 = T(0), my_kab = T(0);
                {
                    // the feature of entry e: the last lane whose list start is <= e (entries past the range: any)
                    int sel = 0;
#pragma unroll
                    for (int step = 16; step >= 1; step >>= 1) {
                        const long long sv = __shfl_sync(0xffffffffu, my_start, sel + step);
                        if (sv <= e) sel += step;
                    }
                    const long long fs = __shfl_sync(0xffffffffu, my_start, sel);
                    if (e < hi) {
                        const long long f = f0 + sel;
                        const long long j = cons[e];
                        const long long a_j = ia[j], b_j = ib[j];
                        // a neuron fed twice by f is listed twice in a row: the first entry is w.r.t. a, the second w.r.t. b
                        const bool second = (a_j == f) && (b_j == f) && (e > fs) && (cons[e - 1] == j);
                        const bool wrt_a = (a_j == f) && !second;
                        const Gate<T> g = gate_load<T>(w + j * 16, wmode);
                        my_j = (int)j, my_other = (int)(wrt_a ? b_j : a_j), my_f = sel;
                        my_k0 = wrt_a ? g.ka : g.kb, my_kab = g.kab;
                    }
                }
                const int n = (int)min((long long)32, hi - c0);
                for (int i0 = 0; i0 < n; i0 += U) {
                    T o[U][SLOTS][V], d[U][SLOTS][V], k0[U], kab[U];
                    int fi[U];
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int i = min(i0 + u, n - 1); // past the end: a repeated load that is not added
                        const T *xo = x + (long long)__shfl_sync(0xffffffffu, my_other, i) * B;
                        const T *gr = gy + (long long)__shfl_sync(0xffffffffu, my_j, i) * B;
                        k0[u] = __shfl_sync(0xffffffffu, my_k0, i), kab[u] = __shfl_sync(0xffffffffu, my_kab, i);
                        fi[u] = __shfl_sync(0xffffffffu, my_f, i);
#pragma unroll
                        for (int q = 0; q < SLOTS; ++q) {
                            const long long b0 = bb + ((long long)q * 32 + lane) * V;
                            if (b0 < bhi) {
                                vload<T, V>(xo + b0, o[u][q]);
                                vload<T, V>(gr + b0, d[u][q]);
                            } else {
#pragma unroll
                                for (int k = 0; k < V; ++k) o[u][q][k] = T(0), d[u][q][k] = T(0);
                            }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        if (i0 + u < n) {
                            flush_to(f0 + fi[u]);
#pragma unroll
                            for (int q = 0; q < SLOTS; ++q)
#pragma unroll
                                for (int k = 0; k < V; ++k) acc[q][k] = fma_t<T>(d[u][q][k], fma_t<T>(kab[u], o[u][q][k], k0[u]), acc[q][k]);
                        }
                    }
                }
            }
            flush_to(f1);
        }
    }
}

// ----------------------------------------------------------------------------------- group sum
// GroupSum on the feature-major activations the flat layers produce ([F][B]; class c owns rows [c*S, (c+1)*S)):
// out[b][c] = (sum of the class's rows at sample b) / tau.  Two stages with a fixed order: block (batch tile,
// class, part) adds its share of the rows warp by warp and combines the eight warps in order; the finalize kernel
// adds the parts in order.  No transposed copy of the activations, no atomics.
constexpr int kGroupSumParts = 16;

template <typename T>
__global__ void __launch_bounds__(256) group_sum_partial_kernel(const T *__restrict__ y, T *__restrict__ partial, long long S, long long B, int k)
{
    __shared__ T red[8][32];
    const int lane = threadIdx.x & 31, wv = threadIdx.x >> 5;
    const long long b = (long long)blockIdx.x * 32 + lane;
    const int c = blockIdx.y, part = blockIdx.z;
    const long long r0 = S * part / gridDim.z, r1 = S * (part + 1) / gridDim.z;
    T acc = T(0);
    if (b < B)
        for (long long r = r0 + wv; r < r1; r += 8) acc += y[((long long)c * S + r) * B + b];
    red[wv][lane] = acc;
    __syncthreads();
    if (wv == 0 && b < B) {
        T t = red[0][lane];
#pragma unroll
        for (int i = 1; i < 8; ++i) t += red[i][lane];
        partial[((long long)part * k + c) * B + b] = t;
    }
}

template <typename T>
__global__ void group_sum_finalize_kernel(const T *__restrict__ partial, T *__restrict__ out, long long B, int k, int parts, T tau)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; // (c, b), b fastest
    if (i >= B * k) return;
    const long long c = i / B, b = i - c * B;
    T t = T(0);
    for (int p = 0; p < parts; ++p) t += partial[((long long)p * k + c) * B + b];
    out[b * k + c] = t / tau;
}

// GroupSum + cross-entropy finish (src/convlogic/model.py:137-152: CrossEntropyLoss on the GroupSum scores):
// scores[b][c] = (sum of the parts) / tau, loss = mean_b (logsumexp(scores[b]) - scores[b][label_b]), and
// dscore[b][c] = (softmax(scores[b])[c] - [c == label_b]) / B, the gradient of the mean loss w.r.t. the scores.
// A warp per sample, lane c = class c (k <= 32): the parts are added in part order with all loads in flight, the
// soft-max is two warp reductions.  The sample's loss overwrites partial[b] (part 0, class 0 of that sample: read by this
// warp alone, before the write); group_sum_loss_mean_kernel adds the B losses in a fixed tree.
__global__ void __launch_bounds__(256) group_sum_ce_sample_kernel(float *__restrict__ partial, const int64_t *__restrict__ labels,
                                                                  float *__restrict__ scores, float *__restrict__ dscore, long long B, int k,
                                                                  int parts, float tau)
{
    const int lane = threadIdx.x & 31;
    const long long b = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (b >= B) return; // the whole warp
    float sc = -3.0e38f;
    if (lane < k) {
        float t = 0.f;
        int p = 0;
        for (; p + 8 <= parts; p += 8) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = partial[((long long)(p + j) * k + lane) * B + b];
#pragma unroll
            for (int j = 0; j < 8; ++j) t += v[j];
        }
        for (; p < parts; ++p) t += partial[((long long)p * k + lane) * B + b];
        sc = t / tau;
    }
    float mx = sc;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float e = lane < k ? expf(sc - mx) : 0.f;
    const float sum = warp_sum<float>(e);
    const int lab = (int)labels[b];
    const bool lab_ok = lab >= 0 && lab < k;
    const float sc_lab = __shfl_sync(0xffffffffu, sc, lab_ok ? lab : 0);
    if (lane < k) {
        if (scores != nullptr) scores[b * k + lane] = sc;
        dscore[b * k + lane] = (e / sum - (lane == lab ? 1.f : 0.f)) / (float)B;
    }
    __syncwarp();
    if (lane == 0) partial[b] = mx + logf(sum) - (lab_ok ? sc_lab : 0.f);
}

__global__ void __launch_bounds__(256) group_sum_loss_mean_kernel(const float *__restrict__ sample_loss, float *__restrict__ loss, long long B)
{
    __shared__ float red[256];
    float mine = 0.f;
    for (long long b = threadIdx.x; b < B; b += 256) mine += sample_loss[b];
    red[threadIdx.x] = mine;
    __syncthreads();
    for (int half = 128; half >= 1; half >>= 1) {
        if ((int)threadIdx.x < half) red[threadIdx.x] += red[threadIdx.x + half];
        __syncthreads();
    }
    if (threadIdx.x == 0) *loss = red[0] / (float)B;
}

// out[c][r] = in[r][c]: 32 x 32 tiles through shared memory (33-float rows: no bank conflicts), both sides coalesced.
// The flat layers work on feature-major activations [features][batch]; this is the copy between that and the
// [batch][features] tensors of the layers around them.
__global__ void __launch_bounds__(256) transpose_f32_kernel(const float *__restrict__ in, float *__restrict__ out, long long R, long long Cc)
{
    __shared__ float tile[32][33];
    const long long c0 = (long long)blockIdx.x * 32, r0 = (long long)blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long r = r0 + ty + 8 * i, c = c0 + tx;
        if (r < R && c < Cc) tile[ty + 8 * i][tx] = __ldg(in + r * Cc + c);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long c = c0 + ty + 8 * i, r = r0 + tx;
        if (r < R && c < Cc) out[c * R + r] = tile[tx][ty + 8 * i];
    }
}

// Adam / AdamW over one flat parameter buffer (src/convlogic/model.py:179-180 uses torch.optim.AdamW): one thread per
// four elements, 128-bit accesses.  step_size = lr / (1 - beta1^t), bc2_sqrt = sqrt(1 - beta2^t).
__global__ void __launch_bounds__(256) adam_step_kernel(float *__restrict__ p, const float *__restrict__ g, float *__restrict__ m,
                                                        float *__restrict__ v, long long n, float lr, float beta1, float beta2, float eps,
                                                        float weight_decay, float step_size, float bc2_sqrt, int decoupled)
{
    auto one = [&](float &pp, float gg, float &mm, float &vv) {
        if (weight_decay != 0.f) {
            if (decoupled)
                pp *= 1.f - lr * weight_decay;
            else
                gg = fmaf(weight_decay, pp, gg);
        }
        mm = fmaf(1.f - beta1, gg - mm, mm);           // exp_avg.lerp_(grad, 1 - beta1)
        vv = fmaf(1.f - beta2, gg * gg, beta2 * vv);   // exp_avg_sq.mul_(beta2).addcmul_(grad, grad, 1 - beta2)
        const float denom = sqrtf(vv) / bc2_sqrt + eps;
        pp -= step_size * (mm / denom);
    };
    const long long n4 = n >> 2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
        float4 pp = reinterpret_cast<float4 *>(p)[i], mm = reinterpret_cast<float4 *>(m)[i], vv = reinterpret_cast<float4 *>(v)[i];
        const float4 gg = reinterpret_cast<const float4 *>(g)[i];
        one(pp.x, gg.x, mm.x, vv.x), one(pp.y, gg.y, mm.y, vv.y), one(pp.z, gg.z, mm.z, vv.z), one(pp.w, gg.w, mm.w, vv.w);
        reinterpret_cast<float4 *>(p)[i] = pp, reinterpret_cast<float4 *>(m)[i] = mm, reinterpret_cast<float4 *>(v)[i] = vv;
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
        const long long i = (n4 << 2) + threadIdx.x;
        one(p[i], g[i], m[i], v[i]);
    }
}

// gy[f][b] = gout[b][f / S] / tau.  grid (row chunks, k): a thread keeps the quotients of its batch positions
// in registers and writes them to every row of its chunk (coalesced along the batch).
template <typename T>
__global__ void __launch_bounds__(256) group_sum_bwd_kernel(const T *__restrict__ gout, const T *__restrict__ scale, T *__restrict__ gy,
                                                            long long S, long long B, int k, T tau)
{
    const int c = blockIdx.y;
    if (scale != nullptr) tau = tau / scale[0]; // an upstream scalar gradient, read on the device
    const long long r0 = S * blockIdx.x / gridDim.x, r1 = S * (blockIdx.x + 1) / gridDim.x;
    for (long long b0 = 0; b0 < B; b0 += 4 * 256) {
        T v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const long long b = b0 + q * 256 + threadIdx.x;
            v[q] = b < B ? gout[b * k + c] / tau : T(0);
        }
        for (long long r = r0; r < r1; ++r) {
            T *row = gy + ((long long)c * S + r) * B;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const long long b = b0 + q * 256 + threadIdx.x;
                if (b < B) row[b] = v[q];
            }
        }
    }
}

// ----------------------------------------------------------------------------------- fused flat layers (training)
// Three consecutive flat layers whose outputs are each read at most once by the next one, as ONE differentiable
// gate tree per neuron of the last layer: leaf [T][8] are rows of the first layer's input (gate p of the first
// level reads leaves 2p, 2p+1), node [T][7] the neuron that sits at each tree position (4 of the first layer, 2 of
// the second, 1 of the third: its logits are the gate's).  The two intermediate activations are never written.
// Forward: a warp per tree, lanes along the batch.  Backward pass 1: the chain recomputed from the leaves, the
// gradient w.r.t. each leaf written as a row of `tapgrad` [T*8][B], the 28 basis sums of the 7 gates reduced over
// the batch and turned into the logit (or mixture) gradients of the 7 neurons.  Pass 2: gx[f] = sum of the
// tapgrad rows of the leaves that are feature f (CSR by feature, fixed order).
struct TreeTables {
    const int32_t *leaf; // [T][8]
    const int32_t *node; // [T][7]
    const float *w[3];   // logits (or mixtures) of the three layers
};

// ---- the seven gates of a tree on the warp's lanes: the quad of lanes 4g..4g+3 owns gate g (lanes 28..31 idle), lane
// q = lane & 3 of a quad holds entries 4q..4q+3 of the gate's 16.  Gate id j = 4q + i has truth-table bits (q >> 1,
// q & 1, i >> 1, i & 1), so the coefficients of the multilinear form follow from three sums of the lane's four entries.
__device__ __forceinline__ float quad_sum(float v)
{
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// the lane's four entries of the mixture over the 16 gates (zeros on an idle lane); every lane of the warp calls this
__device__ __forceinline__ void quad_mixture(const float *__restrict__ w16, int wmode, int q, bool active, float (&p)[4])
{
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = active ? __ldg(w16 + 4 * q + i) : 0.f;
    if (wmode == CLB_W_SOFTMAX) {
        float m = fmaxf(fmaxf(p[0], p[1]), fmaxf(p[2], p[3]));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = expf(p[i] - m);
        const float inv = 1.f / quad_sum((p[0] + p[1]) + (p[2] + p[3]));
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] *= inv;
    } else if (wmode == CLB_W_ARGMAX) {   // the first largest entry, as a scan from entry 0 finds it
        float m = p[0];
        int best = 4 * q;
#pragma unroll
        for (int i = 1; i < 4; ++i)
            if (p[i] > m) m = p[i], best = 4 * q + i;
#pragma unroll
        for (int o = 1; o <= 2; o <<= 1) {
            const float mo = __shfl_xor_sync(0xffffffffu, m, o);
            const int bo = __shfl_xor_sync(0xffffffffu, best, o);
            if (mo > m || (mo == m && bo < best)) m = mo, best = bo;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = (4 * q + i == best) ? 1.f : 0.f;
    }
}

// coefficients of the quad's gate from the four lanes' mixture entries (every lane of the quad gets them)
__device__ __forceinline__ Gate<float> quad_gate(const float (&p)[4], int q)
{
    const float q3 = (float)(q >> 1), q2 = (float)(q & 1);
    const float all = (p[0] + p[1]) + (p[2] + p[3]), hi = p[2] + p[3], odd = p[1] + p[3];
    Gate<float> g;
    g.k1 = quad_sum(q3 * all);
    g.ka = quad_sum(hi - q3 * all);
    g.kb = quad_sum((q2 - q3) * all);
    g.kab = quad_sum(odd - hi + (q3 - q2) * all);
    return g;
}

// neuron behind the lane's gate (lane < 28) and that neuron's row of 16 values
__device__ __forceinline__ long long tree_node(const TreeTables &tt, long long t, int lane) { return __ldg(tt.node + t * 7 + (lane >> 2)); }
__device__ __forceinline__ const float *tree_row(const TreeTables &tt, int lane, long long n)
{
    const int g = lane >> 2;
    return tt.w[g < 4 ? 0 : (g < 6 ? 1 : 2)] + n * 16;
}

// every lane gets all seven gates
__device__ __forceinline__ void tree_gates(const TreeTables &tt, long long t, int lane, int wmode, Gate<float> (&g)[7])
{
    const bool active = lane < 28;
    const long long n = active ? tree_node(tt, t, lane) : 0;
    float p[4];
    quad_mixture(tree_row(tt, active ? lane : 0, n), wmode, lane & 3, active, p);
    const Gate<float> mine = quad_gate(p, lane & 3);
#pragma unroll
    for (int i = 0; i < 7; ++i) {
        g[i].k1 = __shfl_sync(0xffffffffu, mine.k1, 4 * i), g[i].ka = __shfl_sync(0xffffffffu, mine.ka, 4 * i);
        g[i].kb = __shfl_sync(0xffffffffu, mine.kb, 4 * i), g[i].kab = __shfl_sync(0xffffffffu, mine.kab, 4 * i);
    }
}
// the same with the lane's neuron already known (lanes >= 28: any value); p = the lane's four mixture entries
__device__ __forceinline__ void tree_gates_of(const TreeTables &tt, long long n, int lane, int wmode, Gate<float> (&g)[7], float (&p)[4])
{
    const bool active = lane < 28;
    quad_mixture(tree_row(tt, active ? lane : 0, n), wmode, lane & 3, active, p);
    const Gate<float> mine = quad_gate(p, lane & 3);
#pragma unroll
    for (int i = 0; i < 7; ++i) {
        g[i].k1 = __shfl_sync(0xffffffffu, mine.k1, 4 * i), g[i].ka = __shfl_sync(0xffffffffu, mine.ka, 4 * i);
        g[i].kb = __shfl_sync(0xffffffffu, mine.kb, 4 * i), g[i].kab = __shfl_sync(0xffffffffu, mine.kab, 4 * i);
    }
}

template <int V>
__global__ void __launch_bounds__(256, 3) logic_tree_fwd_kernel(const float *__restrict__ x, TreeTables tt, float *__restrict__ y, long long T,
                                                             long long B, int wmode)
{
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    // The tables of a tree (leaf rows on lanes 0..7, the gates' neurons on lanes 0..27) are fetched one tree ahead, so that
    // a tree's own chain of dependent loads is one hop (the rows, the logits) instead of two (index, then data).
    int my_leaf = (warp < T && lane < 8) ? __ldg(tt.leaf + warp * 8 + lane) : 0;
    int my_node = (warp < T && lane < 28) ? __ldg(tt.node + warp * 7 + (lane >> 2)) : 0;
    for (long long t = warp; t < T; t += nwarps) {
        const long long tn = t + nwarps;
        const int nx_leaf = (tn < T && lane < 8) ? __ldg(tt.leaf + tn * 8 + lane) : 0;
        const int nx_node = (tn < T && lane < 28) ? __ldg(tt.node + tn * 7 + (lane >> 2)) : 0;
        Gate<float> g[7];
        float pq[4];
        tree_gates_of(tt, my_node, lane, wmode, g, pq);
        const float *row[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) row[k] = x + (long long)__shfl_sync(0xffffffffu, my_leaf, k) * B;
        my_leaf = nx_leaf, my_node = nx_node;
        for (long long b0 = (long long)lane * V; b0 < B; b0 += 32 * V) {
            float a[8][V], r[V];
#pragma unroll
            for (int k = 0; k < 8; ++k) vload<float, V>(row[k] + b0, a[k]);
#pragma unroll
            for (int e = 0; e < V; ++e) {
                const float g0 = gate_eval<float>(g[0], a[0][e], a[1][e]), g1 = gate_eval<float>(g[1], a[2][e], a[3][e]);
                const float g2 = gate_eval<float>(g[2], a[4][e], a[5][e]), g3 = gate_eval<float>(g[3], a[6][e], a[7][e]);
                r[e] = gate_eval<float>(g[6], gate_eval<float>(g[4], g0, g1), gate_eval<float>(g[5], g2, g3));
            }
            vstore<float, V>(y + t * B + b0, r);
        }
    }
}

// Forward of the trees when they feed GroupSum: the class sums directly, without the activation [T][B] (nothing but the
// class sums reads it in a training step).  Block (part, class): its 8 warps share the trees of one part of one class
// (tree i of the part goes to warp i % 8), a lane adds up the outputs of its samples over the warp's trees in tree order, the
// 8 warps' sums are added in warp order: partial[(part * k + class) * B + b], the layout group_sum_ce_sample_kernel reads.
template <int TR>
__global__ void __launch_bounds__(256, TR <= 2 ? 3 : 2) logic_tree_fwd_sum_kernel(const float *__restrict__ x, TreeTables tt, float *__restrict__ partial,
                                                                 long long T, long long B, int k, int wmode)
{
    __shared__ float red[8][TR * 128];
    const int lane = threadIdx.x & 31, wv = threadIdx.x >> 5;
    const int cls = blockIdx.y, part = blockIdx.x, parts = gridDim.x;
    const long long S = T / k;
    const long long t_lo = cls * S + S * part / parts, t_hi = cls * S + S * (part + 1) / parts;
    float acc[TR][4];
#pragma unroll
    for (int tr = 0; tr < TR; ++tr)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[tr][e] = 0.f;
    const long long t0 = t_lo + wv;
    int my_leaf = (t0 < t_hi && lane < 8) ? __ldg(tt.leaf + t0 * 8 + lane) : 0;   // index tables one tree ahead
    int my_node = (t0 < t_hi && lane < 28) ? __ldg(tt.node + t0 * 7 + (lane >> 2)) : 0;
    for (long long t = t0; t < t_hi; t += 8) {
        const long long tn = t + 8;
        const int nx_leaf = (tn < t_hi && lane < 8) ? __ldg(tt.leaf + tn * 8 + lane) : 0;
        const int nx_node = (tn < t_hi && lane < 28) ? __ldg(tt.node + tn * 7 + (lane >> 2)) : 0;
        Gate<float> g[7];
        float pq[4];
        tree_gates_of(tt, my_node, lane, wmode, g, pq);
        const float *row[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) row[q] = x + (long long)__shfl_sync(0xffffffffu, my_leaf, q) * B;
        my_leaf = nx_leaf, my_node = nx_node;
#pragma unroll
        for (int tr = 0; tr < TR; ++tr) {
            const long long b0 = ((long long)tr * 32 + lane) * 4;
            if (b0 < B) {
                float a[8][4];
#pragma unroll
                for (int q = 0; q < 8; ++q) vload<float, 4>(row[q] + b0, a[q]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float g0 = gate_eval<float>(g[0], a[0][e], a[1][e]), g1 = gate_eval<float>(g[1], a[2][e], a[3][e]);
                    const float g2 = gate_eval<float>(g[2], a[4][e], a[5][e]), g3 = gate_eval<float>(g[3], a[6][e], a[7][e]);
                    acc[tr][e] += gate_eval<float>(g[6], gate_eval<float>(g[4], g0, g1), gate_eval<float>(g[5], g2, g3));
                }
            }
        }
    }
#pragma unroll
    for (int tr = 0; tr < TR; ++tr)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[wv][(tr * 32 + lane) * 4 + e] = acc[tr][e];
    __syncthreads();
    for (int i = threadIdx.x; i < TR * 128; i += 256) {
        if (i < B) {
            float t = red[0][i];
#pragma unroll
            for (int w = 1; w < 8; ++w) t += red[w][i];
            partial[((long long)part * k + cls) * B + i] = t;
        }
    }
}

// HEAD: the upstream gradient is not a tensor [T][B] but the GroupSum + cross-entropy head's d loss / d score [B][k]:
// tree t belongs to class t / S and gy[t][b] = dscore[b][class] / (tau / scale), exactly what group_sum_bwd_kernel would
// have written -- the [T][B] gradient is then neither written nor read.
struct TreeHead {
    const float *dscore, *scale; // scale: the scalar gradient that reaches the loss, on the device
    int k;
    unsigned S;                  // trees per class
    float tau;
};

template <int V, bool HEAD>
__global__ void __launch_bounds__(128, 3) logic_tree_bwd_kernel(const float *__restrict__ x, TreeTables tt, const float *__restrict__ gy,
                                                             float *__restrict__ tapgrad, float *__restrict__ gw0, float *__restrict__ gw1,
                                                             float *__restrict__ gw2, long long T, long long B, int wmode, TreeHead head)
{
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    // 128-thread blocks, three per SM: 168 registers, nothing spilled (at 256 threads x 2 blocks the limit of 128 registers
    // spilled 144 bytes).  The index tables are fetched one tree ahead, as in the forward kernel.
    int my_leaf = (warp < T && lane < 8) ? __ldg(tt.leaf + warp * 8 + lane) : 0;
    int my_node = (warp < T && lane < 28) ? __ldg(tt.node + warp * 7 + (lane >> 2)) : 0;
    for (long long t = warp; t < T; t += nwarps) {
        const long long tn = t + nwarps;
        const int nx_leaf = (tn < T && lane < 8) ? __ldg(tt.leaf + tn * 8 + lane) : 0;
        const int nx_node = (tn < T && lane < 28) ? __ldg(tt.node + tn * 7 + (lane >> 2)) : 0;
        Gate<float> g[7];
        float pq[4]; // the lane's four mixture entries, kept for the soft-max Jacobian at the end
        tree_gates_of(tt, my_node, lane, wmode, g, pq);
        const float *row[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) row[k] = x + (long long)__shfl_sync(0xffffffffu, my_leaf, k) * B;
        float bs[28];
#pragma unroll
        for (int i = 0; i < 28; ++i) bs[i] = 0.f;
        for (long long b0 = (long long)lane * V; b0 < B; b0 += 32 * V) {
            float a[8][V], dz[V], dg[4][V];
#pragma unroll
            for (int k = 0; k < 8; ++k) vload<float, V>(row[k] + b0, a[k]);
            if (HEAD) {
                const float taus = head.tau / __ldg(head.scale);
                const float *ds = head.dscore + b0 * head.k + (unsigned)t / head.S;
#pragma unroll
                for (int e = 0; e < V; ++e) dz[e] = __ldg(ds + e * head.k) / taus;
            } else {
                vload<float, V>(gy + t * B + b0, dz);
            }
#pragma unroll
            for (int e = 0; e < V; ++e) {
                const float g0 = gate_eval<float>(g[0], a[0][e], a[1][e]), g1 = gate_eval<float>(g[1], a[2][e], a[3][e]);
                const float g2 = gate_eval<float>(g[2], a[4][e], a[5][e]), g3 = gate_eval<float>(g[3], a[6][e], a[7][e]);
                const float t0 = gate_eval<float>(g[4], g0, g1), t1 = gate_eval<float>(g[5], g2, g3);
                const float d = dz[e];
                const float dt0 = d * gate_da<float>(g[6], t1), dt1 = d * gate_db<float>(g[6], t0);
                dg[0][e] = dt0 * gate_da<float>(g[4], g1), dg[1][e] = dt0 * gate_db<float>(g[4], g0);
                dg[2][e] = dt1 * gate_da<float>(g[5], g3), dg[3][e] = dt1 * gate_db<float>(g[5], g2);
                bs[16] = fmaf(dt0, g0 * g1, bs[16]), bs[17] = fmaf(dt0, g0, bs[17]), bs[18] = fmaf(dt0, g1, bs[18]), bs[19] += dt0;
                bs[20] = fmaf(dt1, g2 * g3, bs[20]), bs[21] = fmaf(dt1, g2, bs[21]), bs[22] = fmaf(dt1, g3, bs[22]), bs[23] += dt1;
                bs[24] = fmaf(d, t0 * t1, bs[24]), bs[25] = fmaf(d, t0, bs[25]), bs[26] = fmaf(d, t1, bs[26]), bs[27] += d;
            }
            // leaf gradients pair by pair, stored at once so that they do not occupy registers
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                float ta[V], tb[V];
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    const float x0 = a[2 * p][e], x1 = a[2 * p + 1][e], d = dg[p][e];
                    ta[e] = d * gate_da<float>(g[p], x1), tb[e] = d * gate_db<float>(g[p], x0);
                    bs[4 * p] = fmaf(d, x0 * x1, bs[4 * p]), bs[4 * p + 1] = fmaf(d, x0, bs[4 * p + 1]);
                    bs[4 * p + 2] = fmaf(d, x1, bs[4 * p + 2]), bs[4 * p + 3] += d;
                }
                vstore<float, V>(tapgrad + (t * 8 + 2 * p) * B + b0, ta);
                vstore<float, V>(tapgrad + (t * 8 + 2 * p + 1) * B + b0, tb);
            }
        }
        // batch totals: a transposed butterfly leaves total i on lane i, i.e. basis sum k = lane & 3 of gate lane >> 2 on
        // the lane that owns entries 4k..4k+3 of that gate; the quad then finishes the gate's 16 gradients together
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = i < 28 ? bs[i] : 0.f;
#pragma unroll
        for (int half = 16; half >= 1; half >>= 1) {
            const bool upper = (lane & half) != 0;
#pragma unroll
            for (int i = 0; i < half; ++i) {
                const float keep = upper ? v[i + half] : v[i];
                const float send = upper ? v[i] : v[i + half];
                v[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
            }
        }
        float s4[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) s4[k] = __shfl_sync(0xffffffffu, v[0], (lane & ~3) + k);
        const float(&p)[4] = pq;
        const long long n = my_node;
        my_leaf = nx_leaf, my_node = nx_node;
        const int q = lane & 3;
        const float q3 = (float)(q >> 1), q2 = (float)(q & 1);
        const float base = (q3 - q2) * s4[0] - q3 * s4[1] + (q2 - q3) * s4[2] + q3 * s4[3];
        float gr[4] = {base, base + s4[0], base + (s4[1] - s4[0]), base + s4[1]}; // entry i adds (i & 1) s0 + (i >> 1) (s1 - s0)
        if (wmode == CLB_W_SOFTMAX) {
            const float dot = quad_sum((p[0] * gr[0] + p[1] * gr[1]) + (p[2] * gr[2] + p[3] * gr[3]));
#pragma unroll
            for (int i = 0; i < 4; ++i) gr[i] = p[i] * (gr[i] - dot);
        }
        if (lane < 28) {
            const int gi = lane >> 2;
            float *out = (gi < 4 ? gw0 : gi < 6 ? gw1 : gw2) + n * 16 + 4 * q;
#pragma unroll
            for (int i = 0; i < 4; ++i) out[i] = gr[i];
        }
    }
}

// gx[f][b] = sum over the entries e of feature f of rows[list[e]][b]  (rows = tapgrad, list = leaf slots t*8+k)
template <int V>
__global__ void __launch_bounds__(256) row_segment_sum_kernel(const float *__restrict__ rows, const int64_t *__restrict__ start,
                                                              const int32_t *__restrict__ list, float *__restrict__ gx, long long F,
                                                              long long B)
{
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long f = warp; f < F; f += nwarps) {
        const long long lo = start[f], hi = start[f + 1];
        for (long long bb = 0; bb < B; bb += 32 * V) { // uniform over the warp: the shuffles below need every lane
            const long long b0 = bb + (long long)lane * V;
            const bool in = b0 < B;
            float acc[V];
#pragma unroll
            for (int k = 0; k < V; ++k) acc[k] = 0.f;
            for (long long c0 = lo; c0 < hi; c0 += 32) {
                const int mine = c0 + lane < hi ? __ldg(list + c0 + lane) : 0;
                const int n = (int)min((long long)32, hi - c0);
                for (int i0 = 0; i0 < n; i0 += 4) {
                    float v[4][V];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int r = __shfl_sync(0xffffffffu, mine, min(i0 + u, n - 1));
                        if (in) {
                            vload<float, V>(rows + (long long)r * B + b0, v[u]);
                        } else {
#pragma unroll
                            for (int k = 0; k < V; ++k) v[u][k] = 0.f;
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (i0 + u < n)
#pragma unroll
                            for (int k = 0; k < V; ++k) acc[k] += v[u][k];
                }
            }
            if (in)
                vstore<float, V>(gx + f * B + b0, acc);
        }
    }
}

} // namespace clb

using namespace clb;
using namespace clb_host;

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int logic_grid(long long units_of_warps)
{
    long long blocks = (units_of_warps + 7) / 8; // 8 warps per block
    const long long cap = (long long)sm_count() * 8 * 4;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

extern "C" int clb_logic_fwd(const void *x, const int64_t *a, const int64_t *b, const void *w, void *y, int64_t in_dim,
                             int64_t out_dim, int64_t B, int wmode, int dtype, void *stream)
{
    if (!x || !a || !b || !w || !y || in_dim <= 0 || out_dim < 0 || B < 0 || wmode < 0 || wmode > 2) return CLB_ERR_ARG;
    if (out_dim == 0 || B == 0) return CLB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int grid = logic_grid((out_dim + 1) / 2);
    if (dtype == CLB_F32) {
        if (B % 4 == 0 && aligned16(x) && aligned16(y))
            CLB_TRACED("logic_fwd_kernel", st, logic_fwd_kernel<float, 4><<<grid, 256, 0, st>>>((const float *)x, a, b, (const float *)w, (float *)y, out_dim, B, wmode));
        else
            CLB_TRACED("logic_fwd_kernel", st, logic_fwd_kernel<float, 1><<<grid, 256, 0, st>>>((const float *)x, a, b, (const float *)w, (float *)y, out_dim, B, wmode));
    } else if (dtype == CLB_F64) {
        CLB_TRACED("logic_fwd_kernel", st, logic_fwd_kernel<double, 1><<<grid, 256, 0, st>>>((const double *)x, a, b, (const double *)w, (double *)y, out_dim, B, wmode));
    } else
        return CLB_ERR_ARG;
    return check_launch();
}

extern "C" int clb_logic_bwd_w(const void *x, const int64_t *a, const int64_t *b, const void *w, const void *gy, void *gw,
                               int64_t in_dim, int64_t out_dim, int64_t B, int wmode, int dtype, void *stream)
{
    if (!x || !a || !b || !w || !gy || !gw || in_dim <= 0 || out_dim < 0 || B < 0 || wmode < 0 || wmode > 2) return CLB_ERR_ARG;
    if (out_dim == 0) return CLB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int grid = logic_grid((out_dim + 1) / 2);
    if (dtype == CLB_F32) {
        if (B % 4 == 0 && aligned16(x) && aligned16(gy))
            CLB_TRACED("logic_bwd_w_kernel", st, logic_bwd_w_kernel<float, 4><<<grid, 256, 0, st>>>((const float *)x, a, b, (const float *)w, (const float *)gy, (float *)gw, out_dim, B, wmode));
        else
            CLB_TRACED("logic_bwd_w_kernel", st, logic_bwd_w_kernel<float, 1><<<grid, 256, 0, st>>>((const float *)x, a, b, (const float *)w, (const float *)gy, (float *)gw, out_dim, B, wmode));
    } else if (dtype == CLB_F64) {
        CLB_TRACED("logic_bwd_w_kernel", st, logic_bwd_w_kernel<double, 1><<<grid, 256, 0, st>>>((const double *)x, a, b, (const double *)w, (const double *)gy, (double *)gw, out_dim, B, wmode));
    } else
        return CLB_ERR_ARG;
    return check_launch();
}

extern "C" int clb_logic_bwd_x(const void *x, const int64_t *a, const int64_t *b, const void *w, const void *gy, void *gx,
                               const int64_t *start, const int64_t *consumers, int64_t in_dim, int64_t out_dim, int64_t B,
                               int wmode, int dtype, void *stream)
{
    if (!x || !a || !b || !w || !gy || !gx || !start || !consumers || in_dim <= 0 || out_dim < 0 || B < 0 || wmode < 0 || wmode > 2)
        return CLB_ERR_ARG;
    if (B == 0) return CLB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const bool vec = dtype == CLB_F32 && B % 4 == 0 && aligned16(x) && aligned16(gy) && aligned16(gx);
    const int V = vec ? 4 : 1;
    // features per warp: about 32 consumer entries per unit (one feature when the fan-out 2*out/in is wide)
    long long fpu = out_dim > 0 ? (16 * in_dim + out_dim - 1) / out_dim : 1;
    if (fpu > 32) fpu = 32;
    if (fpu < 1) fpu = 1;
    while (fpu > 1 && (in_dim + fpu - 1) / fpu < (long long)sm_count() * 8 * 8) fpu /= 2; // keep enough units to occupy the GPU
    const long long funits = (in_dim + fpu - 1) / fpu;
    // split the batch when there are too few units to occupy the GPU
    long long splits = 1;
    const long long max_splits = (B + 32LL * V * 4 - 1) / (32LL * V * 4);
    while (funits * splits < (long long)sm_count() * 8 * 8 && splits < max_splits) splits *= 2;
    if (splits > max_splits) splits = max_splits;
    const int grid = logic_grid(funits * splits);
    if (out_dim > 0x7fffffffLL || in_dim > 0x7fffffffLL) return CLB_ERR_SHAPE; // consumer and row indices travel as 32-bit shuffles
    // vector slots a lane needs for its share of a split: 1, 2 or 4 at a time
    const long long span = ((B + splits * 32 * V - 1) / (splits * 32 * V));
    const int slots = span <= 1 ? 1 : span <= 2 ? 2 : 4;
#define CLB_BWD_X(T, VV, SS)                                                                                                     \
    logic_bwd_x_kernel<T, VV, SS><<<grid, 256, 0, st>>>((const T *)x, a, b, (const T *)w, (const T *)gy, (T *)gx, start, consumers, \
                                                        in_dim, out_dim, B, wmode, (int)splits, (int)fpu)
    clb_host::TraceScope trace_scope("logic_bwd_x_kernel", st);
    if (dtype == CLB_F32) {
        if (vec) {
            if (slots == 1) CLB_BWD_X(float, 4, 1);
            else if (slots == 2) CLB_BWD_X(float, 4, 2);
            else CLB_BWD_X(float, 4, 4);
        } else {
            if (slots == 1) CLB_BWD_X(float, 1, 1);
            else if (slots == 2) CLB_BWD_X(float, 1, 2);
            else CLB_BWD_X(float, 1, 4);
        }
    } else if (dtype == CLB_F64) {
        if (slots == 1) CLB_BWD_X(double, 1, 1);
        else if (slots == 2) CLB_BWD_X(double, 1, 2);
        else CLB_BWD_X(double, 1, 4);
    } else
        return CLB_ERR_ARG;
#undef CLB_BWD_X
    return check_launch();
}

static int group_sum_parts(long long S) { return S >= 8 * kGroupSumParts ? kGroupSumParts : 1; }

extern "C" size_t clb_group_sum_scratch_bytes(int64_t F, int64_t B, int k, int dtype)
{
    if (F <= 0 || B <= 0 || k <= 0 || F % k) return 0;
    return (size_t)group_sum_parts(F / k) * (size_t)k * (size_t)B * (dtype == CLB_F64 ? 8 : 4);
}

extern "C" int clb_group_sum_fwd(const void *y, void *out, void *scratch, size_t scratch_bytes, int64_t F, int64_t B, int k, double tau,
                                 int dtype, void *stream)
{
    if (!y || !out || F < 0 || B < 0 || k <= 0 || tau == 0.0 || (dtype != CLB_F32 && dtype != CLB_F64)) return CLB_ERR_ARG;
    if (F % k) return CLB_ERR_SHAPE;
    if (B == 0) return CLB_OK;
    if (F == 0) return CLB_ERR_SHAPE;
    if (!scratch || scratch_bytes < clb_group_sum_scratch_bytes(F, B, k, dtype)) return CLB_ERR_SCRATCH;
    const long long S = F / k;
    const int parts = group_sum_parts(S);
    if (k > 65535) return CLB_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid((unsigned)((B + 31) / 32), (unsigned)k, (unsigned)parts);
    const int fb = (int)((B * k + 255) / 256);
    if (dtype == CLB_F32) {
        CLB_TRACED("group_sum_partial_kernel", st, group_sum_partial_kernel<float><<<grid, 256, 0, st>>>((const float *)y, (float *)scratch, S, B, k));
        CLB_TRACED("group_sum_finalize_kernel", st, group_sum_finalize_kernel<float><<<fb, 256, 0, st>>>((const float *)scratch, (float *)out, B, k, parts, (float)tau));
    } else {
        CLB_TRACED("group_sum_partial_kernel", st, group_sum_partial_kernel<double><<<grid, 256, 0, st>>>((const double *)y, (double *)scratch, S, B, k));
        CLB_TRACED("group_sum_finalize_kernel", st, group_sum_finalize_kernel<double><<<fb, 256, 0, st>>>((const double *)scratch, (double *)out, B, k, parts, tau));
    }
    return check_launch(2);
}

extern "C" int clb_group_sum_ce(const float *y, const int64_t *labels, float *scores, float *dscore, float *loss, void *scratch,
                                size_t scratch_bytes, int64_t F, int64_t B, int k, double tau, void *stream)
{
    if (!y || !labels || !dscore || !loss || F <= 0 || B <= 0 || k <= 0 || tau == 0.0) return CLB_ERR_ARG;
    if (F % k || k > 32) return CLB_ERR_SHAPE;
    if (!scratch || scratch_bytes < clb_group_sum_scratch_bytes(F, B, k, CLB_F32)) return CLB_ERR_SCRATCH;
    const long long S = F / k;
    const int parts = group_sum_parts(S);
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid((unsigned)((B + 31) / 32), (unsigned)k, (unsigned)parts);
    CLB_TRACED("group_sum_partial_kernel", st, group_sum_partial_kernel<float><<<grid, 256, 0, st>>>(y, (float *)scratch, S, B, k));
    CLB_TRACED("group_sum_ce_sample_kernel", st,
               group_sum_ce_sample_kernel<<<(unsigned)((B + 7) / 8), 256, 0, st>>>((float *)scratch, labels, scores, dscore, B, k, parts, (float)tau));
    CLB_TRACED("group_sum_loss_mean_kernel", st, group_sum_loss_mean_kernel<<<1, 256, 0, st>>>((const float *)scratch, loss, B));
    return check_launch(3);
}

extern "C" int clb_transpose_f32(const float *in, float *out, int64_t rows, int64_t cols, void *stream)
{
    if (!in || !out || rows < 0 || cols < 0 || in == out) return CLB_ERR_ARG;
    if (rows == 0 || cols == 0) return CLB_OK;
    const long long gx = (cols + 31) / 32, gy = (rows + 31) / 32;
    if (gy > 65535 || gx > 0x7fffffffLL) return CLB_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    CLB_TRACED("transpose_f32_kernel", st, transpose_f32_kernel<<<dim3((unsigned)gx, (unsigned)gy), 256, 0, st>>>(in, out, rows, cols));
    return check_launch();
}

extern "C" int clb_adam_step(float *p, const float *g, float *m, float *v, int64_t n, double lr, double beta1, double beta2, double eps,
                             double weight_decay, int64_t step, int decoupled, void *stream)
{
    if (!p || !g || !m || !v || n < 0 || step < 1 || beta1 < 0 || beta1 >= 1 || beta2 < 0 || beta2 >= 1) return CLB_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15)
        return CLB_ERR_ARG;
    if (n == 0) return CLB_OK;
    const double bc1 = 1.0 - std::pow(beta1, (double)step), bc2 = 1.0 - std::pow(beta2, (double)step);
    cudaStream_t st = (cudaStream_t)stream;
    long long blocks = ((n >> 2) + 255) / 256;
    const long long cap = (long long)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    CLB_TRACED("adam_step_kernel", st,
               adam_step_kernel<<<(unsigned)blocks, 256, 0, st>>>(p, g, m, v, n, (float)lr, (float)beta1, (float)beta2, (float)eps, (float)weight_decay,
                                                                  (float)(lr / bc1), (float)std::sqrt(bc2), decoupled));
    return check_launch();
}

extern "C" int clb_group_sum_bwd_scaled(const void *gout, const void *scale, void *gy, int64_t F, int64_t B, int k, double tau, int dtype,
                                        void *stream);
extern "C" int clb_group_sum_bwd(const void *gout, void *gy, int64_t F, int64_t B, int k, double tau, int dtype, void *stream)
{
    return clb_group_sum_bwd_scaled(gout, nullptr, gy, F, B, k, tau, dtype, stream);
}

extern "C" int clb_group_sum_bwd_scaled(const void *gout, const void *scale, void *gy, int64_t F, int64_t B, int k, double tau, int dtype,
                                        void *stream)
{
    if (!gout || !gy || F < 0 || B < 0 || k <= 0 || tau == 0.0 || (dtype != CLB_F32 && dtype != CLB_F64)) return CLB_ERR_ARG;
    if (F % k) return CLB_ERR_SHAPE;
    if (B == 0 || F == 0) return CLB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const long long S = F / k;
    if (k > 65535) return CLB_ERR_SHAPE;
    long long chunks = ((long long)sm_count() * 16 + k - 1) / k; // about sixteen blocks per SM in all
    if (chunks > S) chunks = S;
    dim3 grid((unsigned)chunks, (unsigned)k);
    if (dtype == CLB_F32)
        CLB_TRACED("group_sum_bwd_kernel", st, group_sum_bwd_kernel<float><<<grid, 256, 0, st>>>((const float *)gout, (const float *)scale, (float *)gy, S, B, k, (float)tau));
    else
        CLB_TRACED("group_sum_bwd_kernel", st, group_sum_bwd_kernel<double><<<grid, 256, 0, st>>>((const double *)gout, (const double *)scale, (double *)gy, S, B, k, tau));
    return check_launch();
}

// ---- fused flat layers (training) ------------------------------------------------------------------
static bool tree_args_ok(const void *x, const int32_t *leaf, const int32_t *node, const void *w0, const void *w1, const void *w2, int64_t T,
                         int64_t B, int wmode)
{
    return x && leaf && node && w0 && w1 && w2 && T >= 0 && B >= 0 && wmode >= 0 && wmode <= 2;
}

extern "C" int clb_logic_tree_fwd(const float *x, const int32_t *leaf, const int32_t *node, const float *w0, const float *w1, const float *w2,
                                  float *y, int64_t T, int64_t B, int wmode, void *stream)
{
    if (!tree_args_ok(x, leaf, node, w0, w1, w2, T, B, wmode) || !y) return CLB_ERR_ARG;
    if (T == 0 || B == 0) return CLB_OK;
    TreeTables tt{leaf, node, {w0, w1, w2}};
    const int grid = logic_grid(T);
    cudaStream_t st = (cudaStream_t)stream;
    if (B % 4 == 0 && aligned16(x) && aligned16(y))
        CLB_TRACED("logic_tree_fwd_kernel", st, logic_tree_fwd_kernel<4><<<grid, 256, 0, st>>>(x, tt, y, T, B, wmode));
    else
        CLB_TRACED("logic_tree_fwd_kernel", st, logic_tree_fwd_kernel<1><<<grid, 256, 0, st>>>(x, tt, y, T, B, wmode));
    return check_launch();
}

// tapgrad: scratch of T*8*B floats.  gw0/gw1/gw2 must be zeroed by the caller: neurons no tree uses keep zero.
// start int64 [in_dim + 1], list int32 [T*8]: the leaf slots (t*8 + k) grouped by the input feature they read.
// parts of a class for the fused forward + class sums: enough blocks to fill the GPU a few times over
static int tree_sum_parts(int64_t T, int k)
{
    long long parts = ((long long)sm_count() * 4 + k - 1) / k;
    const long long most = T / k / 8; // at least eight trees (one per warp) per part
    if (parts > most) parts = most;
    return (int)(parts < 1 ? 1 : parts);
}

extern "C" size_t clb_logic_tree_fwd_ce_scratch_bytes(int64_t T, int64_t B, int k)
{
    if (T <= 0 || B <= 0 || k <= 0 || T % k) return 0;
    return (size_t)tree_sum_parts(T, k) * (size_t)k * (size_t)B * sizeof(float);
}

extern "C" int clb_logic_tree_fwd_ce(const float *x, const int32_t *leaf, const int32_t *node, const float *w0, const float *w1,
                                     const float *w2, const int64_t *labels, float *dscore, float *loss, void *scratch,
                                     size_t scratch_bytes, int64_t T, int64_t B, int k, double tau, int wmode, void *stream)
{
    if (!tree_args_ok(x, leaf, node, w0, w1, w2, T, B, wmode) || !labels || !dscore || !loss || k <= 0 || tau == 0.0) return CLB_ERR_ARG;
    if (T <= 0 || B <= 0 || T % k || k > 32 || B % 4 || B > 512 || !aligned16(x) || T / k > 0x7fffffffLL) return CLB_ERR_SHAPE;
    if (!scratch || scratch_bytes < clb_logic_tree_fwd_ce_scratch_bytes(T, B, k)) return CLB_ERR_SCRATCH;
    TreeTables tt{leaf, node, {w0, w1, w2}};
    cudaStream_t st = (cudaStream_t)stream;
    const int parts = tree_sum_parts(T, k);
    const dim3 grid((unsigned)parts, (unsigned)k);
    float *partial = (float *)scratch;
    if (B <= 128)
        CLB_TRACED("logic_tree_fwd_sum_kernel", st, logic_tree_fwd_sum_kernel<1><<<grid, 256, 0, st>>>(x, tt, partial, T, B, k, wmode));
    else if (B <= 256)
        CLB_TRACED("logic_tree_fwd_sum_kernel", st, logic_tree_fwd_sum_kernel<2><<<grid, 256, 0, st>>>(x, tt, partial, T, B, k, wmode));
    else
        CLB_TRACED("logic_tree_fwd_sum_kernel", st, logic_tree_fwd_sum_kernel<4><<<grid, 256, 0, st>>>(x, tt, partial, T, B, k, wmode));
    CLB_TRACED("group_sum_ce_sample_kernel", st,
               group_sum_ce_sample_kernel<<<(unsigned)((B + 7) / 8), 256, 0, st>>>(partial, labels, nullptr, dscore, B, k, parts, (float)tau));
    CLB_TRACED("group_sum_loss_mean_kernel", st, group_sum_loss_mean_kernel<<<1, 256, 0, st>>>(partial, loss, B));
    return check_launch(3);
}

static int logic_tree_bwd_impl(const float *x, const int32_t *leaf, const int32_t *node, const float *w0, const float *w1, const float *w2,
                               const float *gy, const TreeHead *head, float *tapgrad, float *gw0, float *gw1, float *gw2, float *gx,
                               const int64_t *start, const int32_t *list, int64_t in_dim, int64_t T, int64_t B, int wmode, void *stream)
{
    if (!tree_args_ok(x, leaf, node, w0, w1, w2, T, B, wmode) || (!gy && !head) || !tapgrad || !gw0 || !gw1 || !gw2 || in_dim <= 0) return CLB_ERR_ARG;
    if (gx && (!start || !list)) return CLB_ERR_ARG;
    if (T * 8 > 0x7fffffffLL) return CLB_ERR_SHAPE;
    if (B == 0) return CLB_OK;
    TreeTables tt{leaf, node, {w0, w1, w2}};
    cudaStream_t st = (cudaStream_t)stream;
    const bool vec = B % 4 == 0 && aligned16(x) && (head || aligned16(gy)) && aligned16(tapgrad) && (!gx || aligned16(gx));
    const TreeHead none{nullptr, nullptr, 1, 1u, 1.f};
    int launched = 0;
    if (T > 0) {
        const int grid = 2 * logic_grid(T);
        if (head && vec)
            CLB_TRACED("logic_tree_bwd_kernel", st, logic_tree_bwd_kernel<4, true><<<grid, 128, 0, st>>>(x, tt, gy, tapgrad, gw0, gw1, gw2, T, B, wmode, *head));
        else if (head)
            CLB_TRACED("logic_tree_bwd_kernel", st, logic_tree_bwd_kernel<1, true><<<grid, 128, 0, st>>>(x, tt, gy, tapgrad, gw0, gw1, gw2, T, B, wmode, *head));
        else if (vec)
            CLB_TRACED("logic_tree_bwd_kernel", st, logic_tree_bwd_kernel<4, false><<<grid, 128, 0, st>>>(x, tt, gy, tapgrad, gw0, gw1, gw2, T, B, wmode, none));
        else
            CLB_TRACED("logic_tree_bwd_kernel", st, logic_tree_bwd_kernel<1, false><<<grid, 128, 0, st>>>(x, tt, gy, tapgrad, gw0, gw1, gw2, T, B, wmode, none));
        ++launched;
    }
    if (gx) {
        if (vec)
            CLB_TRACED("row_segment_sum_kernel", st, row_segment_sum_kernel<4><<<logic_grid(in_dim), 256, 0, st>>>(tapgrad, start, list, gx, in_dim, B));
        else
            CLB_TRACED("row_segment_sum_kernel", st, row_segment_sum_kernel<1><<<logic_grid(in_dim), 256, 0, st>>>(tapgrad, start, list, gx, in_dim, B));
        ++launched;
    }
    return check_launch(launched);
}

extern "C" int clb_logic_tree_bwd(const float *x, const int32_t *leaf, const int32_t *node, const float *w0, const float *w1, const float *w2,
                                  const float *gy, float *tapgrad, float *gw0, float *gw1, float *gw2, float *gx, const int64_t *start,
                                  const int32_t *list, int64_t in_dim, int64_t T, int64_t B, int wmode, void *stream)
{
    if (!gy) return CLB_ERR_ARG;
    return logic_tree_bwd_impl(x, leaf, node, w0, w1, w2, gy, nullptr, tapgrad, gw0, gw1, gw2, gx, start, list, in_dim, T, B, wmode, stream);
}

extern "C" int clb_logic_tree_bwd_scores(const float *x, const int32_t *leaf, const int32_t *node, const float *w0, const float *w1,
                                         const float *w2, const float *dscore, const float *scale, int k, double tau, float *tapgrad,
                                         float *gw0, float *gw1, float *gw2, float *gx, const int64_t *start, const int32_t *list,
                                         int64_t in_dim, int64_t T, int64_t B, int wmode, void *stream)
{
    if (!dscore || !scale || k <= 0 || tau == 0.0) return CLB_ERR_ARG;
    if (T % k) return CLB_ERR_SHAPE;
    const TreeHead head{dscore, scale, k, (unsigned)(T / k > 0 ? T / k : 1), (float)tau};
    return logic_tree_bwd_impl(x, leaf, node, w0, w1, w2, nullptr, &head, tapgrad, gw0, gw1, gw2, gx, start, list, in_dim, T, B, wmode, stream);
}
