// ConvLogic block kernels: fused (gather -> 4 -> 2 -> 1 gates -> 2x2 max pool) and stand-alone
// first level, forward and backward.  General-shape path (any stride / padding / kernel window /
// image size, fp32 and fp64); the shape-specialised fp32 forward lives in convtree_fast.cu.
//
// Layouts (all contiguous): x [N,Ci,H,W]; fused y [N,C,Hp,Wp] with Hp = Ho/2; split y [N,C,Ho,Wo,4].
// One thread block works on ONE output channel c at a time, so the 7 gates (4 coefficients each,
// see clb_common.cuh) and the 8 tap offsets are block-uniform values kept in shared memory.
//
// Backward design (deterministic, no floating-point atomics):
//   * input gradient: a block owns the gradient tile of `nb` images x `cg` consecutive input channels
//     in shared memory and walks, in ascending order, the output channels that have a tap in those
//     channels.  For one (output channel, tap) the map output position -> input pixel is a
//     translation, hence injective, so all threads can add their contribution with a plain
//     read-modify-write; a block barrier separates the 8 taps.  The order of additions into any
//     pixel is therefore fixed: (channel ascending, tap ascending).
//   * gate gradient: every thread accumulates the 4 basis sums of each gate in registers over its
//     share of (image, position), then warp shuffles + one shared-memory stage give a per-block
//     partial; a second kernel adds the partials in a fixed order and applies K^T (and, for
//     CLB_W_SOFTMAX, the soft-max Jacobian).
#include "clb_common.cuh"

#include <mutex>

namespace clb {

struct ConvShape {
    int N, Ci, H, W, C, Ho, Wo, sh, sw, ph, pw;
};

template <typename T> struct BlockGates {
    Gate<T> g[7];
    Tap tap[8];
};

// Threads 0..ngates-1 build the gates of channel c, threads 32..39 the taps.  Caller syncs.
template <typename T>
__device__ __forceinline__ void load_channel(BlockGates<T> &bg, const T *__restrict__ w, const int32_t *__restrict__ sel,
                                             int c, int ngates, int wmode, int ph, int pw)
{
    const int t = threadIdx.x;
    if (t < ngates) bg.g[t] = gate_load<T>(w + ((size_t)c * ngates + t) * 16, wmode);
    if (t >= 32 && t < 40) bg.tap[t - 32] = unpack_tap(sel[c * 8 + (t - 32)], ph, pw);
}

template <typename T>
__device__ __forceinline__ T tap_value(const T *__restrict__ ximg, const Tap &tp, int oy, int ox, const ConvShape &s)
{
    const int iy = oy * s.sh + tp.dy, ix = ox * s.sw + tp.dx;
    if ((unsigned)iy < (unsigned)s.H && (unsigned)ix < (unsigned)s.W) return __ldg(ximg + ((size_t)tp.ch * s.H + iy) * s.W + ix);
    return T(0);
}

template <typename T> struct Chain {
    T a[8], g[4], t[2], z;
};

template <typename T>
__device__ __forceinline__ void eval_chain(Chain<T> &ch, const BlockGates<T> &bg, const T *__restrict__ ximg, int oy, int ox,
                                           const ConvShape &s, bool full)
{
#pragma unroll
    for (int k = 0; k < 8; ++k) ch.a[k] = tap_value<T>(ximg, bg.tap[k], oy, ox, s);
#pragma unroll
    for (int p = 0; p < 4; ++p) ch.g[p] = gate_eval<T>(bg.g[p], ch.a[2 * p], ch.a[2 * p + 1]);
    if (full) {
        ch.t[0] = gate_eval<T>(bg.g[4], ch.g[0], ch.g[1]);
        ch.t[1] = gate_eval<T>(bg.g[5], ch.g[2], ch.g[3]);
        ch.z = gate_eval<T>(bg.g[6], ch.t[0], ch.t[1]);
    }
}

// ---------------------------------------------------------------------------------------- forward
// grid (chunks of windows, C); thread <-> pooled window (n, py, px), px fastest.
template <typename T>
__global__ void __launch_bounds__(256) convtree_fwd_kernel(const T *__restrict__ x, const T *__restrict__ w,
                                                           const int32_t *__restrict__ sel, T *__restrict__ y,
                                                           uint8_t *__restrict__ amax, T *__restrict__ x2, T *__restrict__ x3,
                                                           int32_t *__restrict__ idx, ConvShape s, int wmode)
{
    __shared__ BlockGates<T> bg;
    const int c = blockIdx.y;
    load_channel<T>(bg, w, sel, c, 7, wmode, s.ph, s.pw);
    __syncthreads();
    const int Hp = s.Ho / 2, Wp = s.Wo / 2, I = Hp * Wp;
    const long long total = (long long)s.N * I;
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < total; j += (long long)gridDim.x * blockDim.x) {
        const int n = (int)(j / I), rem = (int)(j % I);
        const int py = rem / Wp, px = rem % Wp;
        const T *ximg = x + (size_t)n * s.Ci * s.H * s.W;
        T best = T(0);
        int bd = 0;
#pragma unroll
        for (int d = 0; d < 4; ++d) {
            const int oy = 2 * py + (d >> 1), ox = 2 * px + (d & 1);
            Chain<T> ch;
            eval_chain<T>(ch, bg, ximg, oy, ox, s, true);
            if (x2 != nullptr) {
                const size_t pos = (((size_t)n * s.C + c) * s.Ho + oy) * s.Wo + ox;
#pragma unroll
                for (int p = 0; p < 4; ++p) x2[pos * 4 + p] = ch.g[p];
                x3[pos * 2] = ch.t[0];
                x3[pos * 2 + 1] = ch.t[1];
            }
            if (d == 0 || ch.z > best) { // strict '>' in scan order keeps the first maximum
                best = ch.z;
                bd = d;
            }
        }
        const size_t o = ((size_t)n * s.C + c) * I + rem;
        y[o] = best;
        if (amax != nullptr) amax[o] = (uint8_t)bd;
        if (idx != nullptr) idx[o] = (2 * py + (bd >> 1)) * s.Wo + 2 * px + (bd & 1);
    }
}

// Forward for layers with many input channels and small images (fp32, at most 256 pooled windows per
// image, no intermediates): grid (parts, C); the block size is a multiple of the windows per image, so a
// thread keeps ONE pooled window for its whole life and only the image advances.  The 8 tap offsets of
// the window's first position and the in-bounds flags of all 4 x 8 (position, tap) pairs are computed
// once per thread; per image a tap costs a predicate and one cached global load.  An output channel
// reads only the (normally two) input channels its taps name, so staging whole images is pointless here.
__global__ void __launch_bounds__(256) convtree_fwd_win_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                               const int32_t *__restrict__ sel, float *__restrict__ y,
                                                               uint8_t *__restrict__ amax, ConvShape s, int wmode)
{
    __shared__ BlockGates<float> bg;
    const int c = blockIdx.y;
    load_channel<float>(bg, w, sel, c, 7, wmode, s.ph, s.pw);
    __syncthreads();
    const int Wp = s.Wo / 2, I = (s.Ho / 2) * Wp;
    const int ipb = blockDim.x / I;
    const int lane_img = threadIdx.x / I, win = threadIdx.x - lane_img * I;
    const int py = win / Wp, px = win - py * Wp;
    const int HW = s.H * s.W;
    int base[8];
    unsigned valid = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const Tap tp = bg.tap[k];
        const int iy0 = 2 * py * s.sh + tp.dy, ix0 = 2 * px * s.sw + tp.dx;
        base[k] = tp.ch * HW + iy0 * s.W + ix0;
#pragma unroll
        for (int d = 0; d < 4; ++d) {
            const int iy = iy0 + (d >> 1) * s.sh, ix = ix0 + (d & 1) * s.sw;
            if ((unsigned)iy < (unsigned)s.H && (unsigned)ix < (unsigned)s.W) valid |= 1u << (d * 8 + k);
        }
    }
    Gate<float> g[7];
#pragma unroll
    for (int i = 0; i < 7; ++i) g[i] = bg.g[i];
    const int n_lo = (int)((long long)s.N * blockIdx.x / gridDim.x), n_hi = (int)((long long)s.N * (blockIdx.x + 1) / gridDim.x);
    if (lane_img >= ipb) return;
    const int rowstep = s.sh * s.W;
    for (int n = n_lo + lane_img; n < n_hi; n += ipb) {
        const float *ximg = x + (size_t)n * s.Ci * HW;
        float best = 0.f;
        int bd = 0;
#pragma unroll
        for (int d = 0; d < 4; ++d) {
            const float *p = ximg + ((d >> 1) ? rowstep : 0) + ((d & 1) ? s.sw : 0);
            const unsigned vm = valid >> (d * 8);
            float a[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) a[k] = ((vm >> k) & 1u) ? __ldg(p + base[k]) : 0.f;
            const float g0 = gate_eval<float>(g[0], a[0], a[1]), g1 = gate_eval<float>(g[1], a[2], a[3]);
            const float g2 = gate_eval<float>(g[2], a[4], a[5]), g3 = gate_eval<float>(g[3], a[6], a[7]);
            const float z = gate_eval<float>(g[6], gate_eval<float>(g[4], g0, g1), gate_eval<float>(g[5], g2, g3));
            if (d == 0 || z > best) { // strict '>' in scan order keeps the first maximum
                best = z;
                bd = d;
            }
        }
        const size_t o = ((size_t)n * s.C + c) * I + win;
        y[o] = best;
        if (amax != nullptr) amax[o] = (uint8_t)bd;
    }
}

// grid (chunks of positions, C); thread <-> conv position (n, oy, ox); writes the 4 first-level gates.
template <typename T>
__global__ void __launch_bounds__(256) conv_fwd_kernel(const T *__restrict__ x, const T *__restrict__ w,
                                                       const int32_t *__restrict__ sel, T *__restrict__ y, ConvShape s, int wmode)
{
    __shared__ BlockGates<T> bg;
    const int c = blockIdx.y;
    load_channel<T>(bg, w, sel, c, 4, wmode, s.ph, s.pw);
    __syncthreads();
    const int P = s.Ho * s.Wo;
    const long long total = (long long)s.N * P;
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < total; j += (long long)gridDim.x * blockDim.x) {
        const int n = (int)(j / P), rem = (int)(j % P);
        Chain<T> ch;
        eval_chain<T>(ch, bg, x + (size_t)n * s.Ci * s.H * s.W, rem / s.Wo, rem % s.Wo, s, false);
        T *o = y + (((size_t)n * s.C + c) * P + rem) * 4;
#pragma unroll
        for (int p = 0; p < 4; ++p) o[p] = ch.g[p];
    }
}

// ------------------------------------------------------------------------------- backward helpers
// Position and upstream gradients of work item j (a pooled window in fused mode, a conv position in
// split mode) of channel c.  Returns false when j is out of range.
template <typename T, bool FUSED> struct Upstream {
    int oy, ox;
    T dg[4]; // gradient arriving at the 4 first-level gate outputs
};

template <typename T, bool FUSED>
__device__ __forceinline__ void backprop_item(Upstream<T, FUSED> &u, Chain<T> &ch, const BlockGates<T> &bg,
                                              const T *__restrict__ ximg, const T *__restrict__ gy, const uint8_t *__restrict__ amax,
                                              size_t item /* (n*C + c)*items_per_image + rem */, int rem, const ConvShape &s,
                                              T *acc /* 28 or 16 basis sums, may be null */)
{
    if (FUSED) {
        const int Wp = s.Wo / 2;
        const int py = rem / Wp, px = rem % Wp;
        int bd;
        if (amax != nullptr) {
            bd = amax[item];
        } else {
            T best = T(0);
            bd = 0;
#pragma unroll
            for (int d = 0; d < 4; ++d) {
                eval_chain<T>(ch, bg, ximg, 2 * py + (d >> 1), 2 * px + (d & 1), s, true);
                if (d == 0 || ch.z > best) {
                    best = ch.z;
                    bd = d;
                }
            }
        }
        u.oy = 2 * py + (bd >> 1);
        u.ox = 2 * px + (bd & 1);
        eval_chain<T>(ch, bg, ximg, u.oy, u.ox, s, true);
        const T dz = gy[item];
        const T dt0 = dz * gate_da<T>(bg.g[6], ch.t[1]);
        const T dt1 = dz * gate_db<T>(bg.g[6], ch.t[0]);
        u.dg[0] = dt0 * gate_da<T>(bg.g[4], ch.g[1]);
        u.dg[1] = dt0 * gate_db<T>(bg.g[4], ch.g[0]);
        u.dg[2] = dt1 * gate_da<T>(bg.g[5], ch.g[3]);
        u.dg[3] = dt1 * gate_db<T>(bg.g[5], ch.g[2]);
        if (acc != nullptr) {
            acc[24] = fma_t<T>(dz, ch.t[0] * ch.t[1], acc[24]);
            acc[25] = fma_t<T>(dz, ch.t[0], acc[25]);
            acc[26] = fma_t<T>(dz, ch.t[1], acc[26]);
            acc[27] += dz;
            acc[16] = fma_t<T>(dt0, ch.g[0] * ch.g[1], acc[16]);
            acc[17] = fma_t<T>(dt0, ch.g[0], acc[17]);
            acc[18] = fma_t<T>(dt0, ch.g[1], acc[18]);
            acc[19] += dt0;
            acc[20] = fma_t<T>(dt1, ch.g[2] * ch.g[3], acc[20]);
            acc[21] = fma_t<T>(dt1, ch.g[2], acc[21]);
            acc[22] = fma_t<T>(dt1, ch.g[3], acc[22]);
            acc[23] += dt1;
        }
    } else {
        u.oy = rem / s.Wo;
        u.ox = rem % s.Wo;
        eval_chain<T>(ch, bg, ximg, u.oy, u.ox, s, false);
#pragma unroll
        for (int p = 0; p < 4; ++p) u.dg[p] = gy[item * 4 + p];
    }
    if (acc != nullptr) {
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const T a = ch.a[2 * p], b = ch.a[2 * p + 1], d = u.dg[p];
            acc[4 * p + 0] = fma_t<T>(d, a * b, acc[4 * p + 0]);
            acc[4 * p + 1] = fma_t<T>(d, a, acc[4 * p + 1]);
            acc[4 * p + 2] = fma_t<T>(d, b, acc[4 * p + 2]);
            acc[4 * p + 3] += d;
        }
    }
}

// --------------------------------------------------------------------------- backward: input grad
// grid (ceil(N / nb), G); dynamic shared memory: tile [nb][cg][H][W] of T, then 2 BlockGates<T>.
template <typename T, bool FUSED>
__global__ void __launch_bounds__(256) conv_bwd_x_kernel(const T *__restrict__ gy, const T *__restrict__ x, const T *__restrict__ w,
                                                         const int32_t *__restrict__ sel, const uint8_t *__restrict__ amax,
                                                         T *__restrict__ gx, const int32_t *__restrict__ grp_start,
                                                         const int32_t *__restrict__ grp_list, int cg, int nb, ConvShape s, int wmode)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int HW = s.H * s.W;
    T *tile = reinterpret_cast<T *>(smem_raw);
    const size_t tile_elems = (size_t)nb * cg * HW;
    BlockGates<T> *bgs = reinterpret_cast<BlockGates<T> *>(smem_raw + ((tile_elems * sizeof(T) + 15) / 16) * 16);

    const int g = blockIdx.y, n0 = blockIdx.x * nb;
    const int nimg = min(nb, s.N - n0);
    const int ch0 = g * cg;
    for (size_t i = threadIdx.x; i < tile_elems; i += blockDim.x) tile[i] = T(0);

    const int items = FUSED ? (s.Ho / 2) * (s.Wo / 2) : s.Ho * s.Wo; // per image and channel
    const int total = nimg * items;
    const int lo = grp_start[g], hi = grp_start[g + 1];
    constexpr int NG = FUSED ? 7 : 4;
    for (int li = lo; li < hi; ++li) {
        const int c = grp_list[li];
        BlockGates<T> &bg = bgs[(li - lo) & 1];
        load_channel<T>(bg, w, sel, c, NG, wmode, s.ph, s.pw);
        __syncthreads(); // publishes bg; also orders the tile zero-fill / previous channel's last tap
        for (int base = 0; base < total; base += blockDim.x) {
            const int j = base + threadIdx.x;
            const bool live = j < total;
            Upstream<T, FUSED> u;
            Chain<T> chn;
            int img = 0;
            if (live) {
                img = j / items;
                const int rem = j % items;
                const int n = n0 + img;
                backprop_item<T, FUSED>(u, chn, bg, x + (size_t)n * s.Ci * HW, gy, amax, ((size_t)n * s.C + c) * items + rem, rem, s,
                                        nullptr);
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const Tap tp = bg.tap[k];
                const int chl = tp.ch - ch0;
                if (chl >= 0 && chl < cg) { // block-uniform
                    if (live) {
                        const int iy = u.oy * s.sh + tp.dy, ix = u.ox * s.sw + tp.dx;
                        if ((unsigned)iy < (unsigned)s.H && (unsigned)ix < (unsigned)s.W) {
                            const T other = chn.a[k ^ 1];
                            const T d = (k & 1) ? gate_db<T>(bg.g[k >> 1], other) : gate_da<T>(bg.g[k >> 1], other);
                            T *cell = tile + ((size_t)img * cg + chl) * HW + iy * s.W + ix;
                            *cell = fma_t<T>(d, u.dg[k >> 1], *cell);
                        }
                    }
                    __syncthreads();
                }
            }
        }
    }
    __syncthreads();
    const int nch = min(cg, s.Ci - ch0);
    for (size_t i = threadIdx.x; i < (size_t)nimg * nch * HW; i += blockDim.x) {
        const int img = (int)(i / ((size_t)nch * HW));
        const size_t r = i % ((size_t)nch * HW);
        const int chl = (int)(r / HW), p = (int)(r % HW);
        gx[((size_t)(n0 + img) * s.Ci + ch0 + chl) * HW + p] = tile[((size_t)img * cg + chl) * HW + p];
    }
}

// Faster variant of the kernel above for the fused block in fp32 with the arg-max available and at most
// 256 (image, window) items per block, i.e. the layers behind the first one of a stack (many input
// channels, small images).  Differences: a thread keeps one (image, window) for its whole life; the
// gates and taps of the next few listed channels are prepared by all threads at once instead of one
// channel at a time; gy / arg-max are fetched one channel ahead; the gradient tile uses the
// parity-class layout (see convtree_fast.cu) so that arg-max dependent addresses spread over the banks.
// Same accumulation order as above: deterministic, no atomics.
constexpr int kGrpBatch = 8;

struct alignas(16) GrpRec {
    float g[28];
    int xo[8];    // channel*H*W + ty*W + tx: offset of the tap's pixel from the conv position's pixel
    int ty[8];    // tap row / col displacement (pad subtracted), for the bounds test
    int tx[8];
    int cbase[8]; // float offset of the tap's cell in the gradient tile for a window's first position, from the
                  // window's own offset; -1 when the tap's channel is not in the block's group
    int dA[8];    // added when the arg-max is in the window's second row / column (parity-class layout)
    int dB[8];
};

__global__ void __launch_bounds__(256, 3) convtree_bwd_x_grp_kernel(const float *__restrict__ gy, const float *__restrict__ x,
                                                                    const float *__restrict__ w, const int32_t *__restrict__ sel,
                                                                    const uint8_t *__restrict__ amax, float *__restrict__ gx,
                                                                    const int32_t *__restrict__ grp_start,
                                                                    const int32_t *__restrict__ grp_list, int cg, int nb, ConvShape s,
                                                                    int wmode)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    GrpRec *rec = reinterpret_cast<GrpRec *>(smem_raw);
    float *tile = reinterpret_cast<float *>(smem_raw + sizeof(GrpRec) * kGrpBatch);

    const int HW = s.H * s.W, Hh = (s.H + 1) / 2, Wh = (s.W + 1) / 2, PL = Hh * Wh;
    const int Wp = s.Wo / 2, I = (s.Ho / 2) * Wp;
    const int tid = threadIdx.x;
    const int g = blockIdx.y, n0 = blockIdx.x * nb;
    const int nimg = min(nb, s.N - n0);
    const int ch0 = g * cg;
    const int tile_elems = nb * cg * 4 * PL;
    for (int i = tid; i < tile_elems; i += blockDim.x) tile[i] = 0.f;

    const int img = tid / I, win = tid - img * I;
    const bool live = img < nimg;
    const int py = win / Wp, px = win - py * Wp;
    const int n = n0 + img;
    // stride-1 layers only (checked by the launcher): conv position (2py+dy, 2px+dx) reads pixel (position + tap)
    const float *xwin = x + (size_t)n * s.Ci * HW + 2 * py * s.W + 2 * px;
    float *twin = tile + img * cg * 4 * PL + py * Wh + px;
    const size_t obase = ((size_t)n * s.C) * I + win; // + c * I
    auto fy = [&](int t) { return (t & 1) * 2 * PL + (t >> 1) * Wh; };
    auto fx = [&](int t) { return (t & 1) * PL + (t >> 1); };

    const int lo = grp_start[g], hi = grp_start[g + 1];
    for (int l0 = lo; l0 < hi; l0 += kGrpBatch) {
        const int cnt = min(kGrpBatch, hi - l0);
        __syncthreads(); // the previous batch's records are no longer read
        for (int i = tid; i < cnt * 7; i += blockDim.x) {
            const int e = i / 7, gi = i - e * 7;
            const Gate<float> gt = gate_load<float>(w + ((size_t)grp_list[l0 + e] * 7 + gi) * 16, wmode);
            float *o = rec[e].g + gi * 4;
            o[0] = gt.k1, o[1] = gt.ka, o[2] = gt.kb, o[3] = gt.kab;
        }
        for (int i = tid; i < cnt * 8; i += blockDim.x) {
            const int e = i >> 3, k = i & 7;
            const Tap tp = unpack_tap(sel[grp_list[l0 + e] * 8 + k], s.ph, s.pw);
            rec[e].xo[k] = tp.ch * HW + tp.dy * s.W + tp.dx;
            rec[e].ty[k] = tp.dy;
            rec[e].tx[k] = tp.dx;
            const int chl = tp.ch - ch0;
            rec[e].cbase[k] = (chl >= 0 && chl < cg) ? chl * 4 * PL + fy(tp.dy) + fx(tp.dx) : -1;
            rec[e].dA[k] = fy(tp.dy + 1) - fy(tp.dy);
            rec[e].dB[k] = fx(tp.dx + 1) - fx(tp.dx);
        }
        __syncthreads();

        // Software pipeline over the batch: gy / arg-max are fetched two channels ahead and the 8 taps of the
        // next channel are gathered (arg-max -> address -> load is a chain of global latencies) while the
        // current channel is evaluated and accumulated.
        float dz1 = 0.f, dz2 = 0.f, a1[8];
        int bd1 = 0, bd2 = 0;
        unsigned vm1 = 0;
        auto gather = [&](int e, int bd, float(&a)[8], unsigned &vm) {
            const GrpRec &r = rec[e];
            const int dyi = bd >> 1, dxi = bd & 1;
            const int oy = 2 * py + dyi, ox = 2 * px + dxi;
            const float *xpos = xwin + dyi * s.W + dxi;
            vm = 0;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int4 xo4 = reinterpret_cast<const int4 *>(r.xo)[q], ty4 = reinterpret_cast<const int4 *>(r.ty)[q];
                const int4 tx4 = reinterpret_cast<const int4 *>(r.tx)[q];
                const int xo[4] = {xo4.x, xo4.y, xo4.z, xo4.w}, ty[4] = {ty4.x, ty4.y, ty4.z, ty4.w}, tx[4] = {tx4.x, tx4.y, tx4.z, tx4.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const bool v = (unsigned)(oy + ty[j]) < (unsigned)s.H && (unsigned)(ox + tx[j]) < (unsigned)s.W;
                    a[q * 4 + j] = v ? __ldg(xpos + xo[j]) : 0.f;
                    vm |= (v ? 1u : 0u) << (q * 4 + j);
                }
            }
        };
#pragma unroll
        for (int k = 0; k < 8; ++k) a1[k] = 0.f;
        if (live) {
            const size_t o = obase + (size_t)grp_list[l0] * I;
            dz1 = __ldg(gy + o);
            bd1 = amax[o];
            gather(0, bd1, a1, vm1);
            if (cnt > 1) {
                const size_t o2 = obase + (size_t)grp_list[l0 + 1] * I;
                dz2 = __ldg(gy + o2);
                bd2 = amax[o2];
            }
        }
        for (int e = 0; e < cnt; ++e) {
            const float dz = dz1;
            const int bd = bd1;
            const unsigned vm = vm1;
            float a[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) a[k] = a1[k];
            dz1 = dz2;
            bd1 = bd2;
            if (live && e + 1 < cnt) gather(e + 1, bd1, a1, vm1);
            if (live && e + 2 < cnt) {
                const size_t o = obase + (size_t)grp_list[l0 + e + 2] * I;
                dz2 = __ldg(gy + o);
                bd2 = amax[o];
            }
            const GrpRec &r = rec[e];
            int cb[8];
            {
                const int4 c0 = reinterpret_cast<const int4 *>(r.cbase)[0], c1 = reinterpret_cast<const int4 *>(r.cbase)[1];
                cb[0] = c0.x, cb[1] = c0.y, cb[2] = c0.z, cb[3] = c0.w, cb[4] = c1.x, cb[5] = c1.y, cb[6] = c1.z, cb[7] = c1.w;
            }
            float tg[8];
            int cell[8];
            if (live) {
                const int dyi = bd >> 1, dxi = bd & 1;
#pragma unroll
                for (int k = 0; k < 8; ++k) cell[k] = ((vm >> k) & 1u) ? 0 : -1;
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    if (cb[4 * q] >= 0 || cb[4 * q + 1] >= 0 || cb[4 * q + 2] >= 0 || cb[4 * q + 3] >= 0) { // block-uniform
                        const int4 a4 = reinterpret_cast<const int4 *>(r.dA)[q], b4 = reinterpret_cast<const int4 *>(r.dB)[q];
                        const int dA[4] = {a4.x, a4.y, a4.z, a4.w}, dB[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int k = q * 4 + j;
                            if (cell[k] == 0) cell[k] = cb[k] + dyi * dA[j] + dxi * dB[j];
                        }
                    }
                }
                Gate<float> gg[7];
                const float4 *gp = reinterpret_cast<const float4 *>(r.g);
#pragma unroll
                for (int i = 0; i < 7; ++i) {
                    const float4 q = gp[i];
                    gg[i].k1 = q.x, gg[i].ka = q.y, gg[i].kb = q.z, gg[i].kab = q.w;
                }
                const float g0 = gate_eval<float>(gg[0], a[0], a[1]), g1 = gate_eval<float>(gg[1], a[2], a[3]);
                const float g2 = gate_eval<float>(gg[2], a[4], a[5]), g3 = gate_eval<float>(gg[3], a[6], a[7]);
                const float t0 = gate_eval<float>(gg[4], g0, g1), t1 = gate_eval<float>(gg[5], g2, g3);
                const float dt0 = dz * gate_da<float>(gg[6], t1), dt1 = dz * gate_db<float>(gg[6], t0);
                const float dg0 = dt0 * gate_da<float>(gg[4], g1), dg1 = dt0 * gate_db<float>(gg[4], g0);
                const float dg2 = dt1 * gate_da<float>(gg[5], g3), dg3 = dt1 * gate_db<float>(gg[5], g2);
                tg[0] = dg0 * gate_da<float>(gg[0], a[1]), tg[1] = dg0 * gate_db<float>(gg[0], a[0]);
                tg[2] = dg1 * gate_da<float>(gg[1], a[3]), tg[3] = dg1 * gate_db<float>(gg[1], a[2]);
                tg[4] = dg2 * gate_da<float>(gg[2], a[5]), tg[5] = dg2 * gate_db<float>(gg[2], a[4]);
                tg[6] = dg3 * gate_da<float>(gg[3], a[7]), tg[7] = dg3 * gate_db<float>(gg[3], a[6]);
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (cb[k] >= 0) { // block-uniform: taps outside the group cost no barrier
                    if (live && cell[k] >= 0) twin[cell[k]] += tg[k];
                    __syncthreads();
                }
            }
        }
    }
    __syncthreads();
    const int nch = min(cg, s.Ci - ch0);
    for (int i = tid; i < nimg * nch * HW; i += blockDim.x) {
        const int col = i % s.W;
        int q = i / s.W;
        const int row = q % s.H;
        q /= s.H;
        const int chl = q % nch, im = q / nch;
        gx[((size_t)(n0 + im) * s.Ci + ch0 + chl) * HW + row * s.W + col] =
            tile[(im * cg + chl) * 4 * PL + ((row & 1) * 2 + (col & 1)) * PL + (row >> 1) * Wh + (col >> 1)];
    }
}

// Input gradient from precomputed tap gradients (convtree_bwd_w_win_kernel's `tapgrad`): channel-group tiles and
// group lists as in the kernel above, but a listed channel costs only its arg-max byte, the tap gradients of the
// taps that fall into the group and their read-modify-writes; the gate chain is not recomputed and x is not
// read.  The tile is row-major with a zero-weight halo of the padding's width, so an out-of-image tap needs no
// test (its cell is never written out) and a cell is  window offset + tap offset + (dy ? row : 0) + dx.
// Threads of one image only ever touch that image's tile and a warp owns whole images (WPT windows per lane
// when an image has more than 32), so the ordering between the taps needs __syncwarp only.  Same fixed
// accumulation order as the kernels above: deterministic, no atomics.
constexpr int kScatBatch = 16;

template <int WPT>
__global__ void __launch_bounds__(256, 3) convtree_bwd_x_scatter_kernel(const float *__restrict__ tapgrad, const int32_t *__restrict__ sel,
                                                                        const uint8_t *__restrict__ amax, float *__restrict__ gx,
                                                                        const int32_t *__restrict__ grp_start,
                                                                        const int32_t *__restrict__ grp_list, int cg, int nb, ConvShape s)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    int(*cbase)[8] = reinterpret_cast<int(*)[8]>(smem_raw); // [kScatBatch][8]: tap cell offset inside the image's tile, -1 = other group
    float *tile = reinterpret_cast<float *>(smem_raw + sizeof(int) * 8 * kScatBatch);

    const int HW = s.H * s.W, PW = s.W + 2 * s.pw, PP = (s.H + 2 * s.ph) * PW;
    const int Wp = s.Wo / 2, I = (s.Ho / 2) * Wp;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = blockIdx.y, n0 = blockIdx.x * nb;
    const int nimg = min(nb, s.N - n0);
    const int ch0 = g * cg;
    const int tile_elems = nb * cg * PP;
    for (int i = tid; i < tile_elems; i += blockDim.x) tile[i] = 0.f;

    // a lane's WPT slots: slot = lane + 32*j.  Images of 32 or more windows: the warp's image, window = slot.
    // Smaller images: the warp holds 32*WPT / I of them, image = slot / I, window = slot % I.
    const int ipw = I >= 32 ? 1 : (32 * WPT) / I;
    bool live[WPT];
    int toff[WPT];
    size_t ob[WPT], tb[WPT]; // index of the slot's arg-max byte / first tap gradient for output channel 0
#pragma unroll
    for (int j = 0; j < WPT; ++j) {
        const int slot = lane + 32 * j;
        const int img = I >= 32 ? warp : warp * ipw + slot / I;
        const int win = I >= 32 ? slot : slot % I;
        live[j] = img < nimg && (I >= 32 ? win < I : slot < ipw * I);
        const int py = win / Wp, px = win - py * Wp;
        toff[j] = img * cg * PP + 2 * py * PW + 2 * px;
        ob[j] = ((size_t)(n0 + img) * s.C) * I + win;
        tb[j] = (ob[j] - win) * 8 + win;
    }

    const int lo = grp_start[g], hi = grp_start[g + 1];
    for (int l0 = lo; l0 < hi; l0 += kScatBatch) {
        const int cnt = min(kScatBatch, hi - l0);
        __syncthreads(); // the previous batch's records are no longer read
        for (int i = tid; i < cnt * 8; i += blockDim.x) {
            const int e = i >> 3, k = i & 7;
            const Tap tp = unpack_tap(sel[grp_list[l0 + e] * 8 + k], s.ph, s.pw); // dy, dx: tap offset minus padding
            const int chl = tp.ch - ch0;
            cbase[e][k] = (chl >= 0 && chl < cg) ? chl * PP + (tp.dy + s.ph) * PW + tp.dx + s.pw : -1;
        }
        __syncthreads();
        // software pipeline: the arg-max bytes and the in-group tap gradients of the next listed channel are in flight
        // while this one is added (their addresses do not depend on the arg-max)
        int bd1[WPT];
        float v1[WPT][8];
        auto fetch = [&](int e) {
            const size_t co = (size_t)grp_list[l0 + e] * I;
            const int4 c0 = reinterpret_cast<const int4 *>(cbase[e])[0], c1 = reinterpret_cast<const int4 *>(cbase[e])[1];
            const int cb[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
            for (int j = 0; j < WPT; ++j) {
                bd1[j] = live[j] ? (int)amax[ob[j] + co] : 0;
                const float *t = tapgrad + tb[j] + co * 8;
#pragma unroll
                for (int k = 0; k < 8; ++k, t += I) v1[j][k] = (live[j] && cb[k] >= 0) ? __ldg(t) : 0.f;
            }
        };
        fetch(0);
        for (int e = 0; e < cnt; ++e) {
            int woff[WPT];
            float v[WPT][8];
#pragma unroll
            for (int j = 0; j < WPT; ++j) {
                woff[j] = toff[j] + ((bd1[j] >> 1) ? PW : 0) + (bd1[j] & 1);
#pragma unroll
                for (int k = 0; k < 8; ++k) v[j][k] = v1[j][k];
            }
            const int4 c0 = reinterpret_cast<const int4 *>(cbase[e])[0], c1 = reinterpret_cast<const int4 *>(cbase[e])[1];
            const int cb[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            if (e + 1 < cnt) fetch(e + 1);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (cb[k] < 0) continue; // block-uniform: taps outside the group cost nothing
#pragma unroll
                for (int j = 0; j < WPT; ++j)
                    if (live[j]) tile[woff[j] + cb[k]] += v[j][k];
                __syncwarp();
            }
        }
    }
    __syncthreads();
    const int nch = min(cg, s.Ci - ch0);
    for (int i = tid; i < nimg * nch * HW; i += blockDim.x) {
        const int col = i % s.W;
        int q = i / s.W;
        const int row = q % s.H;
        q /= s.H;
        const int chl = q % nch, im = q / nch;
        gx[((size_t)(n0 + im) * s.Ci + ch0 + chl) * HW + row * s.W + col] = tile[(im * cg + chl) * PP + (row + s.ph) * PW + col + s.pw];
    }
}

// ---------------------------------------------------------------------------- backward: gate grad
// grid (parts, C).  Block `part` covers items [part*per, (part+1)*per) of the N*items range of channel c.
template <typename T, bool FUSED>
__global__ void __launch_bounds__(256) conv_bwd_w_kernel(const T *__restrict__ gy, const T *__restrict__ x, const T *__restrict__ w,
                                                         const int32_t *__restrict__ sel, const uint8_t *__restrict__ amax,
                                                         T *__restrict__ partial /* [parts][C][NB] */, ConvShape s, int wmode)
{
    constexpr int NG = FUSED ? 7 : 4, NB = NG * 4;
    __shared__ BlockGates<T> bg;
    __shared__ T red[8][NB];
    const int c = blockIdx.y;
    load_channel<T>(bg, w, sel, c, NG, wmode, s.ph, s.pw);
    __syncthreads();
    const int items = FUSED ? (s.Ho / 2) * (s.Wo / 2) : s.Ho * s.Wo;
    const long long total = (long long)s.N * items;
    const long long per = (total + gridDim.x - 1) / gridDim.x;
    const long long lo = per * blockIdx.x, hi = min(total, lo + per);
    T acc[NB];
#pragma unroll
    for (int i = 0; i < NB; ++i) acc[i] = T(0);
    const int HW = s.H * s.W;
    for (long long j = lo + threadIdx.x; j < hi; j += blockDim.x) {
        const int n = (int)(j / items), rem = (int)(j % items);
        Upstream<T, FUSED> u;
        Chain<T> chn;
        backprop_item<T, FUSED>(u, chn, bg, x + (size_t)n * s.Ci * HW, gy, amax, ((size_t)n * s.C + c) * items + rem, rem, s, acc);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        const T v = warp_sum<T>(acc[i]);
        if (lane == 0) red[warp][i] = v;
    }
    __syncthreads();
    if (threadIdx.x < NB) {
        T v = T(0);
        for (int wv = 0; wv < (int)(blockDim.x >> 5); ++wv) v += red[wv][threadIdx.x];
        partial[((size_t)blockIdx.x * s.C + c) * NB + threadIdx.x] = v;
    }
}

// Fused block, fp32, arg-max available, at most 256 pooled positions per image: the block size is a
// multiple of the positions per image, so a thread keeps ONE pooled window for its whole life and
// only the image index advances.  Its 8 tap offsets (for the window's first position) and the
// in-bounds flags of the 4 x 8 (position, tap) pairs are computed once; per image a tap costs one
// add, one predicate and one cached global load.  grid (parts, C); block `part` covers images
// [N*part/parts, N*(part+1)/parts).
template <bool TAPGRAD>
__global__ void __launch_bounds__(256, TAPGRAD ? 2 : 1) convtree_bwd_w_win_kernel(const float *__restrict__ gy, const float *__restrict__ x,
                                                                 const float *__restrict__ w, const int32_t *__restrict__ sel,
                                                                 const uint8_t *__restrict__ amax, float *__restrict__ partial,
                                                                 float *__restrict__ tapgrad, ConvShape s, int wmode)
{
    __shared__ BlockGates<float> bg;
    __shared__ float red[8][28];
    const int c = blockIdx.y;
    load_channel<float>(bg, w, sel, c, 7, wmode, s.ph, s.pw);
    __syncthreads();
    const int Wp = s.Wo / 2, I = (s.Ho / 2) * Wp;
    const int ipb = blockDim.x / I; // images per block iteration
    const int lane_img = threadIdx.x / I, win = threadIdx.x - lane_img * I;
    const int py = win / Wp, px = win - py * Wp;
    const int HW = s.H * s.W;
    int base[8];
    unsigned valid = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const Tap tp = bg.tap[k];
        const int iy0 = 2 * py * s.sh + tp.dy, ix0 = 2 * px * s.sw + tp.dx;
        base[k] = tp.ch * HW + iy0 * s.W + ix0;
#pragma unroll
        for (int d = 0; d < 4; ++d) {
            const int iy = iy0 + (d >> 1) * s.sh, ix = ix0 + (d & 1) * s.sw;
            if ((unsigned)iy < (unsigned)s.H && (unsigned)ix < (unsigned)s.W) valid |= 1u << (d * 8 + k);
        }
    }
    Gate<float> g[7];
#pragma unroll
    for (int i = 0; i < 7; ++i) g[i] = bg.g[i];
    float acc[28];
#pragma unroll
    for (int i = 0; i < 28; ++i) acc[i] = 0.f;

    const int n_lo = (int)((long long)s.N * blockIdx.x / gridDim.x), n_hi = (int)((long long)s.N * (blockIdx.x + 1) / gridDim.x);
    const bool active = lane_img < ipb;
    // Software pipeline over this thread's images: the arg-max / gy of image i+2 and the 8 gathered
    // taps of image i+1 are in flight while image i is evaluated (arg-max -> address -> gather are
    // two dependent global-memory latencies otherwise).
    const size_t item_step = (size_t)ipb * s.C * I;
    const size_t x_step = (size_t)ipb * s.Ci * HW;
    int n = n_lo + lane_img;
    size_t item = ((size_t)n * s.C + c) * I + win;
    const float *ximg = x + (size_t)n * s.Ci * HW;
    int bd1 = 0, bd2 = 0;
    float dz1 = 0.f, dz2 = 0.f, a1[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) a1[k] = 0.f;
    auto gather = [&](float(&a)[8], int bd, const float *img) {
        const float *p = img + ((bd >> 1) ? s.sh * s.W : 0) + ((bd & 1) ? s.sw : 0);
        const unsigned vm = valid >> (bd * 8);
#pragma unroll
        for (int k = 0; k < 8; ++k) a[k] = ((vm >> k) & 1u) ? __ldg(p + base[k]) : 0.f;
    };
    if (active && n < n_hi) {
        bd1 = amax[item];
        dz1 = __ldg(gy + item);
        gather(a1, bd1, ximg);
        if (n + ipb < n_hi) {
            bd2 = amax[item + item_step];
            dz2 = __ldg(gy + item + item_step);
        }
    }
    for (; active && n < n_hi; n += ipb) {
        float a[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) a[k] = a1[k];
        const float dz = dz1;
        const size_t item_now = item;
        // advance the pipeline
        item += item_step;
        ximg += x_step;
        bd1 = bd2;
        dz1 = dz2;
        if (n + ipb < n_hi) gather(a1, bd1, ximg);
        if (n + 2 * ipb < n_hi) {
            bd2 = amax[item + item_step];
            dz2 = __ldg(gy + item + item_step);
        }
        const float g0 = gate_eval<float>(g[0], a[0], a[1]), g1 = gate_eval<float>(g[1], a[2], a[3]);
        const float g2 = gate_eval<float>(g[2], a[4], a[5]), g3 = gate_eval<float>(g[3], a[6], a[7]);
        const float t0 = gate_eval<float>(g[4], g0, g1), t1 = gate_eval<float>(g[5], g2, g3);
        const float dt0 = dz * gate_da<float>(g[6], t1), dt1 = dz * gate_db<float>(g[6], t0);
        float dg[4];
        dg[0] = dt0 * gate_da<float>(g[4], g1), dg[1] = dt0 * gate_db<float>(g[4], g0);
        dg[2] = dt1 * gate_da<float>(g[5], g3), dg[3] = dt1 * gate_db<float>(g[5], g2);
        acc[24] = fmaf(dz, t0 * t1, acc[24]), acc[25] = fmaf(dz, t0, acc[25]), acc[26] = fmaf(dz, t1, acc[26]), acc[27] += dz;
        acc[16] = fmaf(dt0, g0 * g1, acc[16]), acc[17] = fmaf(dt0, g0, acc[17]), acc[18] = fmaf(dt0, g1, acc[18]), acc[19] += dt0;
        acc[20] = fmaf(dt1, g2 * g3, acc[20]), acc[21] = fmaf(dt1, g2, acc[21]), acc[22] = fmaf(dt1, g3, acc[22]), acc[23] += dt1;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            acc[4 * p] = fmaf(dg[p], a[2 * p] * a[2 * p + 1], acc[4 * p]);
            acc[4 * p + 1] = fmaf(dg[p], a[2 * p], acc[4 * p + 1]);
            acc[4 * p + 2] = fmaf(dg[p], a[2 * p + 1], acc[4 * p + 2]);
            acc[4 * p + 3] += dg[p];
        }
        if (TAPGRAD) {
            // gradient w.r.t. each of the 8 taps at the arg-max position, [n][c][tap][window]: the input-gradient
            // scatter kernel adds them into the pixels without recomputing the gate chain
            float *t = tapgrad + (item_now - win) * 8 + win;
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                t[(2 * p) * I] = dg[p] * gate_da<float>(g[p], a[2 * p + 1]);
                t[(2 * p + 1) * I] = dg[p] * gate_db<float>(g[p], a[2 * p]);
            }
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < 28; ++i) {
        const float v = warp_sum<float>(acc[i]);
        if (lane == 0) red[warp][i] = v;
    }
    __syncthreads();
    if (threadIdx.x < 28) {
        float v = 0.f;
        for (int wv = 0; wv < (int)((blockDim.x + 31) >> 5); ++wv) v += red[wv][threadIdx.x];
        partial[((size_t)blockIdx.x * s.C + c) * 28 + threadIdx.x] = v;
    }
}

// One thread per gate: adds the per-part basis sums in part order and writes the 16 gradients.
template <typename T>
__global__ void gate_grad_finalize_kernel(const T *__restrict__ partial, const T *__restrict__ w, T *__restrict__ gw, int parts,
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

// ================================================================================== host side ====
using namespace clb;
using namespace clb_host;

static int make_shape(ConvShape &s, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, bool fused)
{
    if (!conv_args_ok(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw)) return CLB_ERR_ARG;
    s = ConvShape{N, Ci, H, W, C, conv_out(H, ph, kh, sh), conv_out(W, pw, kw, sw), sh, sw, ph, pw};
    if (s.Ho <= 0 || s.Wo <= 0) return CLB_ERR_SHAPE;
    if (fused && ((s.Ho & 1) || (s.Wo & 1))) return CLB_ERR_ODD_OUTPUT;
    return CLB_OK;
}

static int grid_x_for(long long total_items, int C)
{
    long long want = (total_items + 255) / 256;
    // enough blocks to fill 148 SMs several times over, without starving each block of work
    long long cap = ((long long)sm_count() * 16 + C - 1) / (C > 0 ? C : 1);
    if (cap < 1) cap = 1;
    if (want > cap) want = cap;
    if (want < 1) want = 1;
    return (int)want;
}

// implemented in convtree_plane.cu; returns CLB_ERR_SHAPE when the shape is outside the plane kernels
int clb_convtree_fwd_plane_f32(const float *x, const float *w, const int32_t *sel, float *y, uint8_t *amax, int N, int Ci, int H, int W,
                               int C, int sh, int sw, int ph, int pw, int kh, int kw, int wmode, cudaStream_t st);
// implemented in convtree_fast.cu; returns CLB_ERR_SHAPE when the shape is outside its fast path
int clb_convtree_fwd_fast_f32(const float *x, const float *w, const int32_t *sel, float *y, uint8_t *amax, int N, int Ci, int H,
                              int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int wmode, cudaStream_t st);

extern "C" int clb_convtree_fwd(const void *x, const void *w, const int32_t *sel, void *y, uint8_t *amax, void *x2, void *x3,
                                int32_t *idx, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw,
                                int wmode, int dtype, void *stream)
{
    const bool sel_unbounded = (wmode & CLB_SEL_UNBOUNDED) != 0;
    const bool y_fm = (wmode & CLB_Y_FEATURE_MAJOR) != 0;
    wmode &= ~(CLB_SEL_UNBOUNDED | CLB_Y_FEATURE_MAJOR);
    ConvShape s;
    int rc = make_shape(s, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, true);
    if (rc) return rc;
    if (!x || !w || !sel || !y || (x2 == nullptr) != (x3 == nullptr) || wmode < 0 || wmode > 2) return CLB_ERR_ARG;
    if (N == 0 || C == 0) return CLB_OK;
    if (C > 65535) return CLB_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    if (y_fm) { // feature-major output: the plane kernels or nothing
        if (dtype != CLB_F32 || x2 || idx || sel_unbounded) return CLB_ERR_SHAPE;
        return clb_convtree_fwd_plane_f32((const float *)x, (const float *)w, sel, (float *)y, amax, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw,
                                          wmode | CLB_Y_FEATURE_MAJOR, st);
    }
    if (dtype == CLB_F32 && !x2 && !idx && !sel_unbounded) {
        rc = clb_convtree_fwd_fast_f32((const float *)x, (const float *)w, sel, (float *)y, amax, N, Ci, H, W, C, sh, sw, ph, pw,
                                       kh, kw, wmode, st);
        if (rc != CLB_ERR_SHAPE) return rc;
    }
    const long long total = (long long)N * (s.Ho / 2) * (s.Wo / 2);
    const int items = (s.Ho / 2) * (s.Wo / 2);
    if (dtype == CLB_F32 && !x2 && !idx && items <= 256) {
        const int threads = (256 / items) * items;
        int parts = (int)(((long long)sm_count() * 20 + C - 1) / C); // about ten waves of two resident blocks per SM
        const int ipb = threads / items;
        if (parts > (N + ipb - 1) / ipb) parts = (N + ipb - 1) / ipb;
        if (parts < 1) parts = 1;
        CLB_TRACED("convtree_fwd_win_kernel", st, convtree_fwd_win_kernel<<<dim3(parts, C), threads, 0, st>>>((const float *)x, (const float *)w, sel, (float *)y, amax, s, wmode));
        return check_launch();
    }
    dim3 grid(grid_x_for(total, C), C);
    if (dtype == CLB_F32)
        CLB_TRACED("convtree_fwd_kernel", st, convtree_fwd_kernel<float><<<grid, 256, 0, st>>>((const float *)x, (const float *)w, sel, (float *)y, amax, (float *)x2,
                                                          (float *)x3, idx, s, wmode));
    else if (dtype == CLB_F64)
        CLB_TRACED("convtree_fwd_kernel", st, convtree_fwd_kernel<double><<<grid, 256, 0, st>>>((const double *)x, (const double *)w, sel, (double *)y, amax,
                                                           (double *)x2, (double *)x3, idx, s, wmode));
    else
        return CLB_ERR_ARG;
    return check_launch();
}

extern "C" int clb_conv_fwd(const void *x, const void *w, const int32_t *sel, void *y, int N, int Ci, int H, int W, int C, int sh,
                            int sw, int ph, int pw, int kh, int kw, int wmode, int dtype, void *stream)
{
    wmode &= ~CLB_SEL_UNBOUNDED;
    ConvShape s;
    int rc = make_shape(s, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, false);
    if (rc) return rc;
    if (!x || !w || !sel || !y || wmode < 0 || wmode > 2) return CLB_ERR_ARG;
    if (N == 0 || C == 0) return CLB_OK;
    if (C > 65535) return CLB_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid(grid_x_for((long long)N * s.Ho * s.Wo, C), C);
    if (dtype == CLB_F32)
        CLB_TRACED("conv_fwd_kernel", st, conv_fwd_kernel<float><<<grid, 256, 0, st>>>((const float *)x, (const float *)w, sel, (float *)y, s, wmode));
    else if (dtype == CLB_F64)
        CLB_TRACED("conv_fwd_kernel", st, conv_fwd_kernel<double><<<grid, 256, 0, st>>>((const double *)x, (const double *)w, sel, (double *)y, s, wmode));
    else
        return CLB_ERR_ARG;
    return check_launch();
}

// ---- input gradient ---------------------------------------------------------------------------
// Shared-memory budget of one block's gradient tile: 4 KiB per warp that works on it, so that about fifty warps
// stay resident per SM.  A small channel group costs nothing extra: an output channel reads two input channels
// and therefore appears in at most two groups' lists whatever the group size.
static const size_t kTileBudgetPerWarp = 4 * 1024;
static const size_t kTileBudgetMax = 200 * 1024;

extern "C" int clb_conv_group_plan(int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int dtype,
                                   int *cg, int *nb)
{
    if (!cg || !nb || (dtype != CLB_F32 && dtype != CLB_F64)) return CLB_ERR_ARG;
    if (!conv_args_ok(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw)) return CLB_ERR_ARG;
    const size_t esz = dtype == CLB_F32 ? 4 : 8;
    // per channel and image: parity-class planes (odd sizes rounded up) or the plane with its padding halo, whichever is larger
    size_t hw = (size_t)4 * ((H + 1) / 2) * ((W + 1) / 2);
    const size_t halo = (size_t)(H + 2 * ph) * (W + 2 * pw);
    if (halo > hw) hw = halo;
    const int Ho = conv_out(H, ph, kh, sh), Wo = conv_out(W, pw, kw, sw);
    if (Ho <= 0 || Wo <= 0) return CLB_ERR_SHAPE;
    if (hw * esz > kTileBudgetMax) return CLB_ERR_SHAPE; // one channel plane must fit in shared memory
    // as many whole images as give at most 256 (image, window) items: a thread then keeps its item
    long long items = (long long)((Ho + 1) / 2) * ((Wo + 1) / 2);
    int n_b = (int)(256 / items);
    if (n_b < 1) n_b = 1;
    if (n_b > (N > 0 ? N : 1)) n_b = N > 0 ? N : 1;
    long long warps = items >= 32 ? n_b : (n_b * items + 63) / 64; // the scatter kernel: a warp per image (or per 64 / items images)
    if (items > 64) warps = 8;                                     // large images: the 256-thread kernels
    if (warps < 2) warps = 2;
    if (warps > 8) warps = 8;
    size_t budget = kTileBudgetPerWarp * (size_t)warps;
    while (n_b > 1 && (size_t)n_b * hw * esz > budget) --n_b;
    if ((size_t)n_b * hw * esz > budget) budget = kTileBudgetMax;
    long long c_g = (long long)(budget / ((size_t)n_b * hw * esz));
    if (c_g < 1) c_g = 1;
    if (c_g > Ci) c_g = Ci;
    *cg = (int)c_g;
    *nb = n_b;
    return CLB_OK;
}

extern "C" int clb_conv_build_groups(const int32_t *sel_host, int C, int Ci, int cg, int32_t *grp_start, int32_t *grp_list,
                                     int list_cap)
{
    if (!sel_host || !grp_start || (!grp_list && list_cap > 0) || C < 0 || Ci <= 0 || cg <= 0) return CLB_ERR_ARG;
    const int G = (Ci + cg - 1) / cg;
    int n = 0;
    for (int g = 0; g < G; ++g) {
        grp_start[g] = n;
        for (int c = 0; c < C; ++c) {
            bool hit = false;
            for (int k = 0; k < 8 && !hit; ++k) {
                const int ch = (sel_host[c * 8 + k] >> 16) & 0xFFFF;
                if (ch >= Ci) return CLB_ERR_ARG; // selection names a channel the input does not have
                hit = ch / cg == g;
            }
            if (hit) {
                if (n >= list_cap) return CLB_ERR_SCRATCH;
                grp_list[n++] = c;
            }
        }
    }
    grp_start[G] = n;
    return n;
}

template <bool FUSED>
static int launch_bwd_x(const void *gy, const void *x, const void *w, const int32_t *sel, const uint8_t *amax, void *gx,
                        const int32_t *grp_start, const int32_t *grp_list, int cg, int nb, int N, int Ci, int H, int W, int C,
                        int sh, int sw, int ph, int pw, int kh, int kw, int wmode, int dtype, void *stream)
{
    wmode &= ~CLB_SEL_UNBOUNDED;
    ConvShape s;
    int rc = make_shape(s, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, FUSED);
    if (rc) return rc;
    if (!gy || !x || !w || !sel || !gx || !grp_start || !grp_list || cg <= 0 || nb <= 0 || wmode < 0 || wmode > 2) return CLB_ERR_ARG;
    if (dtype != CLB_F32 && dtype != CLB_F64) return CLB_ERR_ARG;
    if (N == 0) return CLB_OK;
    const size_t esz = dtype == CLB_F32 ? 4 : 8;
    const size_t tile = (((size_t)nb * cg * H * W * esz + 15) / 16) * 16;
    const size_t bgsz = dtype == CLB_F32 ? sizeof(BlockGates<float>) : sizeof(BlockGates<double>);
    const size_t smem = tile + 2 * bgsz;
    if (smem > 227 * 1024) return CLB_ERR_SHAPE;
    const int G = (Ci + cg - 1) / cg;
    if (G > 65535) return CLB_ERR_SHAPE;
    dim3 grid((N + nb - 1) / nb, G);
    cudaStream_t st = (cudaStream_t)stream;
    const long long items = (long long)(s.Ho / 2) * (s.Wo / 2);
    if (FUSED && dtype == CLB_F32 && amax != nullptr && (long long)nb * items <= 256 && sh == 1 && sw == 1) {
        const int PL = ((H + 1) / 2) * ((W + 1) / 2);
        const size_t smem2 = sizeof(GrpRec) * kGrpBatch + (size_t)nb * cg * 4 * PL * sizeof(float);
        if (smem2 <= 227 * 1024) {
            auto k = convtree_bwd_x_grp_kernel;
            if (clb_host::ensure_dynamic_smem(k, (int)smem2) != cudaSuccess) return check_launch(0);
            CLB_TRACED("convtree_bwd_x_grp_kernel", st, k<<<grid, 256, smem2, st>>>((const float *)gy, (const float *)x, (const float *)w, sel, amax, (float *)gx,
                                                                                     grp_start, grp_list, cg, nb, s, wmode));
            return check_launch();
        }
    }
    if (dtype == CLB_F32) {
        auto k = conv_bwd_x_kernel<float, FUSED>;
        if (clb_host::ensure_dynamic_smem(k, (int)smem) != cudaSuccess) return check_launch();
        CLB_TRACED("conv_bwd_x_kernel", st, k<<<grid, 256, smem, st>>>((const float *)gy, (const float *)x, (const float *)w, sel, amax, (float *)gx, grp_start,
                                                                        grp_list, cg, nb, s, wmode));
    } else {
        auto k = conv_bwd_x_kernel<double, FUSED>;
        if (clb_host::ensure_dynamic_smem(k, (int)smem) != cudaSuccess) return check_launch();
        CLB_TRACED("conv_bwd_x_kernel", st, k<<<grid, 256, smem, st>>>((const double *)gy, (const double *)x, (const double *)w, sel, amax, (double *)gx,
                                                                        grp_start, grp_list, cg, nb, s, wmode));
    }
    return check_launch();
}

size_t clb_convtree_bwd_x_fast_scratch(int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw);
int clb_convtree_bwd_x_fast_f32(const float *gy, const float *x, const float *w, const int32_t *sel, const uint8_t *amax, float *gx,
                                void *scratch, size_t scratch_bytes, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw,
                                int kh, int kw, int wmode, cudaStream_t st);

extern "C" size_t clb_convtree_bwd_x_scratch_bytes(int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw,
                                                   int dtype)
{
    if (dtype != CLB_F32 || !conv_args_ok(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw)) return 0;
    return clb_convtree_bwd_x_fast_scratch(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw);
}

extern "C" int clb_convtree_bwd_x(const void *gy, const void *x, const void *w, const int32_t *sel, const uint8_t *amax, void *gx,
                                  const int32_t *grp_start, const int32_t *grp_list, int cg, int nb, void *scratch,
                                  size_t scratch_bytes, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh,
                                  int kw, int wmode, int dtype, void *stream)
{
    if (dtype == CLB_F32 && !(wmode & CLB_SEL_UNBOUNDED) && scratch && amax && gy && x && w && sel && gx && N > 0 && C > 0 &&
        (wmode & 0xff) <= 2 && conv_args_ok(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw)) {
        const int rc = clb_convtree_bwd_x_fast_f32((const float *)gy, (const float *)x, (const float *)w, sel, amax, (float *)gx, scratch,
                                                   scratch_bytes, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, wmode, (cudaStream_t)stream);
        if (rc != CLB_ERR_SHAPE) return rc;
    }
    return launch_bwd_x<true>(gy, x, w, sel, amax, gx, grp_start, grp_list, cg, nb, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, wmode,
                              dtype, stream);
}

extern "C" int clb_conv_bwd_x(const void *gy, const void *x, const void *w, const int32_t *sel, void *gx, const int32_t *grp_start,
                              const int32_t *grp_list, int cg, int nb, int N, int Ci, int H, int W, int C, int sh, int sw, int ph,
                              int pw, int kh, int kw, int wmode, int dtype, void *stream)
{
    return launch_bwd_x<false>(gy, x, w, sel, nullptr, gx, grp_start, grp_list, cg, nb, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw,
                               wmode, dtype, stream);
}

// ---- gate gradient ----------------------------------------------------------------------------
static int bwd_w_parts(long long total_items, int C)
{
    long long parts = ((long long)sm_count() * 20 + C - 1) / (C > 0 ? C : 1); // about ten waves of two resident blocks per SM
    long long most = total_items / 2048;
    if (parts > most) parts = most;
    if (parts < 1) parts = 1;
    if (parts > 1024) parts = 1024;
    return (int)parts;
}

static size_t bwd_w_scratch(int N, int C, long long items, int ngates, int dtype)
{
    const size_t esz = dtype == CLB_F64 ? 8 : 4;
    return (size_t)bwd_w_parts((long long)N * items, C) * (size_t)C * ngates * 4 * esz;
}

extern "C" size_t clb_convtree_bwd_w_scratch_bytes(int N, int C, int Ho, int Wo, int dtype)
{
    return bwd_w_scratch(N, C, (long long)(Ho / 2) * (Wo / 2), 7, dtype);
}
extern "C" size_t clb_conv_bwd_w_scratch_bytes(int N, int C, int Ho, int Wo, int dtype)
{
    return bwd_w_scratch(N, C, (long long)Ho * Wo, 4, dtype);
}

template <bool FUSED>
static int launch_bwd_w(const void *gy, const void *x, const void *w, const int32_t *sel, const uint8_t *amax, void *gw,
                        void *scratch, size_t scratch_bytes, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw,
                        int kh, int kw, int wmode, int dtype, void *stream)
{
    wmode &= ~CLB_SEL_UNBOUNDED;
    ConvShape s;
    int rc = make_shape(s, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, FUSED);
    if (rc) return rc;
    if (!gy || !x || !w || !sel || !gw || wmode < 0 || wmode > 2) return CLB_ERR_ARG;
    if (dtype != CLB_F32 && dtype != CLB_F64) return CLB_ERR_ARG;
    if (C == 0) return CLB_OK;
    if (C > 65535) return CLB_ERR_SHAPE;
    constexpr int NG = FUSED ? 7 : 4;
    const long long items = FUSED ? (long long)(s.Ho / 2) * (s.Wo / 2) : (long long)s.Ho * s.Wo;
    const int parts = bwd_w_parts((long long)N * items, C);
    const size_t need = bwd_w_scratch(N, C, items, NG, dtype);
    if (!scratch || scratch_bytes < need) return CLB_ERR_SCRATCH;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid(parts, C);
    const long long ngates = (long long)C * NG;
    const int fb = (int)((ngates + 127) / 128);
    if (dtype == CLB_F32 && FUSED && amax != nullptr && items <= 256 && parts <= N) {
        const int threads = (int)((256 / items) * items); // whole images per block iteration
        CLB_TRACED("convtree_bwd_w_win_kernel", st, convtree_bwd_w_win_kernel<false><<<grid, threads, 0, st>>>((const float *)gy, (const float *)x, (const float *)w, sel, amax,
                                                                   (float *)scratch, nullptr, s, wmode));
        CLB_TRACED("gate_grad_finalize_kernel", st, gate_grad_finalize_kernel<float><<<fb, 128, 0, st>>>((const float *)scratch, (const float *)w, (float *)gw, parts, ngates, wmode));
    } else if (dtype == CLB_F32) {
        CLB_TRACED("conv_bwd_w_kernel", st, conv_bwd_w_kernel<float, FUSED><<<grid, 256, 0, st>>>((const float *)gy, (const float *)x, (const float *)w, sel, amax,
                                                               (float *)scratch, s, wmode));
        CLB_TRACED("gate_grad_finalize_kernel", st, gate_grad_finalize_kernel<float><<<fb, 128, 0, st>>>((const float *)scratch, (const float *)w, (float *)gw, parts, ngates, wmode));
    } else {
        CLB_TRACED("conv_bwd_w_kernel", st, conv_bwd_w_kernel<double, FUSED><<<grid, 256, 0, st>>>((const double *)gy, (const double *)x, (const double *)w, sel, amax,
                                                                (double *)scratch, s, wmode));
        CLB_TRACED("gate_grad_finalize_kernel", st, gate_grad_finalize_kernel<double><<<fb, 128, 0, st>>>((const double *)scratch, (const double *)w, (double *)gw, parts, ngates,
                                                              wmode));
    }
    return check_launch(2);
}

extern "C" int clb_convtree_bwd_w(const void *gy, const void *x, const void *w, const int32_t *sel, const uint8_t *amax, void *gw,
                                  void *scratch, size_t scratch_bytes, int N, int Ci, int H, int W, int C, int sh, int sw, int ph,
                                  int pw, int kh, int kw, int wmode, int dtype, void *stream)
{
    return launch_bwd_w<true>(gy, x, w, sel, amax, gw, scratch, scratch_bytes, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, wmode, dtype,
                              stream);
}
extern "C" int clb_conv_bwd_w(const void *gy, const void *x, const void *w, const int32_t *sel, void *gw, void *scratch,
                              size_t scratch_bytes, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh,
                              int kw, int wmode, int dtype, void *stream)
{
    return launch_bwd_w<false>(gy, x, w, sel, nullptr, gw, scratch, scratch_bytes, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, wmode,
                               dtype, stream);
}

// ---- gate gradient of the fused block for callers that must not allocate -----------------------
// Same kernels as clb_convtree_bwd_w; the per-block partial sums live in a fixed array that is part
// of the loaded library image instead of a caller-supplied buffer.
constexpr size_t kStaticScratchBytes = 4u << 20; // 4 MiB, held by every GPU that loads the library
static __device__ __align__(256) unsigned char g_bwd_w_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_scratch_mutex;
void *g_static_scratch_addr[kMaxDevices] = {}; // device address of the array, per device ordinal

// In host code the array's name is only a handle for the runtime; the address a kernel can use has
// to be asked for, once per device, with that device current.
int static_scratch_for_current_device(void **out)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        return CLB_ERR_LAUNCH;
    }
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_addr[dev] == nullptr) {
        void *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_bwd_w_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_last_cuda_error((int)e);
            cudaGetLastError();
            return CLB_ERR_LAUNCH;
        }
        g_static_scratch_addr[dev] = p;
    }
    *out = g_static_scratch_addr[dev];
    return CLB_OK;
}
} // namespace

extern "C" size_t clb_convtree_bwd_w_noalloc_max_bytes(void) { return kStaticScratchBytes; }

extern "C" int clb_convtree_bwd_w_noalloc(const void *gy, const void *x, const void *w, const int32_t *sel, const uint8_t *amax,
                                          void *gw, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw,
                                          int wmode, int dtype, void *stream)
{
    if (!conv_args_ok(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw)) return CLB_ERR_ARG;
    const size_t need = clb_convtree_bwd_w_scratch_bytes(N, C, conv_out(H, ph, kh, sh), conv_out(W, pw, kw, sw), dtype);
    if (need > kStaticScratchBytes) return CLB_ERR_TOO_LARGE;
    void *scratch = nullptr;
    const int rc = static_scratch_for_current_device(&scratch);
    if (rc != CLB_OK) return rc;
    return launch_bwd_w<true>(gy, x, w, sel, amax, gw, scratch, kStaticScratchBytes, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, wmode,
                              dtype, stream);
}

// ---- both gradients of the fused block --------------------------------------------------------
size_t clb_convtree_bwd_fast_scratch(int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int want_gx,
                                     int want_gw);
int clb_convtree_bwd_fast_f32(const float *gy, const float *x, const float *w, const int32_t *sel, const uint8_t *amax, float *gx,
                              float *gw, void *scratch, size_t scratch_bytes, int N, int Ci, int H, int W, int C, int sh, int sw, int ph,
                              int pw, int kh, int kw, int wmode, cudaStream_t st);

// Two-pass backward of the many-channel layers: convtree_bwd_w_win_kernel also writes the tap gradients
// [N][C][8][I] (after its own partial sums in the scratch), convtree_bwd_x_scatter_kernel adds them into gx.
// 0 when the shape does not take that path.
// The batch is walked in slices of S images, pass 1 and pass 2 alternating on ONE tap-gradient buffer of a slice's
// size: when that buffer fits the L2 cache (CLB_TUNE_TAPGRAD_SLICE_BYTES) the second pass finds the tap gradients
// there, and the next slice overwrites them before they were ever written back to HBM.
struct TwoPassPlan {
    int S;        // images per slice
    int slices;
    int parts;    // blocks per output channel and slice in pass 1
    size_t partial_bytes, tapgrad_bytes;
};
static bool two_pass_plan(TwoPassPlan &p, int N, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int want_gx, int dtype)
{
    if (!want_gx || dtype != CLB_F32 || sh != 1 || sw != 1 || N <= 0 || C <= 0 || C > 65535) return false;
    const int Ho = conv_out(H, ph, kh, 1), Wo = conv_out(W, pw, kw, 1);
    if (Ho <= 0 || Wo <= 0 || (Ho & 1) || (Wo & 1)) return false;
    const long long items = (long long)(Ho / 2) * (Wo / 2);
    if (items > 256) return false;
    const long long per_image = (long long)C * 8 * items * (long long)sizeof(float);
    const long long budget = tune_get(CLB_TUNE_TAPGRAD_SLICE_BYTES);
    long long S = N;
    if (budget > 0 && per_image * N > budget) {
        const long long ipb = 256 / items; // images per block iteration of pass 1
        S = budget / per_image / ipb * ipb;
        if (S < ipb) S = ipb;
        if (S > N) S = N;
    }
    p.S = (int)S;
    p.slices = (int)((N + S - 1) / S);
    p.parts = bwd_w_parts(S * items, C);
    if (p.parts > S) return false;
    p.partial_bytes = ((size_t)p.slices * p.parts * C * 28 * sizeof(float) + 255) / 256 * 256;
    p.tapgrad_bytes = (size_t)S * C * 8 * items * sizeof(float);
    return true;
}
static size_t two_pass_scratch(int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int want_gx, int dtype)
{
    (void)Ci;
    TwoPassPlan p;
    if (!two_pass_plan(p, N, H, W, C, sh, sw, ph, pw, kh, kw, want_gx, dtype)) return 0;
    return p.partial_bytes + p.tapgrad_bytes;
}

extern "C" size_t clb_convtree_bwd_scratch_bytes(int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw,
                                                 int want_gx, int want_gw, int dtype)
{
    if (!conv_args_ok(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw)) return 0;
    size_t fast = dtype == CLB_F32 ? clb_convtree_bwd_fast_scratch(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, want_gx, want_gw) : 0;
    size_t general = want_gw ? clb_convtree_bwd_w_scratch_bytes(N, C, conv_out(H, ph, kh, sh), conv_out(W, pw, kw, sw), dtype) : 0;
    const size_t two_pass = two_pass_scratch(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, want_gx, dtype);
    if (two_pass > general) general = two_pass;
    return fast > general ? fast : general;
}

extern "C" int clb_convtree_bwd(const void *gy, const void *x, const void *w, const int32_t *sel, const uint8_t *amax, void *gx, void *gw,
                                const int32_t *grp_start, const int32_t *grp_list, int cg, int nb, void *scratch, size_t scratch_bytes,
                                int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int wmode, int dtype,
                                void *stream)
{
    if (!gx && !gw) return CLB_ERR_ARG;
    if (dtype == CLB_F32 && !(wmode & CLB_SEL_UNBOUNDED) && scratch && amax && gy && x && w && sel && N > 0 && C > 0 &&
        (wmode & 0xff) <= 2 && conv_args_ok(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw)) {
        const int rc = clb_convtree_bwd_fast_f32((const float *)gy, (const float *)x, (const float *)w, sel, amax, (float *)gx, (float *)gw,
                                                 scratch, scratch_bytes, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, wmode, (cudaStream_t)stream);
        if (rc != CLB_ERR_SHAPE) return rc;
    }
    // many input channels, small images: one pass over the windows for the gate sums and the tap gradients, then a scatter
    const size_t tp = (amax && scratch && grp_start && grp_list && cg > 0 && nb > 0 && !(wmode & CLB_SEL_UNBOUNDED) && (wmode & 0xff) <= 2)
                          ? two_pass_scratch(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, gx != nullptr, dtype)
                          : 0;
    if (tp && scratch_bytes >= tp && gy && x && w && sel && conv_args_ok(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw)) {
        ConvShape s;
        if (make_shape(s, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, true) == 0) {
            const long long items = (long long)(s.Ho / 2) * (s.Wo / 2);
            const size_t smem = sizeof(int) * 8 * kScatBatch + (size_t)nb * cg * (H + 2 * ph) * (W + 2 * pw) * sizeof(float);
            const int G = (Ci + cg - 1) / cg;
            TwoPassPlan plan;
            if ((long long)nb * items <= 256 && nb <= 256 && smem <= 227 * 1024 && G <= 65535 &&
                two_pass_plan(plan, N, H, W, C, sh, sw, ph, pw, kh, kw, 1, dtype)) {
                cudaStream_t st = (cudaStream_t)stream;
                float *partial = (float *)scratch;
                float *tapgrad = (float *)((unsigned char *)scratch + plan.partial_bytes);
                const int threads = (int)((256 / items) * items);
                const int wpt = items >= 32 ? (int)((items + 31) / 32) : 2;
                const int ipw = items >= 32 ? 1 : (int)(64 / items);
                const int sthreads = (nb + ipw - 1) / ipw * 32; // a warp per image (or per 64 / items images)
                const size_t HW = (size_t)H * W;
                int launched = 0;
                bool ok = true;
                for (int sl = 0; sl < plan.slices && ok; ++sl) {
                    const int n0 = sl * plan.S;
                    ConvShape ss = s;
                    ss.N = N - n0 < plan.S ? N - n0 : plan.S;
                    const float *gy_s = (const float *)gy + (size_t)n0 * C * items, *x_s = (const float *)x + (size_t)n0 * Ci * HW;
                    const uint8_t *amax_s = amax + (size_t)n0 * C * items;
                    float *gx_s = (float *)gx + (size_t)n0 * Ci * HW;
                    CLB_TRACED("convtree_bwd_w_win_kernel<tapgrad>", st,
                               convtree_bwd_w_win_kernel<true><<<dim3(plan.parts, C), threads, 0, st>>>(
                                   gy_s, x_s, (const float *)w, sel, amax_s, partial + (size_t)sl * plan.parts * C * 28, tapgrad, ss, wmode));
                    ++launched;
                    auto go = [&](auto k) {
                        if (clb_host::ensure_dynamic_smem(k, (int)smem) != cudaSuccess) return false;
                        CLB_TRACED("convtree_bwd_x_scatter_kernel", st,
                                   k<<<dim3((ss.N + nb - 1) / nb, G), sthreads, smem, st>>>(tapgrad, sel, amax_s, gx_s, grp_start, grp_list, cg, nb, ss));
                        return true;
                    };
                    ok = wpt == 1 ? go(convtree_bwd_x_scatter_kernel<1>) : wpt == 2 ? go(convtree_bwd_x_scatter_kernel<2>)
                       : wpt <= 4 ? go(convtree_bwd_x_scatter_kernel<4>) : go(convtree_bwd_x_scatter_kernel<8>);
                    // (wpt == 1: images of exactly 32 windows)
                    ++launched;
                }
                if (!ok) return check_launch(0);
                if (gw) {
                    const long long ngates = (long long)C * 7;
                    CLB_TRACED("gate_grad_finalize_kernel", st,
                               gate_grad_finalize_kernel<float><<<(int)((ngates + 127) / 128), 128, 0, st>>>(partial, (const float *)w, (float *)gw,
                                                                                                            plan.slices * plan.parts, ngates, wmode));
                    ++launched;
                }
                return check_launch(launched);
            }
        }
    }
    if (gx) {
        const int rc = launch_bwd_x<true>(gy, x, w, sel, amax, gx, grp_start, grp_list, cg, nb, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw,
                                          wmode, dtype, stream);
        if (rc) return rc;
    }
    if (gw)
        return launch_bwd_w<true>(gy, x, w, sel, amax, gw, scratch, scratch_bytes, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, wmode, dtype,
                                  stream);
    return CLB_OK;
}
