// Shape-specialised fp32 kernels of the fused ConvLogic block for stride 1 and images whose input
// channels all fit in shared memory (the first blocks of the CIFAR/MNIST stacks and the
// single-block benchmark: 9 x 32 x 32 inputs).
//
// Forward (convtree_fwd_tile_kernel)
//   * A persistent grid (one wave: SM count x resident blocks) splits the flattened
//     (image group, output channel) space into equal contiguous ranges, so the load is balanced to
//     within one channel and a block re-stages its input tile only when its range crosses into
//     the next image group.
//   * The tile holds G whole zero-padded images, all Ci channels.  Columns are de-interleaved:
//     a padded row is stored as [even columns | odd columns], PWH floats each.  A thread owns pooled
//     windows, whose four conv positions sit at columns 2px+dx; with de-interleaving, the 32 lanes of
//     a warp (consecutive px, then consecutive window rows) read consecutive words of one plane,
//     and PWH is chosen so that the window rows of a warp fall into disjoint bank ranges:
//     every gather is one conflict-free wavefront.
//   * Per output channel a thread needs 28 gate coefficients and 16 tap base offsets; they are
//     built once per channel by a few threads (soft-max included) and read by all as 128-bit
//     broadcast loads, amortised over WPT windows (4*WPT conv positions) per thread.
//   * Nothing but y (and the 1-byte arg-max the backward uses) is written to global memory.
#include "clb_common.cuh"

namespace clb {

constexpr int kFastThreads = 256;
constexpr int kChanBuf = 16; // channels prepared per refill of the coefficient buffer

struct alignas(16) ChanRec {
    float g[28];  // 7 gates x (k1, ka, kb, kab)
    int tb0[8];   // tile offset of tap k for the dx = 0 positions
    int tb1[8];   // ... for the dx = 1 positions
};

struct FastShape {
    int N, Ci, H, W, C, Ho, Wo, ph, pw, kh, kw;
    int G;      // images per group
    int PH;     // padded rows
    int pwh;    // floats per column-parity plane of a padded row
    int CS, IS; // channel / image stride in floats
    int wmode;
};

// PWH > 0: row stride known at compile time (2*PWH); PWH == 0: taken from the shape.
template <int WPT, int PWH>
__global__ void __launch_bounds__(kFastThreads, 2) convtree_fwd_tile_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                                        const int32_t *__restrict__ sel, float *__restrict__ y,
                                                                        uint8_t *__restrict__ amax, FastShape s)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    ChanRec *chan = reinterpret_cast<ChanRec *>(smem_raw);
    float *tile = reinterpret_cast<float *>(smem_raw + sizeof(ChanRec) * kChanBuf);

    const int pwh = PWH > 0 ? PWH : s.pwh;
    const int RS = 2 * pwh;
    const int Hp = s.Ho / 2, Wp = s.Wo / 2, I = Hp * Wp;
    const int tid = threadIdx.x;

    // contiguous range of (group, channel) units for this block
    const int NG = (s.N + s.G - 1) / s.G;
    const long long units = (long long)NG * s.C;
    const long long lo = units * blockIdx.x / gridDim.x, hi = units * (blockIdx.x + 1) / gridDim.x;
    if (lo >= hi) return;

    // loop-invariant window geometry of this thread
    int toff[WPT], wimg[WPT], wwin[WPT];
#pragma unroll
    for (int j = 0; j < WPT; ++j) {
        const int f = tid + kFastThreads * j;
        const int img = f / I, win = f - img * I;
        const int py = win / Wp, px = win - py * Wp;
        wimg[j] = img < s.G ? img : -1;
        wwin[j] = win;
        toff[j] = img * s.IS + 2 * py * RS + px;
    }

    // halo (and everything else) starts at zero; staging overwrites the interior only
    for (int i = tid; i < s.G * s.IS; i += kFastThreads) tile[i] = 0.f;

    int cur_group = -1;
    for (long long u0 = lo; u0 < hi;) {
        const int grp = (int)(u0 / s.C);
        const int c0 = (int)(u0 - (long long)grp * s.C);
        int cnt = s.C - c0;
        if (cnt > kChanBuf) cnt = kChanBuf;
        if (cnt > hi - u0) cnt = (int)(hi - u0);
        __syncthreads(); // previous chunk's readers are done with chan[] (and with the tile, if it changes)
        if (grp != cur_group) {
            cur_group = grp;
            const int n0 = grp * s.G;
            const int nimg = min(s.G, s.N - n0);
            const int rowsz = s.W;
            if ((rowsz & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) & 15) == 0)) {
                const int q = rowsz >> 2;
                const int total = nimg * s.Ci * s.H * q;
                for (int i = tid; i < total; i += kFastThreads) {
                    const int xq = i % q;
                    int r = i / q;
                    const int row = r % s.H;
                    r /= s.H;
                    const int ch = r % s.Ci, img = r / s.Ci;
                    const float4 v = __ldg(reinterpret_cast<const float4 *>(x + (((size_t)(n0 + img) * s.Ci + ch) * s.H + row) * s.W) + xq);
                    float *dst = tile + img * s.IS + ch * s.CS + (row + s.ph) * RS;
                    const int xp = xq * 4 + s.pw;
                    dst[((xp)&1) * pwh + ((xp) >> 1)] = v.x;
                    dst[((xp + 1) & 1) * pwh + ((xp + 1) >> 1)] = v.y;
                    dst[((xp + 2) & 1) * pwh + ((xp + 2) >> 1)] = v.z;
                    dst[((xp + 3) & 1) * pwh + ((xp + 3) >> 1)] = v.w;
                }
            } else {
                const int total = nimg * s.Ci * s.H * rowsz;
                for (int i = tid; i < total; i += kFastThreads) {
                    const int xc = i % rowsz;
                    int r = i / rowsz;
                    const int row = r % s.H;
                    r /= s.H;
                    const int ch = r % s.Ci, img = r / s.Ci;
                    const int xp = xc + s.pw;
                    tile[img * s.IS + ch * s.CS + (row + s.ph) * RS + (xp & 1) * pwh + (xp >> 1)] =
                        __ldg(x + (((size_t)(n0 + img) * s.Ci + ch) * s.H + row) * s.W + xc);
                }
            }
        }
        // coefficient records of channels c0 .. c0+cnt-1
        for (int i = tid; i < cnt * 7; i += kFastThreads) {
            const int cc = i / 7, gi = i - cc * 7;
            const Gate<float> g = gate_load<float>(w + ((size_t)(c0 + cc) * 7 + gi) * 16, s.wmode);
            float *o = chan[cc].g + gi * 4;
            o[0] = g.k1, o[1] = g.ka, o[2] = g.kb, o[3] = g.kab;
        }
        for (int i = tid; i < cnt * 8; i += kFastThreads) {
            const int cc = i >> 3, k = i & 7;
            const int word = sel[(c0 + cc) * 8 + k];
            // clamped to the tile, so that a selection outside the kernel window (which callers must route
            // to the general kernel) can never index beyond shared memory
            const int ch = min((word >> 16) & 0xFFFF, s.Ci - 1), r = min((word >> 8) & 0xFF, s.kh - 1),
                      sx = min(word & 0xFF, s.kw - 1);
            const int base = ch * s.CS + r * RS;
            chan[cc].tb0[k] = base + (sx & 1) * pwh + (sx >> 1);
            chan[cc].tb1[k] = base + ((sx + 1) & 1) * pwh + ((sx + 1) >> 1);
        }
        __syncthreads();

        const int n0 = grp * s.G;
        for (int cc = 0; cc < cnt; ++cc) {
            const int c = c0 + cc;
            // 11 x 128-bit broadcast loads
            float4 gq[7];
            int4 t0q[2], t1q[2];
            const float4 *gp = reinterpret_cast<const float4 *>(chan[cc].g);
#pragma unroll
            for (int i = 0; i < 7; ++i) gq[i] = gp[i];
            const int4 *tp0 = reinterpret_cast<const int4 *>(chan[cc].tb0);
            const int4 *tp1 = reinterpret_cast<const int4 *>(chan[cc].tb1);
            t0q[0] = tp0[0], t0q[1] = tp0[1], t1q[0] = tp1[0], t1q[1] = tp1[1];
            const int tb0[8] = {t0q[0].x, t0q[0].y, t0q[0].z, t0q[0].w, t0q[1].x, t0q[1].y, t0q[1].z, t0q[1].w};
            const int tb1[8] = {t1q[0].x, t1q[0].y, t1q[0].z, t1q[0].w, t1q[1].x, t1q[1].y, t1q[1].z, t1q[1].w};
            Gate<float> g[7];
#pragma unroll
            for (int i = 0; i < 7; ++i) g[i].k1 = gq[i].x, g[i].ka = gq[i].y, g[i].kb = gq[i].z, g[i].kab = gq[i].w;

#pragma unroll
            for (int j = 0; j < WPT; ++j) {
                if (wimg[j] < 0 || n0 + wimg[j] >= s.N) continue;
                float v[4][8]; // [position d = 2*dy+dx][tap]
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float *p0 = tile + toff[j] + tb0[k];
                    const float *p1 = tile + toff[j] + tb1[k];
                    v[0][k] = p0[0];
                    v[2][k] = p0[RS];
                    v[1][k] = p1[0];
                    v[3][k] = p1[RS];
                }
                float z[4];
#pragma unroll
                for (int d = 0; d < 4; ++d) {
                    const float g0 = gate_eval<float>(g[0], v[d][0], v[d][1]);
                    const float g1 = gate_eval<float>(g[1], v[d][2], v[d][3]);
                    const float g2 = gate_eval<float>(g[2], v[d][4], v[d][5]);
                    const float g3 = gate_eval<float>(g[3], v[d][6], v[d][7]);
                    const float t0 = gate_eval<float>(g[4], g0, g1);
                    const float t1 = gate_eval<float>(g[5], g2, g3);
                    z[d] = gate_eval<float>(g[6], t0, t1);
                }
                float best = z[0];
                int bd = 0;
#pragma unroll
                for (int d = 1; d < 4; ++d)
                    if (z[d] > best) { // strict '>' in scan order keeps the first maximum
                        best = z[d];
                        bd = d;
                    }
                const size_t o = ((size_t)(n0 + wimg[j]) * s.C + c) * I + wwin[j];
                y[o] = best;
                if (amax != nullptr) amax[o] = (uint8_t)bd;
            }
        }
        u0 += cnt;
    }
}

} // namespace clb

using namespace clb;
using namespace clb_host;

// Floats per column-parity plane: at least `need`, with the residue that keeps the window rows a warp
// covers in disjoint shared-memory bank ranges (see the file comment).
static int pick_pwh(int need, int Wp)
{
    if (Wp != 16 && Wp != 8 && Wp != 4) return need;
    for (int v = need; v < need + 8; ++v) {
        const int r = v & 7;
        const bool ok = Wp == 16 ? r == 4 : Wp == 8 ? (r == 2 || r == 6) : (r & 1);
        if (ok) return v;
    }
    return need;
}

template <int WPT, int PWH>
static int launch_fast(const float *x, const float *w, const int32_t *sel, float *y, uint8_t *amax, FastShape s, size_t smem,
                       int blocks_per_sm, cudaStream_t st)
{
    auto k = convtree_fwd_tile_kernel<WPT, PWH>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return check_launch(0);
    const long long units = (long long)((s.N + s.G - 1) / s.G) * s.C;
    long long grid = 148LL * blocks_per_sm;
    if (grid > units) grid = units;
    k<<<(unsigned)grid, kFastThreads, smem, st>>>(x, w, sel, y, amax, s);
    return check_launch();
}

int clb_convtree_fwd_fast_f32(const float *x, const float *w, const int32_t *sel, float *y, uint8_t *amax, int N, int Ci, int H, int W,
                              int C, int sh, int sw, int ph, int pw, int kh, int kw, int wmode, cudaStream_t st)
{
    if (sh != 1 || sw != 1) return CLB_ERR_SHAPE;
    FastShape s;
    s.N = N, s.Ci = Ci, s.H = H, s.W = W, s.C = C, s.ph = ph, s.pw = pw, s.kh = kh, s.kw = kw, s.wmode = wmode;
    s.Ho = conv_out(H, ph, kh, 1), s.Wo = conv_out(W, pw, kw, 1);
    if (s.Ho <= 0 || s.Wo <= 0 || (s.Ho & 1) || (s.Wo & 1)) return CLB_ERR_SHAPE;
    const int I = (s.Ho / 2) * (s.Wo / 2), Wp = s.Wo / 2;
    s.PH = H + 2 * ph;
    // every tap (row < kh, col < kw) of every conv position stays inside the padded image:
    // row <= Ho-1 + kh-1 = PH-1, column <= Wo-1 + kw-1 = W + 2*pw - 1
    const int need = (W + 2 * pw + 1) / 2;
    s.pwh = pick_pwh(need, Wp);
    s.CS = s.PH * 2 * s.pwh;
    s.IS = Ci * s.CS;
    const size_t img_bytes = (size_t)s.IS * 4;
    const size_t fixed = sizeof(ChanRec) * kChanBuf;
    // windows per thread: prefer 2 (amortises the per-channel coefficient loads), fall back to 1
    for (int wpt = 2; wpt >= 1; --wpt) {
        // a thread owns windows f = tid + 256*j of the flattened (image, window) space of a group, so a
        // group is as many WHOLE images as fit into 256*wpt windows
        int G = (kFastThreads * wpt) / I;
        if (G < 1) {
            if (wpt > 1) continue;
            return CLB_ERR_SHAPE; // more pooled positions per image than one block covers
        }
        if (G > N) G = N;
        const size_t smem = fixed + (size_t)G * img_bytes;
        if (smem > 110 * 1024 && wpt > 1) continue; // keep two blocks per SM when possible
        if (smem > 220 * 1024) return CLB_ERR_SHAPE;
        s.G = G;
        const int bps = smem <= 110 * 1024 ? 2 : 1;
        if (wpt == 2) {
            if (s.pwh == 20) return launch_fast<2, 20>(x, w, sel, y, amax, s, smem, bps, st);
            if (s.pwh == 10) return launch_fast<2, 10>(x, w, sel, y, amax, s, smem, bps, st);
            return launch_fast<2, 0>(x, w, sel, y, amax, s, smem, bps, st);
        }
        if (s.pwh == 20) return launch_fast<1, 20>(x, w, sel, y, amax, s, smem, bps, st);
        if (s.pwh == 10) return launch_fast<1, 10>(x, w, sel, y, amax, s, smem, bps, st);
        return launch_fast<1, 0>(x, w, sel, y, amax, s, smem, bps, st);
    }
    return CLB_ERR_SHAPE;
}
