// Shape-specialised fp32 kernels of the fused ConvLogic block for stride 1 and images whose input
// channels all fit in shared memory (the first blocks of the CIFAR/MNIST stacks and the
// single-block benchmark: 9 x 32 x 32 inputs).
//
// Common design
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
//     broadcast loads.
//
// Forward (convtree_fwd_tile_kernel): WPT windows (4*WPT conv positions) per thread and channel;
// nothing but y (and the 1-byte arg-max the backward uses) is written to global memory.
//
// Input gradient (convtree_bwd_x_cls_kernel): a second tile accumulates the gradient of the staged
// images (both tiles use the halo-free parity-class layout described at the kernel).  For one (channel, tap) the map window -> input pixel is injective,
// so threads add with plain read-modify-writes and a block barrier separates the 8 taps: the order
// of additions into a pixel is fixed (channel ascending, tap ascending).  A block whose range holds
// all channels of a group writes the final gradient; otherwise it writes a partial tile to scratch
// and convtree_bwd_x_reduce_kernel adds the partials of a group in block order.  No atomics.
#include "clb_common.cuh"

namespace clb {

constexpr int kFastThreads = 256;
constexpr int kChanBuf = 16; // channels prepared per refill of the coefficient buffer

struct alignas(16) ChanRec {
    float g[28];  // 7 gates x (k1, ka, kb, kab)
    int tb0[8];   // BYTE offset in the tile of tap k for the dx = 0 positions
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

__device__ __forceinline__ int tile_index(const FastShape &s, int pwh, int img, int ch, int row, int col)
{
    const int xp = col + s.pw;
    return img * s.IS + ch * s.CS + (row + s.ph) * 2 * pwh + (xp & 1) * pwh + (xp >> 1);
}

// Copies images n0 .. n0+nimg-1 into the (already zero-haloed) tile.
__device__ __forceinline__ void stage_group(float *tile, const float *__restrict__ x, const FastShape &s, int pwh, int n0, int nimg)
{
    const int tid = threadIdx.x;
    if ((s.W & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) & 15) == 0)) {
        const int q = s.W >> 2;
        const int total = nimg * s.Ci * s.H * q;
        for (int i = tid; i < total; i += kFastThreads) {
            const int xq = i % q;
            int r = i / q;
            const int row = r % s.H;
            r /= s.H;
            const int ch = r % s.Ci, img = r / s.Ci;
            const float4 v = __ldg(reinterpret_cast<const float4 *>(x + (((size_t)(n0 + img) * s.Ci + ch) * s.H + row) * s.W) + xq);
            tile[tile_index(s, pwh, img, ch, row, xq * 4)] = v.x;
            tile[tile_index(s, pwh, img, ch, row, xq * 4 + 1)] = v.y;
            tile[tile_index(s, pwh, img, ch, row, xq * 4 + 2)] = v.z;
            tile[tile_index(s, pwh, img, ch, row, xq * 4 + 3)] = v.w;
        }
    } else {
        const int total = nimg * s.Ci * s.H * s.W;
        for (int i = tid; i < total; i += kFastThreads) {
            const int xc = i % s.W;
            int r = i / s.W;
            const int row = r % s.H;
            r /= s.H;
            const int ch = r % s.Ci, img = r / s.Ci;
            tile[tile_index(s, pwh, img, ch, row, xc)] = __ldg(x + (((size_t)(n0 + img) * s.Ci + ch) * s.H + row) * s.W + xc);
        }
    }
}

// Gate coefficients and tap offsets of channels c0 .. c0+cnt-1.
__device__ __forceinline__ void build_records(ChanRec *chan, const float *__restrict__ w, const int32_t *__restrict__ sel,
                                              const FastShape &s, int pwh, int c0, int cnt)
{
    const int tid = threadIdx.x;
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
        const int ch = min((word >> 16) & 0xFFFF, s.Ci - 1), r = min((word >> 8) & 0xFF, s.kh - 1), sx = min(word & 0xFF, s.kw - 1);
        const int base = ch * s.CS + r * 2 * pwh;
        chan[cc].tb0[k] = 4 * (base + (sx & 1) * pwh + (sx >> 1));
        chan[cc].tb1[k] = 4 * (base + ((sx + 1) & 1) * pwh + ((sx + 1) >> 1));
    }
}

struct ChanRegs {
    Gate<float> g[7];
    int tb0[8], tb1[8];
};
__device__ __forceinline__ void load_record(ChanRegs &r, const ChanRec &rec)
{
    const float4 *gp = reinterpret_cast<const float4 *>(rec.g);
#pragma unroll
    for (int i = 0; i < 7; ++i) {
        const float4 q = gp[i];
        r.g[i].k1 = q.x, r.g[i].ka = q.y, r.g[i].kb = q.z, r.g[i].kab = q.w;
    }
    const int4 *t0 = reinterpret_cast<const int4 *>(rec.tb0), *t1 = reinterpret_cast<const int4 *>(rec.tb1);
    const int4 a0 = t0[0], a1 = t0[1], b0 = t1[0], b1 = t1[1];
    r.tb0[0] = a0.x, r.tb0[1] = a0.y, r.tb0[2] = a0.z, r.tb0[3] = a0.w, r.tb0[4] = a1.x, r.tb0[5] = a1.y, r.tb0[6] = a1.z, r.tb0[7] = a1.w;
    r.tb1[0] = b0.x, r.tb1[1] = b0.y, r.tb1[2] = b0.z, r.tb1[3] = b0.w, r.tb1[4] = b1.x, r.tb1[5] = b1.y, r.tb1[6] = b1.z, r.tb1[7] = b1.w;
}

__device__ __forceinline__ float ld_tile(const unsigned char *base, int byte_off) { return *reinterpret_cast<const float *>(base + byte_off); }

// =========================================================================================== forward
// PWH > 0: row stride known at compile time (2*PWH); PWH == 0: taken from the shape.
template <int WPT, int PWH>
__global__ void __launch_bounds__(kFastThreads, 2) convtree_fwd_tile_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                                           const int32_t *__restrict__ sel, float *__restrict__ y,
                                                                           uint8_t *__restrict__ amax, FastShape s)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    ChanRec *chan = reinterpret_cast<ChanRec *>(smem_raw);
    float *tile = reinterpret_cast<float *>(smem_raw + sizeof(ChanRec) * kChanBuf);
    const unsigned char *tileb = reinterpret_cast<const unsigned char *>(tile);

    const int pwh = PWH > 0 ? PWH : s.pwh;
    const int RSB = 8 * pwh; // row stride in bytes
    const int Hp = s.Ho / 2, Wp = s.Wo / 2, I = Hp * Wp;
    const int tid = threadIdx.x;

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
        toff[j] = 4 * (img * s.IS + 2 * py * 2 * pwh + px);
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
        const int n0 = grp * s.G;
        __syncthreads(); // previous chunk's readers are done with chan[] (and with the tile, if it changes)
        if (grp != cur_group) {
            cur_group = grp;
            stage_group(tile, x, s, pwh, n0, min(s.G, s.N - n0));
        }
        build_records(chan, w, sel, s, pwh, c0, cnt);
        __syncthreads();

        for (int cc = 0; cc < cnt; ++cc) {
            const int c = c0 + cc;
            ChanRegs r;
            load_record(r, chan[cc]);
#pragma unroll
            for (int j = 0; j < WPT; ++j) {
                if (wimg[j] < 0 || n0 + wimg[j] >= s.N) continue;
                float v[4][8]; // [position d = 2*dy+dx][tap]
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int a0 = toff[j] + r.tb0[k], a1 = toff[j] + r.tb1[k];
                    v[0][k] = ld_tile(tileb, a0);
                    v[2][k] = ld_tile(tileb, a0 + RSB);
                    v[1][k] = ld_tile(tileb, a1);
                    v[3][k] = ld_tile(tileb, a1 + RSB);
                }
                float z[4];
#pragma unroll
                for (int d = 0; d < 4; ++d) {
                    const float g0 = gate_eval<float>(r.g[0], v[d][0], v[d][1]);
                    const float g1 = gate_eval<float>(r.g[1], v[d][2], v[d][3]);
                    const float g2 = gate_eval<float>(r.g[2], v[d][4], v[d][5]);
                    const float g3 = gate_eval<float>(r.g[3], v[d][6], v[d][7]);
                    const float t0 = gate_eval<float>(r.g[4], g0, g1);
                    const float t1 = gate_eval<float>(r.g[5], g2, g3);
                    z[d] = gate_eval<float>(r.g[6], t0, t1);
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

// ---- forward on image pairs -----------------------------------------------------------------------------
// The same kernel with the two images a thread works on interleaved in the tile: element (channel, row, column)
// holds the float2 {image 2p, image 2p+1}, so one 64-bit shared load fetches a tap for both images and the gate
// polynomials run as packed two-float FMAs (fma.rn.f32x2: two independent IEEE fused multiply-adds, so the results
// are the scalar kernel's bit for bit) on operands that are pairs to begin with -- no packing moves.  Per pair of
// windows: 32 loads and 84 FMAs instead of 64 and 168.
struct alignas(16) PairRec {
    float g[28]; // 7 gates x (k1, ka, kb, kab)
    int tb0[8];  // BYTE offset in the pair tile of tap k for the dx = 0 positions
    int tb1[8];
};

typedef unsigned long long f32x2; // two floats in one 64-bit register

__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c)
{
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 dup2(unsigned bits)
{
    f32x2 d;
    asm("mov.b64 %0, {%1, %1};" : "=l"(d) : "r"(bits));
    return d;
}
struct Gate2 {
    f32x2 k1, ka, kb, kab;
};
__device__ __forceinline__ f32x2 gate_eval2(const Gate2 &g, f32x2 a, f32x2 b) { return fma2(a, fma2(g.kab, b, g.ka), fma2(g.kb, b, g.k1)); }

template <int PWH>
__global__ void __launch_bounds__(kFastThreads, 2) convtree_fwd_pair_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                                           const int32_t *__restrict__ sel, float *__restrict__ y,
                                                                           uint8_t *__restrict__ amax, FastShape s)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    PairRec *chan = reinterpret_cast<PairRec *>(smem_raw);
    float *tile = reinterpret_cast<float *>(smem_raw + sizeof(PairRec) * kChanBuf); // [pair][IS] float2
    const unsigned char *tileb = reinterpret_cast<const unsigned char *>(tile);

    const int pwh = PWH > 0 ? PWH : s.pwh;
    const int RSB = 16 * pwh; // row stride in bytes
    const int Hp = s.Ho / 2, Wp = s.Wo / 2, I = Hp * Wp;
    const int tid = threadIdx.x;
    const int P = s.G / 2; // image pairs per group (G is even)

    const int NG = (s.N + s.G - 1) / s.G;
    const long long units = (long long)NG * s.C;
    const long long lo = units * blockIdx.x / gridDim.x, hi = units * (blockIdx.x + 1) / gridDim.x;
    if (lo >= hi) return;

    const int pair = tid / I, win = tid - pair * I;
    const int py = win / Wp, px = win - py * Wp;
    const bool mine = pair < P;
    const int toff = 8 * (pair * s.IS + 2 * py * 2 * pwh + px);

    for (int i = tid; i < 2 * P * s.IS; i += kFastThreads) tile[i] = 0.f; // halo (and everything else) starts at zero

    int cur_group = -1;
    for (long long u0 = lo; u0 < hi;) {
        const int grp = (int)(u0 / s.C);
        const int c0 = (int)(u0 - (long long)grp * s.C);
        int cnt = s.C - c0;
        if (cnt > kChanBuf) cnt = kChanBuf;
        if (cnt > hi - u0) cnt = (int)(hi - u0);
        const int n0 = grp * s.G;
        __syncthreads(); // previous chunk's readers are done with chan[] (and with the tile, if it changes)
        if (grp != cur_group) {
            cur_group = grp;
            const int nimg = min(s.G, s.N - n0);
            if (nimg < s.G) // a last, incomplete group: the slots of the missing images must not keep older data
                for (int i = tid; i < 2 * P * s.IS; i += kFastThreads) tile[i] = 0.f;
            if (nimg < s.G) __syncthreads();
            const int q = s.W >> 2; // W % 4 == 0 and x 16-byte aligned: launch conditions
            const int total = nimg * s.Ci * s.H * q;
            for (int i = tid; i < total; i += kFastThreads) {
                const int xq = i % q;
                int r = i / q;
                const int row = r % s.H;
                r /= s.H;
                const int ch = r % s.Ci, img = r / s.Ci;
                const float4 v = __ldg(reinterpret_cast<const float4 *>(x + (((size_t)(n0 + img) * s.Ci + ch) * s.H + row) * s.W) + xq);
                float *t = tile + 2 * (img >> 1) * s.IS + (img & 1);
                const int e0 = ch * s.CS + (row + s.ph) * 2 * pwh;
                const int c = xq * 4 + s.pw;
                t[2 * (e0 + (c & 1) * pwh + (c >> 1))] = v.x;
                t[2 * (e0 + ((c + 1) & 1) * pwh + ((c + 1) >> 1))] = v.y;
                t[2 * (e0 + ((c + 2) & 1) * pwh + ((c + 2) >> 1))] = v.z;
                t[2 * (e0 + ((c + 3) & 1) * pwh + ((c + 3) >> 1))] = v.w;
            }
        }
        for (int i = tid; i < cnt * 7; i += kFastThreads) {
            const int cc = i / 7, gi = i - cc * 7;
            const Gate<float> g = gate_load<float>(w + ((size_t)(c0 + cc) * 7 + gi) * 16, s.wmode);
            float *o = chan[cc].g + gi * 4;
            o[0] = g.k1, o[1] = g.ka, o[2] = g.kb, o[3] = g.kab;
        }
        for (int i = tid; i < cnt * 8; i += kFastThreads) {
            const int cc = i >> 3, k = i & 7;
            const int word = sel[(c0 + cc) * 8 + k];
            const int ch = min((word >> 16) & 0xFFFF, s.Ci - 1), r = min((word >> 8) & 0xFF, s.kh - 1), sx = min(word & 0xFF, s.kw - 1);
            const int base = ch * s.CS + r * 2 * pwh;
            chan[cc].tb0[k] = 8 * (base + (sx & 1) * pwh + (sx >> 1));
            chan[cc].tb1[k] = 8 * (base + ((sx + 1) & 1) * pwh + ((sx + 1) >> 1));
        }
        __syncthreads();

        const int na = n0 + 2 * pair, nb = na + 1; // the thread's two images
        for (int cc = 0; cc < cnt; ++cc) {
            if (!mine || na >= s.N) continue;
            const PairRec &rec = chan[cc];
            Gate2 g[7];
            {
                // a coefficient is read once and doubled in registers: the shared-memory pipe, not the issue slots, binds
                const uint4 *gp = reinterpret_cast<const uint4 *>(rec.g);
#pragma unroll
                for (int i = 0; i < 7; ++i) {
                    const uint4 q = gp[i];
                    g[i].k1 = dup2(q.x), g[i].ka = dup2(q.y), g[i].kb = dup2(q.z), g[i].kab = dup2(q.w);
                }
            }
            int tb0[8], tb1[8];
            {
                const int4 *t0 = reinterpret_cast<const int4 *>(rec.tb0), *t1 = reinterpret_cast<const int4 *>(rec.tb1);
                const int4 a0 = t0[0], a1 = t0[1], b0 = t1[0], b1 = t1[1];
                tb0[0] = a0.x, tb0[1] = a0.y, tb0[2] = a0.z, tb0[3] = a0.w, tb0[4] = a1.x, tb0[5] = a1.y, tb0[6] = a1.z, tb0[7] = a1.w;
                tb1[0] = b0.x, tb1[1] = b0.y, tb1[2] = b0.z, tb1[3] = b0.w, tb1[4] = b1.x, tb1[5] = b1.y, tb1[6] = b1.z, tb1[7] = b1.w;
            }
            f32x2 z[4];
#pragma unroll
            for (int d = 0; d < 4; ++d) {
                f32x2 v[8];
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    v[k] = *reinterpret_cast<const f32x2 *>(tileb + toff + ((d & 1) ? tb1[k] : tb0[k]) + ((d >> 1) ? RSB : 0));
                const f32x2 g0 = gate_eval2(g[0], v[0], v[1]), g1 = gate_eval2(g[1], v[2], v[3]);
                const f32x2 g2 = gate_eval2(g[2], v[4], v[5]), g3 = gate_eval2(g[3], v[6], v[7]);
                z[d] = gate_eval2(g[6], gate_eval2(g[4], g0, g1), gate_eval2(g[5], g2, g3));
            }
            float best[2];
            int bd[2] = {0, 0};
            best[0] = __uint_as_float((unsigned)z[0]), best[1] = __uint_as_float((unsigned)(z[0] >> 32));
#pragma unroll
            for (int d = 1; d < 4; ++d) {
                const float z0 = __uint_as_float((unsigned)z[d]), z1 = __uint_as_float((unsigned)(z[d] >> 32));
                if (z0 > best[0]) best[0] = z0, bd[0] = d; // strict '>' in scan order keeps the first maximum
                if (z1 > best[1]) best[1] = z1, bd[1] = d;
            }
            const int c = c0 + cc;
            const size_t oa = ((size_t)na * s.C + c) * I + win;
            y[oa] = best[0];
            if (amax != nullptr) amax[oa] = (uint8_t)bd[0];
            if (nb < s.N) {
                const size_t ob = oa + (size_t)s.C * I;
                y[ob] = best[1];
                if (amax != nullptr) amax[ob] = (uint8_t)bd[1];
            }
        }
        u0 += cnt;
    }
}

// ======================================================================== forward, many input channels
// Layers behind the first one have hundreds of input channels and small images; an output channel
// reads only the channels its 8 taps name (two, by the reference's construction).  grid (parts, C): a
// block owns ONE output channel, so its 28 coefficients and 16 tap offsets live in registers for the
// whole kernel, and walks its share of the batch in slices of G images.  Per slice it stages just those
// two channel planes of the G images into the de-interleaved zero-haloed layout of the kernel above
// (conflict-free gathers), the next slice's planes being fetched into registers while the current one
// is evaluated.  A tap whose channel is a third or later distinct one (possible only with a
// hand-made selection) is gathered from global memory instead.
constexpr int kChanSlots = 2;
constexpr int kChanPrefetch = 4; // float4 per thread and slice

template <int WPT>
__global__ void __launch_bounds__(kFastThreads, 2) convtree_fwd_chan_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                                           const int32_t *__restrict__ sel, float *__restrict__ y,
                                                                           uint8_t *__restrict__ amax, FastShape s, int q4 /* float4 per thread per slice */)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *tile = reinterpret_cast<float *>(smem_raw);
    const unsigned char *tileb = smem_raw;
    __shared__ Gate<float> sg[7];
    __shared__ int sslot[8], sch[kChanSlots], snslot;
    __shared__ Tap stap[8];

    const int c = blockIdx.y;
    const int tid = threadIdx.x;
    const int pwh = s.pwh, RSB = 8 * pwh;
    const int Hp = s.Ho / 2, Wp = s.Wo / 2, I = Hp * Wp, HW = s.H * s.W;
    if (tid < 7) sg[tid] = gate_load<float>(w + ((size_t)c * 7 + tid) * 16, s.wmode);
    if (tid >= 64 && tid < 72) stap[tid - 64] = unpack_tap(sel[c * 8 + tid - 64], s.ph, s.pw);
    if (tid == 32) { // channel -> slot map of this output channel's taps
        int n = 0;
        int chs[8];
        bool inside = true;
        for (int k = 0; k < 8; ++k) {
            const int word = sel[c * 8 + k];
            const int ch = (word >> 16) & 0xFFFF;
            inside = inside && ch < s.Ci && ((word >> 8) & 0xFF) < s.kh && (word & 0xFF) < s.kw;
            int slot = -1;
            for (int j = 0; j < n; ++j)
                if (chs[j] == ch) slot = j;
            if (slot < 0) {
                slot = n;
                chs[n++] = ch;
            }
            sslot[k] = slot;
        }
        for (int j = 0; j < kChanSlots; ++j) sch[j] = min(chs[j < n ? j : 0], s.Ci - 1);
        snslot = inside ? n : kChanSlots + 1;
    }
    for (int i = tid; i < s.G * s.IS; i += kFastThreads) tile[i] = 0.f; // halo stays zero
    __syncthreads();

    Gate<float> g[7];
#pragma unroll
    for (int i = 0; i < 7; ++i) g[i] = sg[i];
    const int n_lo = (int)((long long)s.N * blockIdx.x / gridDim.x), n_hi = (int)((long long)s.N * (blockIdx.x + 1) / gridDim.x);

    if (snslot > kChanSlots) {
        // Hand-made selection (more than two channels, or taps outside the window): no staging, every tap is a
        // bounds-checked global load.  Block-uniform branch.
        for (int f = tid; f < (n_hi - n_lo) * I; f += kFastThreads) {
            const int img = f / I, win = f - img * I;
            const int py = win / Wp, px = win - py * Wp;
            const float *ximg = x + (size_t)(n_lo + img) * s.Ci * HW;
            float best = 0.f;
            int bd = 0;
            for (int d = 0; d < 4; ++d) {
                float a[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int iy = 2 * py + (d >> 1) + stap[k].dy, ix = 2 * px + (d & 1) + stap[k].dx;
                    a[k] = ((unsigned)iy < (unsigned)s.H && (unsigned)ix < (unsigned)s.W) ? __ldg(ximg + stap[k].ch * HW + iy * s.W + ix) : 0.f;
                }
                const float g0 = gate_eval<float>(g[0], a[0], a[1]), g1 = gate_eval<float>(g[1], a[2], a[3]);
                const float g2 = gate_eval<float>(g[2], a[4], a[5]), g3 = gate_eval<float>(g[3], a[6], a[7]);
                const float z = gate_eval<float>(g[6], gate_eval<float>(g[4], g0, g1), gate_eval<float>(g[5], g2, g3));
                if (d == 0 || z > best) {
                    best = z;
                    bd = d;
                }
            }
            const size_t o = ((size_t)(n_lo + img) * s.C + c) * I + win;
            y[o] = best;
            if (amax != nullptr) amax[o] = (uint8_t)bd;
        }
        return;
    }

    int tb0[8], tb1[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int word = sel[c * 8 + k];
        const int r = (word >> 8) & 0xFF, sx = word & 0xFF;
        const int base = sslot[k] * s.CS + r * 2 * pwh;
        tb0[k] = 4 * (base + (sx & 1) * pwh + (sx >> 1));
        tb1[k] = 4 * (base + ((sx + 1) & 1) * pwh + ((sx + 1) >> 1));
    }
    const int nstage = snslot;
    const int ch_a = sch[0], ch_b = sch[1];

    int toff[WPT], wimg[WPT], wwin[WPT];
#pragma unroll
    for (int j = 0; j < WPT; ++j) {
        const int f = tid + kFastThreads * j;
        const int img = f / I, win = f - img * I;
        const int py = win / Wp, px = win - py * Wp;
        wimg[j] = img < s.G ? img : -1;
        wwin[j] = win;
        toff[j] = 4 * (img * s.IS + 2 * py * 2 * pwh + px);
    }

    // one float4 = 4 consecutive pixels of one row of plane (img, slot); W % 4 == 0 is a launch condition.
    // Which float4s a thread moves, and where they land in the tile, is the same for every slice.
    const int w4 = s.W >> 2, per_plane = s.H * w4, per_slice = s.G * nstage * per_plane;
    int src[kChanPrefetch], dst[kChanPrefetch], simg[kChanPrefetch];
#pragma unroll
    for (int q = 0; q < kChanPrefetch; ++q) {
        const int i = tid + q * kFastThreads;
        simg[q] = -1;
        src[q] = dst[q] = 0;
        if (q < q4 && i < per_slice) {
            const int pl = i / per_plane, e = i - pl * per_plane;
            const int img = pl / nstage, slot = pl - img * nstage;
            const int row = e / w4, col = (e - row * w4) * 4;
            simg[q] = img;
            src[q] = (img * s.Ci + (slot ? ch_b : ch_a)) * HW + e * 4;
            dst[q] = img * s.IS + slot * s.CS + (row + s.ph) * 2 * pwh + ((col + s.pw) >> 1);
        }
    }
    // the 4 pixels of a float4 alternate between the two column-parity planes (col is a multiple of 4)
    const int p0 = (s.pw & 1) * pwh, p1 = ((s.pw + 1) & 1) * pwh + ((s.pw & 1) ? 1 : 0);
    const int p2 = p0 + 1, p3 = p1 + 1;
    float4 pre[kChanPrefetch];
    auto fetch = [&](int n0) {
        const float *xs = x + (size_t)n0 * s.Ci * HW;
#pragma unroll
        for (int q = 0; q < kChanPrefetch; ++q)
            if (simg[q] >= 0)
                pre[q] = n0 + simg[q] < n_hi ? __ldg(reinterpret_cast<const float4 *>(xs + src[q])) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto deposit = [&]() {
#pragma unroll
        for (int q = 0; q < kChanPrefetch; ++q)
            if (simg[q] >= 0) {
                float *d = tile + dst[q];
                d[p0] = pre[q].x, d[p1] = pre[q].y, d[p2] = pre[q].z, d[p3] = pre[q].w;
            }
    };

    fetch(n_lo);
    for (int n0 = n_lo; n0 < n_hi; n0 += s.G) {
        __syncthreads(); // the previous slice has been read
        deposit();
        __syncthreads();
        if (n0 + s.G < n_hi) fetch(n0 + s.G);
#pragma unroll
        for (int j = 0; j < WPT; ++j) {
            if (wimg[j] < 0 || n0 + wimg[j] >= n_hi) continue;
            float v[4][8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int a0 = toff[j] + tb0[k], a1 = toff[j] + tb1[k];
                v[0][k] = ld_tile(tileb, a0);
                v[2][k] = ld_tile(tileb, a0 + RSB);
                v[1][k] = ld_tile(tileb, a1);
                v[3][k] = ld_tile(tileb, a1 + RSB);
            }
            float best = 0.f;
            int bd = 0;
#pragma unroll
            for (int d = 0; d < 4; ++d) {
                const float g0 = gate_eval<float>(g[0], v[d][0], v[d][1]), g1 = gate_eval<float>(g[1], v[d][2], v[d][3]);
                const float g2 = gate_eval<float>(g[2], v[d][4], v[d][5]), g3 = gate_eval<float>(g[3], v[d][6], v[d][7]);
                const float z = gate_eval<float>(g[6], gate_eval<float>(g[4], g0, g1), gate_eval<float>(g[5], g2, g3));
                if (d == 0 || z > best) { // strict '>' in scan order keeps the first maximum
                    best = z;
                    bd = d;
                }
            }
            const size_t o = ((size_t)(n0 + wimg[j]) * s.C + c) * I + wwin[j];
            y[o] = best;
            if (amax != nullptr) amax[o] = (uint8_t)bd;
        }
    }
}

// Image-pair variant of the kernel above (see convtree_fwd_pair_kernel): the slice holds G/2 pairs of images interleaved
// as float2, a thread owns one window of one pair, taps are 64-bit loads and the gates packed two-float FMAs.
__global__ void __launch_bounds__(kFastThreads, 2) convtree_fwd_chan_pair_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                                           const int32_t *__restrict__ sel, float *__restrict__ y,
                                                                           uint8_t *__restrict__ amax, FastShape s, int q4 /* float4 per thread per slice */)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *tile = reinterpret_cast<float *>(smem_raw);
    const unsigned char *tileb = smem_raw;
    __shared__ Gate<float> sg[7];
    __shared__ int sslot[8], sch[kChanSlots], snslot;
    __shared__ Tap stap[8];

    const int c = blockIdx.y;
    const int tid = threadIdx.x;
    const int pwh = s.pwh, RSB = 16 * pwh;
    const int Hp = s.Ho / 2, Wp = s.Wo / 2, I = Hp * Wp, HW = s.H * s.W;
    if (tid < 7) sg[tid] = gate_load<float>(w + ((size_t)c * 7 + tid) * 16, s.wmode);
    if (tid >= 64 && tid < 72) stap[tid - 64] = unpack_tap(sel[c * 8 + tid - 64], s.ph, s.pw);
    if (tid == 32) { // channel -> slot map of this output channel's taps
        int n = 0;
        int chs[8];
        bool inside = true;
        for (int k = 0; k < 8; ++k) {
            const int word = sel[c * 8 + k];
            const int ch = (word >> 16) & 0xFFFF;
            inside = inside && ch < s.Ci && ((word >> 8) & 0xFF) < s.kh && (word & 0xFF) < s.kw;
            int slot = -1;
            for (int j = 0; j < n; ++j)
                if (chs[j] == ch) slot = j;
            if (slot < 0) {
                slot = n;
                chs[n++] = ch;
            }
            sslot[k] = slot;
        }
        for (int j = 0; j < kChanSlots; ++j) sch[j] = min(chs[j < n ? j : 0], s.Ci - 1);
        snslot = inside ? n : kChanSlots + 1;
    }
    for (int i = tid; i < s.G * s.IS; i += kFastThreads) tile[i] = 0.f; // halo stays zero
    __syncthreads();

    Gate<float> g[7];
#pragma unroll
    for (int i = 0; i < 7; ++i) g[i] = sg[i];
    const int n_lo = (int)((long long)s.N * blockIdx.x / gridDim.x), n_hi = (int)((long long)s.N * (blockIdx.x + 1) / gridDim.x);

    if (snslot > kChanSlots) {
        // Hand-made selection (more than two channels, or taps outside the window): no staging, every tap is a
        // bounds-checked global load.  Block-uniform branch.
        for (int f = tid; f < (n_hi - n_lo) * I; f += kFastThreads) {
            const int img = f / I, win = f - img * I;
            const int py = win / Wp, px = win - py * Wp;
            const float *ximg = x + (size_t)(n_lo + img) * s.Ci * HW;
            float best = 0.f;
            int bd = 0;
            for (int d = 0; d < 4; ++d) {
                float a[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int iy = 2 * py + (d >> 1) + stap[k].dy, ix = 2 * px + (d & 1) + stap[k].dx;
                    a[k] = ((unsigned)iy < (unsigned)s.H && (unsigned)ix < (unsigned)s.W) ? __ldg(ximg + stap[k].ch * HW + iy * s.W + ix) : 0.f;
                }
                const float g0 = gate_eval<float>(g[0], a[0], a[1]), g1 = gate_eval<float>(g[1], a[2], a[3]);
                const float g2 = gate_eval<float>(g[2], a[4], a[5]), g3 = gate_eval<float>(g[3], a[6], a[7]);
                const float z = gate_eval<float>(g[6], gate_eval<float>(g[4], g0, g1), gate_eval<float>(g[5], g2, g3));
                if (d == 0 || z > best) {
                    best = z;
                    bd = d;
                }
            }
            const size_t o = ((size_t)(n_lo + img) * s.C + c) * I + win;
            y[o] = best;
            if (amax != nullptr) amax[o] = (uint8_t)bd;
        }
        return;
    }

    int tb0[8], tb1[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int word = sel[c * 8 + k];
        const int r = (word >> 8) & 0xFF, sx = word & 0xFF;
        const int base = sslot[k] * s.CS + r * 2 * pwh;
        tb0[k] = 8 * (base + (sx & 1) * pwh + (sx >> 1));
        tb1[k] = 8 * (base + ((sx + 1) & 1) * pwh + ((sx + 1) >> 1));
    }
    Gate2 g2[7];
#pragma unroll
    for (int i = 0; i < 7; ++i)
        g2[i].k1 = dup2(__float_as_uint(g[i].k1)), g2[i].ka = dup2(__float_as_uint(g[i].ka)), g2[i].kb = dup2(__float_as_uint(g[i].kb)),
        g2[i].kab = dup2(__float_as_uint(g[i].kab));
    const int nstage = snslot;
    const int ch_a = sch[0], ch_b = sch[1];

    // a thread owns window `win` of the image pair (2*pair, 2*pair + 1) of every slice
    const int pair = tid / I, win = tid - pair * I;
    const int wpy = win / Wp, wpx = win - wpy * Wp;
    const bool mine = 2 * pair < s.G;
    const int toff = 8 * (pair * s.IS + 2 * wpy * 2 * pwh + wpx);

    // one float4 = 4 consecutive pixels of one row of plane (img, slot); W % 4 == 0 is a launch condition.
    // Which float4s a thread moves, and where they land in the tile, is the same for every slice.
    const int w4 = s.W >> 2, per_plane = s.H * w4, per_slice = s.G * nstage * per_plane;
    int src[kChanPrefetch], dst[kChanPrefetch], simg[kChanPrefetch];
#pragma unroll
    for (int q = 0; q < kChanPrefetch; ++q) {
        const int i = tid + q * kFastThreads;
        simg[q] = -1;
        src[q] = dst[q] = 0;
        if (q < q4 && i < per_slice) {
            const int pl = i / per_plane, e = i - pl * per_plane;
            const int img = pl / nstage, slot = pl - img * nstage;
            const int row = e / w4, col = (e - row * w4) * 4;
            simg[q] = img;
            src[q] = (img * s.Ci + (slot ? ch_b : ch_a)) * HW + e * 4;
            dst[q] = 2 * ((img >> 1) * s.IS + slot * s.CS + (row + s.ph) * 2 * pwh + ((col + s.pw) >> 1)) + (img & 1);
        }
    }
    // the 4 pixels of a float4 alternate between the two column-parity planes (col is a multiple of 4)
    const int p0 = 2 * ((s.pw & 1) * pwh), p1 = 2 * (((s.pw + 1) & 1) * pwh + ((s.pw & 1) ? 1 : 0));
    const int p2 = p0 + 2, p3 = p1 + 2;
    float4 pre[kChanPrefetch];
    auto fetch = [&](int n0) {
        const float *xs = x + (size_t)n0 * s.Ci * HW;
#pragma unroll
        for (int q = 0; q < kChanPrefetch; ++q)
            if (simg[q] >= 0)
                pre[q] = n0 + simg[q] < n_hi ? __ldg(reinterpret_cast<const float4 *>(xs + src[q])) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto deposit = [&]() {
#pragma unroll
        for (int q = 0; q < kChanPrefetch; ++q)
            if (simg[q] >= 0) {
                float *d = tile + dst[q];
                d[p0] = pre[q].x, d[p1] = pre[q].y, d[p2] = pre[q].z, d[p3] = pre[q].w;
            }
    };

    fetch(n_lo);
    for (int n0 = n_lo; n0 < n_hi; n0 += s.G) {
        __syncthreads(); // the previous slice has been read
        deposit();
        __syncthreads();
        if (n0 + s.G < n_hi) fetch(n0 + s.G);
        const int na = n0 + 2 * pair, nb = na + 1;
        if (mine && na < n_hi) {
            f32x2 z[4];
#pragma unroll
            for (int d = 0; d < 4; ++d) {
                f32x2 v[8];
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    v[k] = *reinterpret_cast<const f32x2 *>(tileb + toff + ((d & 1) ? tb1[k] : tb0[k]) + ((d >> 1) ? RSB : 0));
                const f32x2 g0 = gate_eval2(g2[0], v[0], v[1]), g1 = gate_eval2(g2[1], v[2], v[3]);
                const f32x2 q2 = gate_eval2(g2[2], v[4], v[5]), q3 = gate_eval2(g2[3], v[6], v[7]);
                z[d] = gate_eval2(g2[6], gate_eval2(g2[4], g0, g1), gate_eval2(g2[5], q2, q3));
            }
            float best[2];
            int bd[2] = {0, 0};
            best[0] = __uint_as_float((unsigned)z[0]), best[1] = __uint_as_float((unsigned)(z[0] >> 32));
#pragma unroll
            for (int d = 1; d < 4; ++d) {
                const float z0 = __uint_as_float((unsigned)z[d]), z1 = __uint_as_float((unsigned)(z[d] >> 32));
                if (z0 > best[0]) best[0] = z0, bd[0] = d; // strict '>' in scan order keeps the first maximum
                if (z1 > best[1]) best[1] = z1, bd[1] = d;
            }
            const size_t oa = ((size_t)na * s.C + c) * I + win;
            y[oa] = best[0];
            if (amax != nullptr) amax[oa] = (uint8_t)bd[0];
            if (nb < n_hi) {
                const size_t ob = oa + (size_t)s.C * I;
                y[ob] = best[1];
                if (amax != nullptr) amax[ob] = (uint8_t)bd[1];
            }
        }
    }
}

// ==================================================================================== input gradient
// Layout of the two backward tiles (x and its gradient): NO halo; a channel plane is split into the four
// parity classes of (row, column) -- class = 2*(row & 1) + (col & 1) -- each stored as a dense
// [ceil(H/2)][ceil(W/2)] array.  A thread owns one pooled window; the pixel a tap reaches from the
// window's arg-max position (dy, dx) is  toff + base_k + dy*A_k + dx*B_k  with per-channel uniform
// base/A/B, and whatever (dy, dx) the lanes of a warp have, lane px lands in bank (px + const) of its
// class plane: the data-dependent arg-max costs ~1.7 wavefronts per access instead of ~3 with the
// forward's row-major layout (which also needs a third more shared memory for its halo).
// (Skewing the odd-row / odd-column planes by Wh and 1 floats modulo 32 makes taps with odd offsets conflict-free
// and halves the conflict wavefronts, but it was measured to change nothing in the kernel's time -- the data pipe is
// not what binds it -- while the padding costs two record slots; the planes are therefore dense.)
// Out-of-image taps are predicated off instead of reading a zero halo.
constexpr int kBwdChanBuf = 6; // sized so that three blocks (two tiles + records + static) fit one SM

struct alignas(16) BwdRec {
    float g[28]; // 7 gates x (k1, ka, kb, kab)
    int base[8]; // byte offset of tap k from the window's first position
    int dA[8];   // added when the arg-max is in the window's second row
    int dB[8];   // added when it is in the second column
    int ty[8];   // tap row offset (row - pad), for the bounds test
    int tx[8];
};

struct ClsShape {
    int N, Ci, H, W, C, Ho, Wo, ph, pw, kh, kw;
    int G;          // images per group
    int Hh, Wh;     // class-plane extent
    int PL, CS, IS; // class plane, channel and image stride in floats
    int PR, PC;     // start of the odd-row / odd-column planes inside a channel
    int wmode;
};

__device__ __forceinline__ int cls_index(const ClsShape &s, int img, int ch, int row, int col)
{
    return img * s.IS + ch * s.CS + (row & 1) * s.PR + (col & 1) * s.PC + (row >> 1) * s.Wh + (col >> 1);
}

// Sum over the 32 lanes of 32 per-lane values at once: lane l returns the warp total of v[l].
// A butterfly that halves the number of live values at every step (16+8+4+2+1 = 31 shuffles) instead
// of 32 x 5 for value-by-value reductions.
__device__ __forceinline__ float warp_reduce_transposed(float (&v)[32], int lane)
{
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
    return v[0];
}

// GX: accumulate and write the input gradient.  GW: write, per (image group, channel), the 28 basis sums
// of the gate gradient to `wpartial` [groups][C][28]; both share the gate chain recomputed at the arg-max.
// WPT pooled windows per thread (blocks of 256 / WPT threads): the per-channel record loads and the warp
// reduction of the gate sums are paid once per thread, so WPT = 2 halves them per window.
template <bool GX, bool GW, int WPT>
__global__ void __launch_bounds__(kFastThreads / WPT, 3) convtree_bwd_cls_kernel(const float *__restrict__ gy, const float *__restrict__ x,
                                                                          const float *__restrict__ w, const int32_t *__restrict__ sel,
                                                                          const uint8_t *__restrict__ amax, float *__restrict__ gx,
                                                                          float *__restrict__ partial, float *__restrict__ wpartial,
                                                                          ClsShape s)
{
    constexpr int TPB = kFastThreads / WPT;
    __shared__ float wred[TPB / 32][32];
    extern __shared__ __align__(16) unsigned char smem_raw[];
    BwdRec *chan = reinterpret_cast<BwdRec *>(smem_raw);
    float *xt = reinterpret_cast<float *>(smem_raw + sizeof(BwdRec) * kBwdChanBuf);
    float *gt = xt + s.G * s.IS;
    const unsigned char *xtb = reinterpret_cast<const unsigned char *>(xt);
    unsigned char *gtb = reinterpret_cast<unsigned char *>(gt);

    const int Hp = s.Ho / 2, Wp = s.Wo / 2, I = Hp * Wp;
    const int tid = threadIdx.x;
    const int HW = s.H * s.W;

    const int NG = (s.N + s.G - 1) / s.G;
    const long long units = (long long)NG * s.C;
    const long long lo = units * blockIdx.x / gridDim.x, hi = units * (blockIdx.x + 1) / gridDim.x;
    if (lo >= hi) return;
    const int first_group = (int)(lo / s.C);

    int wimg[WPT], wwin[WPT], wy[WPT], wx[WPT], toff[WPT];
#pragma unroll
    for (int j = 0; j < WPT; ++j) {
        const int f = tid + TPB * j;
        const int img = f / I, win = f - img * I;
        const int py = win / Wp, px = win - py * Wp;
        wimg[j] = img < s.G ? img : -1;
        wwin[j] = win;
        wy[j] = 2 * py, wx[j] = 2 * px;
        toff[j] = 4 * (img * s.IS + py * s.Wh + px);
    }

    if (GX)
        for (int i = tid; i < s.G * s.IS; i += TPB) gt[i] = 0.f;

    auto stage = [&](int n0, int nimg) {
        const int total = nimg * s.Ci * HW;
        if ((s.W & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) & 15) == 0)) {
            for (int i = tid; i < (total >> 2); i += TPB) {
                const float4 v = __ldg(reinterpret_cast<const float4 *>(x + (size_t)n0 * s.Ci * HW) + i);
                const int e = i << 2;
                const int col = e % s.W;
                int r = e / s.W;
                const int row = r % s.H;
                r /= s.H;
                const int ch = r % s.Ci, im = r / s.Ci;
                const int b0 = cls_index(s, im, ch, row, col); // col is a multiple of 4: classes alternate
                xt[b0] = v.x, xt[b0 + s.PC] = v.y, xt[b0 + 1] = v.z, xt[b0 + s.PC + 1] = v.w;
            }
        } else {
            for (int i = tid; i < total; i += TPB) {
                const int col = i % s.W;
                int r = i / s.W;
                const int row = r % s.H;
                r /= s.H;
                xt[cls_index(s, r / s.Ci, r % s.Ci, row, col)] = __ldg(x + (size_t)n0 * s.Ci * HW + i);
            }
        }
    };
    // Writes the gradient tile of group `grp` (final when the block saw all its channels, else partial).
    auto flush = [&](int grp) {
        const int n0 = grp * s.G;
        const int nimg = min(s.G, s.N - n0);
        const bool whole = lo <= (long long)grp * s.C && hi >= (long long)(grp + 1) * s.C;
        float *dst = whole ? gx + (size_t)n0 * s.Ci * HW
                           : partial + ((size_t)blockIdx.x * 2 + (grp == first_group ? 0 : 1)) * (size_t)s.G * s.Ci * HW;
        const int total = nimg * s.Ci * HW;
        for (int i = tid; i < total; i += TPB) {
            const int col = i % s.W;
            int r = i / s.W;
            const int row = r % s.H;
            r /= s.H;
            dst[i] = gt[cls_index(s, r / s.Ci, r % s.Ci, row, col)];
        }
        __syncthreads();
        for (int i = tid; i < s.G * s.IS; i += TPB) gt[i] = 0.f;
    };
    // f(t): offset of row/col displacement t inside the class layout (t may be negative)
    auto fy = [&](int t) { return (t & 1) * s.PR + (t >> 1) * s.Wh; };
    auto fx = [&](int t) { return (t & 1) * s.PC + (t >> 1); };

    int cur_group = -1;
    for (long long u0 = lo; u0 < hi;) {
        const int grp = (int)(u0 / s.C);
        const int c0 = (int)(u0 - (long long)grp * s.C);
        int cnt = s.C - c0;
        if (cnt > kBwdChanBuf) cnt = kBwdChanBuf;
        if (cnt > hi - u0) cnt = (int)(hi - u0);
        const int n0 = grp * s.G;
        __syncthreads();
        if (grp != cur_group) {
            if (GX && cur_group >= 0) flush(cur_group);
            cur_group = grp;
            stage(n0, min(s.G, s.N - n0));
        }
        for (int i = tid; i < cnt * 7; i += TPB) {
            const int cc = i / 7, gi = i - cc * 7;
            const Gate<float> g = gate_load<float>(w + ((size_t)(c0 + cc) * 7 + gi) * 16, s.wmode);
            float *o = chan[cc].g + gi * 4;
            o[0] = g.k1, o[1] = g.ka, o[2] = g.kb, o[3] = g.kab;
        }
        for (int i = tid; i < cnt * 8; i += TPB) {
            const int cc = i >> 3, k = i & 7;
            const int word = sel[(c0 + cc) * 8 + k];
            const int ch = min((word >> 16) & 0xFFFF, s.Ci - 1);
            const int ty = ((word >> 8) & 0xFF) - s.ph, tx = (word & 0xFF) - s.pw;
            chan[cc].base[k] = 4 * (ch * s.CS + fy(ty) + fx(tx));
            chan[cc].dA[k] = 4 * (fy(ty + 1) - fy(ty));
            chan[cc].dB[k] = 4 * (fx(tx + 1) - fx(tx));
            chan[cc].ty[k] = ty;
            chan[cc].tx[k] = tx;
        }
        __syncthreads();

        bool live[WPT];
        size_t obase[WPT];
        float gy_next[WPT];
        int bd_next[WPT];
        // software pipeline: the next channel's gy / arg-max loads are in flight during this channel's work
#pragma unroll
        for (int j = 0; j < WPT; ++j) {
            live[j] = wimg[j] >= 0 && n0 + wimg[j] < s.N;
            obase[j] = live[j] ? ((size_t)(n0 + wimg[j]) * s.C + c0) * I + wwin[j] : 0;
            gy_next[j] = live[j] ? __ldg(gy + obase[j]) : 0.f;
            bd_next[j] = live[j] ? (int)__ldg(amax + obase[j]) : 0;
        }
        for (int cc = 0; cc < cnt; ++cc) {
            const BwdRec &rec = chan[cc];
            Gate<float> g[7];
            {
                const float4 *gp = reinterpret_cast<const float4 *>(rec.g);
#pragma unroll
                for (int i = 0; i < 7; ++i) {
                    const float4 q = gp[i];
                    g[i].k1 = q.x, g[i].ka = q.y, g[i].kb = q.z, g[i].kab = q.w;
                }
            }
            int rb[8], ra[8], rc[8], ry[8], rx[8];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int4 b4 = reinterpret_cast<const int4 *>(rec.base)[q], a4 = reinterpret_cast<const int4 *>(rec.dA)[q];
                const int4 c4 = reinterpret_cast<const int4 *>(rec.dB)[q], y4 = reinterpret_cast<const int4 *>(rec.ty)[q];
                const int4 x4 = reinterpret_cast<const int4 *>(rec.tx)[q];
                rb[4 * q] = b4.x, rb[4 * q + 1] = b4.y, rb[4 * q + 2] = b4.z, rb[4 * q + 3] = b4.w;
                ra[4 * q] = a4.x, ra[4 * q + 1] = a4.y, ra[4 * q + 2] = a4.z, ra[4 * q + 3] = a4.w;
                rc[4 * q] = c4.x, rc[4 * q + 1] = c4.y, rc[4 * q + 2] = c4.z, rc[4 * q + 3] = c4.w;
                ry[4 * q] = y4.x, ry[4 * q + 1] = y4.y, ry[4 * q + 2] = y4.z, ry[4 * q + 3] = y4.w;
                rx[4 * q] = x4.x, rx[4 * q + 1] = x4.y, rx[4 * q + 2] = x4.z, rx[4 * q + 3] = x4.w;
            }
            int addr[WPT][8];
            float tg[WPT][8];
            unsigned ok[WPT];
            float bs[32]; // 28 basis products of this thread's windows (GW), padded to a power of two
#pragma unroll
            for (int i = 0; i < 32; ++i) bs[i] = 0.f;
#pragma unroll
            for (int j = 0; j < WPT; ++j) {
                const float dz = gy_next[j];
                const int bd = bd_next[j];
                if (live[j] && cc + 1 < cnt) {
                    gy_next[j] = __ldg(gy + obase[j] + (size_t)(cc + 1) * I);
                    bd_next[j] = (int)__ldg(amax + obase[j] + (size_t)(cc + 1) * I);
                }
                ok[j] = 0;
                if (live[j]) {
                    const int dyi = bd >> 1, dxi = bd & 1;
                    const int oy = wy[j] + dyi, ox = wx[j] + dxi;
                    float a[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        addr[j][k] = toff[j] + rb[k] + dyi * ra[k] + dxi * rc[k];
                        const bool v = (unsigned)(oy + ry[k]) < (unsigned)s.H && (unsigned)(ox + rx[k]) < (unsigned)s.W;
                        ok[j] |= (v ? 1u : 0u) << k;
                        a[k] = v ? ld_tile(xtb, addr[j][k]) : 0.f;
                    }
                    const float g0 = gate_eval<float>(g[0], a[0], a[1]), g1 = gate_eval<float>(g[1], a[2], a[3]);
                    const float g2 = gate_eval<float>(g[2], a[4], a[5]), g3 = gate_eval<float>(g[3], a[6], a[7]);
                    const float t0 = gate_eval<float>(g[4], g0, g1), t1 = gate_eval<float>(g[5], g2, g3);
                    const float dt0 = dz * gate_da<float>(g[6], t1), dt1 = dz * gate_db<float>(g[6], t0);
                    const float dg0 = dt0 * gate_da<float>(g[4], g1), dg1 = dt0 * gate_db<float>(g[4], g0);
                    const float dg2 = dt1 * gate_da<float>(g[5], g3), dg3 = dt1 * gate_db<float>(g[5], g2);
                    tg[j][0] = dg0 * gate_da<float>(g[0], a[1]), tg[j][1] = dg0 * gate_db<float>(g[0], a[0]);
                    tg[j][2] = dg1 * gate_da<float>(g[1], a[3]), tg[j][3] = dg1 * gate_db<float>(g[1], a[2]);
                    tg[j][4] = dg2 * gate_da<float>(g[2], a[5]), tg[j][5] = dg2 * gate_db<float>(g[2], a[4]);
                    tg[j][6] = dg3 * gate_da<float>(g[3], a[7]), tg[j][7] = dg3 * gate_db<float>(g[3], a[6]);
                    if (GW) {
                        const float dgp[4] = {dg0, dg1, dg2, dg3};
#pragma unroll
                        for (int p = 0; p < 4; ++p) {
                            bs[4 * p] = fmaf(dgp[p], a[2 * p] * a[2 * p + 1], bs[4 * p]), bs[4 * p + 1] = fmaf(dgp[p], a[2 * p], bs[4 * p + 1]);
                            bs[4 * p + 2] = fmaf(dgp[p], a[2 * p + 1], bs[4 * p + 2]), bs[4 * p + 3] += dgp[p];
                        }
                        bs[16] = fmaf(dt0, g0 * g1, bs[16]), bs[17] = fmaf(dt0, g0, bs[17]), bs[18] = fmaf(dt0, g1, bs[18]), bs[19] += dt0;
                        bs[20] = fmaf(dt1, g2 * g3, bs[20]), bs[21] = fmaf(dt1, g2, bs[21]), bs[22] = fmaf(dt1, g3, bs[22]), bs[23] += dt1;
                        bs[24] = fmaf(dz, t0 * t1, bs[24]), bs[25] = fmaf(dz, t0, bs[25]), bs[26] = fmaf(dz, t1, bs[26]), bs[27] += dz;
                    }
                }
            }
            if (GW) {
                // block total of the 28 basis sums of this (group, channel): warps first, then 8 -> 1 by warp 0
                const float tot = warp_reduce_transposed(bs, tid & 31);
                if (!GX) __syncthreads(); // the previous channel's cross-warp read is over
                wred[tid >> 5][tid & 31] = tot;
            }
            if (GX) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
#pragma unroll
                    for (int j = 0; j < WPT; ++j)
                        if ((ok[j] >> k) & 1u) {
                            float *cell = reinterpret_cast<float *>(gtb + addr[j][k]);
                            *cell += tg[j][k];
                        }
                    __syncthreads();
                    if (GW && k == 0 && tid < 28) {
                        float t = 0.f;
#pragma unroll
                        for (int wv = 0; wv < TPB / 32; ++wv) t += wred[wv][tid];
                        wpartial[((size_t)grp * s.C + c0 + cc) * 28 + tid] = t;
                    }
                }
            } else if (GW) {
                __syncthreads();
                if (tid < 28) {
                    float t = 0.f;
#pragma unroll
                    for (int wv = 0; wv < TPB / 32; ++wv) t += wred[wv][tid];
                    wpartial[((size_t)grp * s.C + c0 + cc) * 28 + tid] = t;
                }
            }
        }
        u0 += cnt;
    }
    __syncthreads();
    if (GX) flush(cur_group);
}

// Adds the per-group basis sums and turns them into the 16 gradients of every gate.  Eight threads share a
// gate: each adds a contiguous eighth of the groups in order, then the eight partial sums are added in
// order -- a fixed summation tree, so the result does not depend on scheduling.
__device__ __forceinline__ void gw_finalize_block(const float *__restrict__ wpartial, const float *__restrict__ w, float *__restrict__ gw,
                                                  int groups, int ngates, int wmode, int block)
{
    __shared__ float4 part[32][8];
    const int local = threadIdx.x >> 3, sub = threadIdx.x & 7;
    const int gi = block * 32 + local;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (gi < ngates) {
        const int per = (groups + 7) / 8;
        const int lo = sub * per, hi = min(groups, lo + per);
        for (int p = lo; p < hi; ++p) {
            const float4 q = *reinterpret_cast<const float4 *>(wpartial + ((size_t)p * ngates + gi) * 4);
            acc.x += q.x, acc.y += q.y, acc.z += q.z, acc.w += q.w;
        }
    }
    part[local][sub] = acc;
    __syncthreads();
    if (sub == 0 && gi < ngates) {
        float sums[4] = {0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < 8; ++k) {
            const float4 q = part[local][k];
            sums[0] += q.x, sums[1] += q.y, sums[2] += q.z, sums[3] += q.w;
        }
        gate_grad_store<float>(sums, w + (size_t)gi * 16, wmode, gw + (size_t)gi * 16);
    }
}

__global__ void __launch_bounds__(256) convtree_gw_finalize_kernel(const float *__restrict__ wpartial, const float *__restrict__ w,
                                                                   float *__restrict__ gw, int groups, int ngates, int wmode)
{
    gw_finalize_block(wpartial, w, gw, groups, ngates, wmode, blockIdx.x);
}

// gx of every group that no single block covered = sum of that group's partial tiles, in block order.
// grid (chunks, groups): the owners of a group's first and last channel are found once per thread.
__device__ __forceinline__ void bwd_x_reduce_block(const float *__restrict__ partial, float *__restrict__ gx, const ClsShape &s, int grid,
                                                   int bx, int grp, int chunks)
{
    const int HW = s.H * s.W;
    const int per_group = s.G * s.Ci * HW;
    const int NG = (s.N + s.G - 1) / s.G;
    const long long units = (long long)NG * s.C;
    // owner(u): the block b with units*b/grid <= u < units*(b+1)/grid
    auto owner = [&](long long u) {
        long long b = u * grid / units;
        while (b + 1 < grid && units * (b + 1) / grid <= u) ++b;
        while (b > 0 && units * b / grid > u) --b;
        return (int)b;
    };
    const int b1 = owner((long long)grp * s.C), b2 = owner((long long)(grp + 1) * s.C - 1);
    if (b1 == b2) return; // that block wrote the final values itself
    const int live = min(s.G, s.N - grp * s.G) * s.Ci * HW; // the last group may hold fewer images
    const float *p1 = partial + ((size_t)b1 * 2 + ((int)((units * b1 / grid) / s.C) == grp ? 0 : 1)) * per_group;
    float *out = gx + (size_t)grp * per_group;
    for (int e = bx * blockDim.x + threadIdx.x; e < live; e += chunks * blockDim.x) {
        float acc = p1[e];
        // every later block starts inside this group, so the group is its first: slot 0
        for (int b = b1 + 1; b <= b2; ++b) acc += partial[(size_t)b * 2 * per_group + e];
        out[e] = acc;
    }
}

__global__ void __launch_bounds__(256) convtree_bwd_x_reduce_kernel(const float *__restrict__ partial, float *__restrict__ gx, ClsShape s,
                                                                    int grid)
{
    bwd_x_reduce_block(partial, gx, s, grid, blockIdx.x, blockIdx.y, gridDim.x);
}

// Both of the above in one launch (they do not depend on each other): blocks [0, chunks*groups) reduce the partial
// gradient tiles, the rest finish the gate gradients.
__global__ void __launch_bounds__(256) convtree_bwd_post_kernel(const float *__restrict__ partial, float *__restrict__ gx, ClsShape s, int grid,
                                                                int chunks, int ngroups, const float *__restrict__ wpartial,
                                                                const float *__restrict__ w, float *__restrict__ gw, int ngates, int wmode)
{
    const int rb = chunks * ngroups;
    if ((int)blockIdx.x < rb)
        bwd_x_reduce_block(partial, gx, s, grid, blockIdx.x % chunks, blockIdx.x / chunks, chunks);
    else
        gw_finalize_block(wpartial, w, gw, ngroups, ngates, wmode, blockIdx.x - rb);
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

// Fills everything but G; false when the shape is outside the tiled kernels' domain.
static bool make_fast_shape(FastShape &s, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int wmode)
{
    if (sh != 1 || sw != 1) return false;
    s.N = N, s.Ci = Ci, s.H = H, s.W = W, s.C = C, s.ph = ph, s.pw = pw, s.kh = kh, s.kw = kw, s.wmode = wmode;
    s.Ho = conv_out(H, ph, kh, 1), s.Wo = conv_out(W, pw, kw, 1);
    if (s.Ho <= 0 || s.Wo <= 0 || (s.Ho & 1) || (s.Wo & 1)) return false;
    s.PH = H + 2 * ph;
    // every tap (row < kh, col < kw) of every conv position stays inside the padded image:
    // row <= Ho-1 + kh-1 = PH-1, column <= Wo-1 + kw-1 = W + 2*pw - 1
    s.pwh = pick_pwh((W + 2 * pw + 1) / 2, s.Wo / 2);
    s.CS = s.PH * 2 * s.pwh;
    s.IS = Ci * s.CS;
    s.G = 1;
    return (size_t)s.IS * 4 <= 200 * 1024;
}

template <int PWH>
static int launch_fwd_pair(const float *x, const float *w, const int32_t *sel, float *y, uint8_t *amax, FastShape s, size_t smem,
                           int blocks_per_sm, cudaStream_t st)
{
    auto k = convtree_fwd_pair_kernel<PWH>;
    if (clb_host::ensure_dynamic_smem(k, (int)smem) != cudaSuccess) return check_launch(0);
    const long long units = (long long)((s.N + s.G - 1) / s.G) * s.C;
    long long grid = (long long)sm_count() * blocks_per_sm;
    if (grid > units) grid = units;
    CLB_TRACED("convtree_fwd_pair_kernel", st, k<<<(unsigned)grid, kFastThreads, smem, st>>>(x, w, sel, y, amax, s));
    return check_launch();
}

template <int WPT, int PWH>
static int launch_fwd(const float *x, const float *w, const int32_t *sel, float *y, uint8_t *amax, FastShape s, size_t smem,
                      int blocks_per_sm, cudaStream_t st)
{
    auto k = convtree_fwd_tile_kernel<WPT, PWH>;
    if (clb_host::ensure_dynamic_smem(k, (int)smem) != cudaSuccess) return check_launch(0);
    const long long units = (long long)((s.N + s.G - 1) / s.G) * s.C;
    long long grid = (long long)sm_count() * blocks_per_sm;
    if (grid > units) grid = units;
    CLB_TRACED("convtree_fwd_tile_kernel", st, k<<<(unsigned)grid, kFastThreads, smem, st>>>(x, w, sel, y, amax, s));
    return check_launch();
}

// Two-channel-plane variant: applies when W is a multiple of 4, x is 16-byte aligned and a slice fits.
static int launch_fwd_chan(const float *x, const float *w, const int32_t *sel, float *y, uint8_t *amax, int N, int Ci, int H, int W, int C,
                           int ph, int pw, int kh, int kw, int wmode, cudaStream_t st)
{
    if ((W & 3) || (reinterpret_cast<uintptr_t>(x) & 15) || C > 65535) return CLB_ERR_SHAPE;
    FastShape s;
    s.N = N, s.Ci = Ci, s.H = H, s.W = W, s.C = C, s.ph = ph, s.pw = pw, s.kh = kh, s.kw = kw, s.wmode = wmode;
    s.Ho = conv_out(H, ph, kh, 1), s.Wo = conv_out(W, pw, kw, 1);
    if (s.Ho <= 0 || s.Wo <= 0 || (s.Ho & 1) || (s.Wo & 1)) return CLB_ERR_SHAPE;
    const int I = (s.Ho / 2) * (s.Wo / 2);
    s.PH = H + 2 * ph;
    s.pwh = pick_pwh((W + 2 * pw + 1) / 2, s.Wo / 2);
    s.CS = s.PH * 2 * s.pwh;
    s.IS = kChanSlots * s.CS;
    constexpr int WPT = 2;
    int G = (kFastThreads * WPT) / I;
    if (G < 1) return CLB_ERR_SHAPE;
    if (G > N) G = N;
    s.G = G;
    const size_t smem = (size_t)G * s.IS * 4;
    if (smem > 72 * 1024) return CLB_ERR_SHAPE;
    const int q4 = (G * kChanSlots * H * (W / 4) + kFastThreads - 1) / kFastThreads;
    if (q4 > kChanPrefetch) return CLB_ERR_SHAPE;
    int parts = (int)(((long long)sm_count() * 3 * 8 + C - 1) / C); // about eight waves of three resident blocks per SM
    if (parts > (N + G - 1) / G) parts = (N + G - 1) / G;
    if (parts < 1) parts = 1;
    if (G % 2 == 0 && (G / 2) * I <= kFastThreads) { // image pairs: 64-bit tap loads, packed two-float FMAs
        auto k2 = convtree_fwd_chan_pair_kernel;
        if (clb_host::ensure_dynamic_smem(k2, (int)smem) != cudaSuccess) return check_launch(0);
        CLB_TRACED("convtree_fwd_chan_pair_kernel", st, k2<<<dim3(parts, C), kFastThreads, smem, st>>>(x, w, sel, y, amax, s, q4));
        return check_launch();
    }
    auto k = convtree_fwd_chan_kernel<WPT>;
    if (clb_host::ensure_dynamic_smem(k, (int)smem) != cudaSuccess) return check_launch(0);
    CLB_TRACED("convtree_fwd_chan_kernel", st, k<<<dim3(parts, C), kFastThreads, smem, st>>>(x, w, sel, y, amax, s, q4));
    return check_launch();
}

int clb_convtree_fwd_plane_f32(const float *x, const float *w, const int32_t *sel, float *y, uint8_t *amax, int N, int Ci, int H, int W, int C,
                               int sh, int sw, int ph, int pw, int kh, int kw, int wmode, cudaStream_t st); // convtree_plane.cu

int clb_convtree_fwd_fast_f32(const float *x, const float *w, const int32_t *sel, float *y, uint8_t *amax, int N, int Ci, int H, int W,
                              int C, int sh, int sw, int ph, int pw, int kh, int kw, int wmode, cudaStream_t st)
{
    FastShape s;
    if (sh != 1 || sw != 1) return CLB_ERR_SHAPE;
    // many input channels: an image's channels do not fit shared memory (or barely one image does)
    if ((size_t)Ci * (H + 2 * ph) * (W + 2 * pw) * 4 > 48 * 1024) {
        const int rc = clb_convtree_fwd_plane_f32(x, w, sel, y, amax, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, wmode, st);
        if (rc != CLB_ERR_SHAPE) return rc;
        return launch_fwd_chan(x, w, sel, y, amax, N, Ci, H, W, C, ph, pw, kh, kw, wmode, st);
    }
    if (!make_fast_shape(s, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, wmode)) return CLB_ERR_SHAPE;
    const int I = (s.Ho / 2) * (s.Wo / 2);
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
        if (wpt == 2 && G % 2 == 0 && (W & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
            // two images per thread, interleaved in the tile: packed two-float FMAs
            const size_t smem2 = smem - fixed + sizeof(PairRec) * kChanBuf;
            if (smem2 <= 110 * 1024) {
                if (s.pwh == 20) return launch_fwd_pair<20>(x, w, sel, y, amax, s, smem2, 2, st);
                if (s.pwh == 10) return launch_fwd_pair<10>(x, w, sel, y, amax, s, smem2, 2, st);
                return launch_fwd_pair<0>(x, w, sel, y, amax, s, smem2, 2, st);
            }
        }
        if (wpt == 2) {
            if (s.pwh == 20) return launch_fwd<2, 20>(x, w, sel, y, amax, s, smem, bps, st);
            if (s.pwh == 10) return launch_fwd<2, 10>(x, w, sel, y, amax, s, smem, bps, st);
            return launch_fwd<2, 0>(x, w, sel, y, amax, s, smem, bps, st);
        }
        if (s.pwh == 20) return launch_fwd<1, 20>(x, w, sel, y, amax, s, smem, bps, st);
        if (s.pwh == 10) return launch_fwd<1, 10>(x, w, sel, y, amax, s, smem, bps, st);
        return launch_fwd<1, 0>(x, w, sel, y, amax, s, smem, bps, st);
    }
    return CLB_ERR_SHAPE;
}

// ---- input gradient --------------------------------------------------------------------------
// Plan shared by the scratch-size query and the launch: false when the tiled kernel does not apply.
static bool plan_bwd_x(ClsShape &s, size_t &smem, int &grid, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh,
                       int kw, int wmode)
{
    if (N <= 0 || C <= 0 || sh != 1 || sw != 1) return false;
    s.N = N, s.Ci = Ci, s.H = H, s.W = W, s.C = C, s.ph = ph, s.pw = pw, s.kh = kh, s.kw = kw, s.wmode = wmode;
    s.Ho = conv_out(H, ph, kh, 1), s.Wo = conv_out(W, pw, kw, 1);
    if (s.Ho <= 0 || s.Wo <= 0 || (s.Ho & 1) || (s.Wo & 1)) return false;
    s.Hh = (H + 1) / 2, s.Wh = (W + 1) / 2;
    s.PL = s.Hh * s.Wh;
    s.PC = s.PL, s.PR = 2 * s.PL;
    s.CS = (s.PR + s.PC + s.PL + 3) / 4 * 4;
    s.IS = Ci * s.CS;
    const int I = (s.Ho / 2) * (s.Wo / 2);
    int G = kFastThreads / I;
    if (G < 1) return false;
    if (G > N) G = N;
    const size_t fixed = sizeof(BwdRec) * kBwdChanBuf;
    while (G > 1 && fixed + 2 * (size_t)G * s.IS * 4 > 110 * 1024) --G;
    smem = fixed + 2 * (size_t)G * s.IS * 4;
    if (smem > 220 * 1024) return false;
    s.G = G;
    if ((N + G - 1) / G > 65535) return false; // the reduce kernel's grid.y
    // resident blocks per SM: 233472 bytes of shared memory, 1 KiB reserved per block, 128 static bytes per warp
    const size_t per_block = smem + 1024 + (G * I > kFastThreads / 2 ? kFastThreads / 2 : kFastThreads) / 32 * 128;
    const int bps = 3 * per_block <= 233472 ? 3 : smem <= 110 * 1024 ? 2 : 1;
    const long long units = (long long)((N + G - 1) / G) * C;
    long long g = (long long)sm_count() * bps;
    if (g > units) g = units;
    grid = (int)g;
    return true;
}

size_t clb_convtree_bwd_x_fast_scratch(int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw)
{
    ClsShape s;
    size_t smem;
    int grid;
    if (!plan_bwd_x(s, smem, grid, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, 0)) return 0;
    return 16 + (size_t)grid * 2 * s.G * Ci * H * W * sizeof(float);
}

// Combined fast backward: gx and/or gw (either may be NULL).  Scratch layout:
// [partial gradient tiles: grid*2*G*Ci*H*W floats, only when gx][per-group basis sums: groups*C*28 floats, only when gw].
size_t clb_convtree_bwd_fast_scratch(int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int want_gx,
                                     int want_gw)
{
    ClsShape s;
    size_t smem;
    int grid;
    if (!plan_bwd_x(s, smem, grid, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, 0)) return 0;
    size_t bytes = 16;
    if (want_gx) bytes += (size_t)grid * 2 * s.G * Ci * H * W * sizeof(float);
    if (want_gw) bytes += (size_t)((N + s.G - 1) / s.G) * C * 28 * sizeof(float);
    return bytes;
}

int clb_convtree_bwd_fast_f32(const float *gy, const float *x, const float *w, const int32_t *sel, const uint8_t *amax, float *gx,
                              float *gw, void *scratch, size_t scratch_bytes, int N, int Ci, int H, int W, int C, int sh, int sw, int ph,
                              int pw, int kh, int kw, int wmode, cudaStream_t st)
{
    ClsShape s;
    size_t smem;
    int grid;
    if (amax == nullptr || (!gx && !gw) || !plan_bwd_x(s, smem, grid, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, wmode)) return CLB_ERR_SHAPE;
    const size_t need = clb_convtree_bwd_fast_scratch(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, gx != nullptr, gw != nullptr);
    if (scratch == nullptr || scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 15)) return CLB_ERR_SHAPE;
    const int NG = (s.N + s.G - 1) / s.G;
    float *tiles = (float *)scratch;
    const size_t tile_floats = gx ? (size_t)grid * 2 * s.G * Ci * H * W : 0;
    float *wpartial = tiles + ((tile_floats + 3) / 4) * 4;
    auto launch = [&](auto kern, int threads) {
        if (clb_host::ensure_dynamic_smem(kern, (int)smem) != cudaSuccess) return false;
        CLB_TRACED("convtree_bwd_cls_kernel", st, kern<<<grid, threads, smem, st>>>(gy, x, w, sel, amax, gx, tiles, wpartial, s));
        return true;
    };
    // two windows per thread once a group has more than 128 of them
    const bool two = s.G * ((s.Ho / 2) * (s.Wo / 2)) > kFastThreads / 2;
    bool ok;
    if (gx && gw)
        ok = two ? launch(convtree_bwd_cls_kernel<true, true, 2>, kFastThreads / 2) : launch(convtree_bwd_cls_kernel<true, true, 1>, kFastThreads);
    else if (gx)
        ok = two ? launch(convtree_bwd_cls_kernel<true, false, 2>, kFastThreads / 2) : launch(convtree_bwd_cls_kernel<true, false, 1>, kFastThreads);
    else
        ok = two ? launch(convtree_bwd_cls_kernel<false, true, 2>, kFastThreads / 2) : launch(convtree_bwd_cls_kernel<false, true, 1>, kFastThreads);
    if (!ok) return check_launch(0);
    int launched = 1;
    const int per_group = s.G * s.Ci * s.H * s.W;
    int chunks = (per_group + 1023) / 1024;
    if (chunks > 32) chunks = 32;
    const int ngates = C * 7;
    if (gx && gw && (long long)chunks * NG + (ngates + 31) / 32 < 0x7fffffffLL) {
        CLB_TRACED("convtree_bwd_post_kernel", st, convtree_bwd_post_kernel<<<chunks * NG + (ngates + 31) / 32, 256, 0, st>>>(tiles, gx, s, grid, chunks, NG, wpartial, w, gw, ngates, wmode));
        ++launched;
    } else {
        if (gx) {
            dim3 rgrid(chunks, NG);
            CLB_TRACED("convtree_bwd_x_reduce_kernel", st, convtree_bwd_x_reduce_kernel<<<rgrid, 256, 0, st>>>(tiles, gx, s, grid));
            ++launched;
        }
        if (gw) {
            CLB_TRACED("convtree_gw_finalize_kernel", st, convtree_gw_finalize_kernel<<<(ngates + 31) / 32, 256, 0, st>>>(wpartial, w, gw, NG, ngates, wmode));
            ++launched;
        }
    }
    return check_launch(launched);
}

int clb_convtree_bwd_x_fast_f32(const float *gy, const float *x, const float *w, const int32_t *sel, const uint8_t *amax, float *gx,
                                void *scratch, size_t scratch_bytes, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw,
                                int kh, int kw, int wmode, cudaStream_t st)
{
    return clb_convtree_bwd_fast_f32(gy, x, w, sel, amax, gx, nullptr, scratch, scratch_bytes, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw,
                                     wmode, st);
}
