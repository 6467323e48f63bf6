// Fused ConvLogic block for layers with many input channels (blocks 2-4 of the CIFAR stacks): fp32, stride 1.
//
// An output channel reads only the (normally two) input channels its 8 taps name, so a block owns ONE output
// channel and streams, image by image, just those two channel planes through shared memory.  The planes are
// fetched by the copy engine (TMA, cp.async.bulk.tensor): one elected thread issues a 4-D box load per plane,
//     box = (P columns starting at column -4, R = H + 2*pad rows starting at row -pad, 1 channel, IPW images),
// whose out-of-image elements arrive as zeros -- the padding halo costs no instruction and no bounds test -- into
// a ring of STAGES buffers; arrival is signalled on an mbarrier the consumers poll (bounded).  No thread spends
// instructions on staging, and the loads of the next STAGES-1 images are in flight while one is evaluated.
//
// Forward: a thread owns one COLUMN position ox of one pooled row py of one image, i.e. the two conv positions
// (2py, ox) and (2py+1, ox).  The lanes of a warp are consecutive ox (then py), so a tap is a row-major,
// stride-1 shared load; the row pitch P (a multiple of 4 floats, as the box needs) is chosen so that the pooled rows
// a warp covers fall into disjoint banks.  The 2x2 pool is finished with one shuffle between the lanes ox, ox^1.
//
// Backward, pass 1: a thread owns pooled windows, a warp whole images.  The gate chain is recomputed at the saved
// arg-max position from the staged planes; the 28 gate-gradient basis sums stay in registers until the end; the
// gradient w.r.t. the 8 taps is ADDED INTO a zeroed shared-memory copy of the two planes (one tap after the other,
// __syncwarp between them: within one tap the map window -> pixel is injective), and the two gradient planes of
// (image, output channel) are written out with 128-bit stores.  Pass 2 (plane_sum_kernel) adds, for every input
// channel, the planes of the output channels that read it, in a fixed order: a pure streaming kernel.
// Deterministic, no floating-point atomics.
#include "clb_common.cuh"
#include "clb_tma.cuh"

namespace clb {

constexpr int kPlaneThreads = 128;
constexpr int kPlaneStages = 4;
constexpr int kPlaneLead = 4; // columns in front of the image in a staged row: 16 bytes, so that the box starts aligned

struct PlaneShape {
    int N, Ci, H, W, C, Hp, Wp, Wo, ph, pw, kh, kw;
    int P, R;        // staged row pitch (floats) and rows
    int img_floats;  // R * P
    int slot_floats; // IPW * img_floats rounded up to 32 floats (128 bytes)
    int IPW;         // images per group and iteration
    int TPI;         // threads per image
    int wmode;
};

__device__ int g_plane_error; // set when a bounded wait gave up (never expected); read by clb_plane_error()

struct SlotInfo {
    int slot[8];
    int ch[2];
    int nslot; // 3 = the selection does not fit two staged planes (more channels, or taps outside the window)
};

// channel -> slot map of output channel c's taps; thread `who` fills it.
__device__ __forceinline__ void fill_slots(SlotInfo &si, const int32_t *__restrict__ sel, int c, const PlaneShape &s)
{
    int n = 0, chs[8];
    bool inside = true;
    for (int k = 0; k < 8; ++k) {
        const int word = sel[c * 8 + k];
        const int ch = (word >> 16) & 0xFFFF;
        inside = inside && word >= 0 && ch < s.Ci && ((word >> 8) & 0xFF) < s.kh && (word & 0xFF) < s.kw;
        int slot = -1;
        for (int j = 0; j < n; ++j)
            if (chs[j] == ch) slot = j;
        if (slot < 0) {
            slot = n;
            chs[n++] = ch;
        }
        si.slot[k] = slot;
    }
    si.ch[0] = min(chs[0], s.Ci - 1);
    si.ch[1] = min(chs[n > 1 ? 1 : 0], s.Ci - 1);
    si.nslot = (inside && n <= 2) ? n : 3;
}

// =========================================================================================== forward
__global__ void __launch_bounds__(kPlaneThreads) convtree_fwd_plane_kernel(const __grid_constant__ CUtensorMap xmap, const float *__restrict__ x,
                                                                           const float *__restrict__ w, const int32_t *__restrict__ sel,
                                                                           float *__restrict__ y, uint8_t *__restrict__ amax, PlaneShape s)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full[4][kPlaneStages];
    __shared__ Gate<float> sg[7];
    __shared__ SlotInfo si;
    __shared__ int sabort;

    const int c = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int HW = s.H * s.W, I = s.Hp * s.Wp;
    const bool wide = s.TPI >= kPlaneThreads; // one group of 128 threads; else four independent warps
    const int gid = wide ? 0 : warp, ngroups = wide ? 1 : kPlaneThreads / 32;
    const bool leader = wide ? tid == 0 : lane == 0;

    if (tid < 7) sg[tid] = gate_load<float>(w + ((size_t)c * 7 + tid) * 16, s.wmode);
    if (tid == 32) fill_slots(si, sel, c, s);
    if (tid == 64) {
        for (int g = 0; g < 4; ++g)
            for (int st = 0; st < kPlaneStages; ++st) clb_tma::mbar_init(&full[g][st], 1);
        clb_tma::mbar_init_fence();
        sabort = *reinterpret_cast<volatile int *>(&g_plane_error);
    }
    __syncthreads();
    if (sabort) return; // an earlier block's wait ran out: do not queue more work behind a copy engine that does not answer

    Gate<float> g[7];
#pragma unroll
    for (int i = 0; i < 7; ++i) g[i] = sg[i];
    const int n_lo = (int)((long long)s.N * blockIdx.x / gridDim.x), n_hi = (int)((long long)s.N * (blockIdx.x + 1) / gridDim.x);

    if (si.nslot > 2) {
        // Hand-made selection (more than two channels, or taps outside the window): every tap is a bounds-checked
        // global load.  Block-uniform branch; nothing has been issued to the copy engine.
        for (int f = tid; f < (n_hi - n_lo) * I; f += kPlaneThreads) {
            const int img = f / I, win = f - img * I;
            const int py = win / s.Wp, px = win - py * s.Wp;
            const float *ximg = x + (size_t)(n_lo + img) * s.Ci * HW;
            float best = 0.f;
            int bd = 0;
            for (int d = 0; d < 4; ++d) {
                float a[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const Tap tp = unpack_tap(sel[c * 8 + k], s.ph, s.pw);
                    const int iy = 2 * py + (d >> 1) + tp.dy, ix = 2 * px + (d & 1) + tp.dx;
                    a[k] = ((unsigned)iy < (unsigned)s.H && (unsigned)ix < (unsigned)s.W && tp.ch < s.Ci) ? __ldg(ximg + tp.ch * HW + iy * s.W + ix) : 0.f;
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

    // this thread's place: image `img_local` of the group's batch, pooled row py, column position ox
    const int gt = wide ? tid : lane;
    const int img_local = wide ? 0 : gt / s.TPI;
    const int t = gt - img_local * s.TPI;
    const int py = t / s.Wo, ox = t - py * s.Wo;
    const bool mine = img_local < s.IPW && t < s.TPI;
    const int thr_off = 4 * (img_local * s.img_floats + 2 * py * s.P + ox); // bytes
    int toff[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int word = sel[c * 8 + k];
        toff[k] = 4 * (si.slot[k] * s.slot_floats + ((word >> 8) & 0xFF) * s.P + (word & 0xFF) + kPlaneLead - s.pw) + thr_off;
    }
    const int rowb = 4 * s.P;
    const int ch_a = si.ch[0], ch_b = si.ch[1];

    const int stage_bytes = 2 * s.slot_floats * 4;
    unsigned char *gbase = smem_raw + (size_t)gid * kPlaneStages * stage_bytes;
    const int nbatch = (n_hi - n_lo + s.IPW - 1) / s.IPW;
    const int iters = nbatch > gid ? (nbatch - gid + ngroups - 1) / ngroups : 0;
    const uint32_t tx_bytes = 2u * (uint32_t)(s.IPW * s.img_floats * 4);
    auto issue = [&](int it) {
        const int st = it % kPlaneStages;
        const int n0 = n_lo + (it * ngroups + gid) * s.IPW;
        unsigned char *dst = gbase + (size_t)st * stage_bytes;
        clb_tma::mbar_expect_tx(&full[gid][st], tx_bytes);
        clb_tma::load_box_4d(dst, &xmap, -kPlaneLead, -s.ph, ch_a, n0, &full[gid][st]);
        clb_tma::load_box_4d(dst + s.slot_floats * 4, &xmap, -kPlaneLead, -s.ph, ch_b, n0, &full[gid][st]);
    };
    if (leader)
        for (int it = 0; it < kPlaneStages && it < iters; ++it) issue(it);

    bool failed = false;
    int it = 0;
    for (; it < iters; ++it) {
        const int st = it % kPlaneStages;
        bool ok = clb_tma::mbar_wait(&full[gid][st], (it / kPlaneStages) & 1);
        const unsigned char *tb = gbase + (size_t)st * stage_bytes;
        float z[2];
#pragma unroll
        for (int dy = 0; dy < 2; ++dy) {
            float v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = *reinterpret_cast<const float *>(tb + toff[k] + (dy ? rowb : 0));
            const float g0 = gate_eval<float>(g[0], v[0], v[1]), g1 = gate_eval<float>(g[1], v[2], v[3]);
            const float g2 = gate_eval<float>(g[2], v[4], v[5]), g3 = gate_eval<float>(g[3], v[6], v[7]);
            z[dy] = gate_eval<float>(g[6], gate_eval<float>(g[4], g0, g1), gate_eval<float>(g[5], g2, g3));
        }
        // The tile has been read by the whole group: the leader may refill this stage.  The same vote tells every
        // thread whether anyone's wait ran out (never expected): then nothing of this iteration is stored.
        ok = wide ? (__syncthreads_and(ok ? 1 : 0) != 0) : (__all_sync(0xffffffffu, ok ? 1 : 0) != 0);
        if (!ok) {
            failed = true;
            break;
        }
        if (leader && it + kPlaneStages < iters) issue(it + kPlaneStages);
        // 2x2 pool: lanes ox and ox^1 hold the two columns; candidates in scan order (0,0),(0,1),(1,0),(1,1)
        const float q0 = __shfl_xor_sync(0xffffffffu, z[0], 1), q1 = __shfl_xor_sync(0xffffffffu, z[1], 1);
        const bool odd = ox & 1;
        const float d0 = odd ? q0 : z[0], d1 = odd ? z[0] : q0, d2 = odd ? q1 : z[1], d3 = odd ? z[1] : q1;
        float best = d0;
        int bd = 0;
        if (d1 > best) best = d1, bd = 1; // strict '>' in scan order keeps the first maximum
        if (d2 > best) best = d2, bd = 2;
        if (d3 > best) best = d3, bd = 3;
        const int n = n_lo + (it * ngroups + gid) * s.IPW + img_local;
        if (mine && n < n_hi) {
            const size_t o = ((size_t)n * s.C + c) * I + py * s.Wp + (ox >> 1);
            if (!odd)
                y[o] = best;
            else if (amax != nullptr)
                amax[o] = (uint8_t)bd;
        }
    }
    if (failed && leader) {
        g_plane_error = 1;
        // copies issued for later stages may still be in flight into this block's shared memory: give them a bounded
        // time to land before the block retires
        for (int j = it + 1; j < iters && j < it + kPlaneStages; ++j) clb_tma::mbar_wait(&full[gid][j % kPlaneStages], (j / kPlaneStages) & 1);
    }
}

// ================================================================================== backward, pass 1
// grid (parts, C), 4 warps per block, every warp with its own ring of staged planes.  A warp works on IPW whole
// images per iteration (32 / I of them when an image has I < 32 pooled windows, else one image with WPT = I / 32
// windows per lane).  Per warp: [STAGES x (2 slots of x planes)] + [2 slots of gradient planes].
template <int WPT>
__global__ void __launch_bounds__(kPlaneThreads) convtree_bwd_plane_kernel(const __grid_constant__ CUtensorMap xmap, const float *__restrict__ gy,
                                                                           const float *__restrict__ w, const int32_t *__restrict__ sel,
                                                                           const uint8_t *__restrict__ amax, float *__restrict__ partial,
                                                                           float *__restrict__ planes, PlaneShape s)
{
    constexpr int ST = kPlaneStages - 1; // three stages of input planes + one gradient tile per warp
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full[4][ST];
    __shared__ Gate<float> sg[7];
    __shared__ SlotInfo si;
    __shared__ float red[4][28];
    __shared__ int sabort;

    const int c = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int HW = s.H * s.W, I = s.Hp * s.Wp;
    if (tid < 7) sg[tid] = gate_load<float>(w + ((size_t)c * 7 + tid) * 16, s.wmode);
    if (tid == 32) fill_slots(si, sel, c, s);
    if (tid == 64) {
        for (int g = 0; g < 4; ++g)
            for (int st = 0; st < ST; ++st) clb_tma::mbar_init(&full[g][st], 1);
        clb_tma::mbar_init_fence();
        sabort = *reinterpret_cast<volatile int *>(&g_plane_error);
    }
    __syncthreads();
    if (sabort) return;
    Gate<float> g[7];
#pragma unroll
    for (int i = 0; i < 7; ++i) g[i] = sg[i];
    float acc[28];
#pragma unroll
    for (int i = 0; i < 28; ++i) acc[i] = 0.f;

    const int n_lo = (int)((long long)s.N * blockIdx.x / gridDim.x), n_hi = (int)((long long)s.N * (blockIdx.x + 1) / gridDim.x);
    const int stage_floats = 2 * s.slot_floats, stage_bytes = stage_floats * 4;
    unsigned char *wbase = smem_raw + (size_t)warp * (ST + 1) * stage_bytes;
    float *gt = reinterpret_cast<float *>(wbase + (size_t)ST * stage_bytes);
    for (int i = lane * 4; i < stage_floats; i += 128) *reinterpret_cast<float4 *>(gt + i) = make_float4(0.f, 0.f, 0.f, 0.f);

    // the lane's windows: slot j = lane + 32*j of the warp's (image, window) space
    int img_local[WPT], win[WPT], woff[WPT];
#pragma unroll
    for (int j = 0; j < WPT; ++j) {
        const int f = lane + 32 * j;
        img_local[j] = f / I;
        win[j] = f - img_local[j] * I;
        const int py = win[j] / s.Wp, px = win[j] - py * s.Wp;
        woff[j] = img_local[j] * s.img_floats + 2 * py * s.P + 2 * px;
    }
    int toff[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int word = sel[c * 8 + k];
        toff[k] = si.slot[k] * s.slot_floats + ((word >> 8) & 0xFF) * s.P + (word & 0xFF) + kPlaneLead - s.pw;
    }
    const int ch_a = si.ch[0], ch_b = si.ch[1];
    const bool usable = si.nslot <= 2; // the host only routes selections here that fit two planes

    const int nbatch = (n_hi - n_lo + s.IPW - 1) / s.IPW;
    const int iters = (usable && nbatch > warp) ? (nbatch - warp + 3) / 4 : 0;
    const uint32_t tx_bytes = 2u * (uint32_t)(s.IPW * s.img_floats * 4);
    auto issue = [&](int it) {
        const int st = it % ST;
        const int n0 = n_lo + (it * 4 + warp) * s.IPW;
        unsigned char *dst = wbase + (size_t)st * stage_bytes;
        clb_tma::mbar_expect_tx(&full[warp][st], tx_bytes);
        clb_tma::load_box_4d(dst, &xmap, -kPlaneLead, -s.ph, ch_a, n0, &full[warp][st]);
        clb_tma::load_box_4d(dst + s.slot_floats * 4, &xmap, -kPlaneLead, -s.ph, ch_b, n0, &full[warp][st]);
    };
    if (lane == 0)
        for (int it = 0; it < ST && it < iters; ++it) issue(it);

    // upstream gradient and arg-max of the first iteration; from then on fetched one iteration ahead
    float dz_next[WPT];
    int bd_next[WPT];
    auto fetch = [&](int it) {
#pragma unroll
        for (int j = 0; j < WPT; ++j) {
            const int n = n_lo + (it * 4 + warp) * s.IPW + img_local[j];
            const bool live = it < iters && img_local[j] < s.IPW && n < n_hi;
            const size_t o = ((size_t)n * s.C + c) * I + win[j];
            dz_next[j] = live ? __ldg(gy + o) : 0.f;
            bd_next[j] = live ? (int)__ldg(amax + o) : 0;
        }
    };
    fetch(0);
    // units of the write-out: one float4 of an interior row of (image, slot); the same for every iteration
    const int w4 = s.W >> 2, units = s.IPW * 2 * s.H * w4;

    bool failed = false;
    int it = 0;
    __syncwarp();
    for (; it < iters; ++it) {
        const int st = it % ST;
        float dz[WPT];
        int bd[WPT];
#pragma unroll
        for (int j = 0; j < WPT; ++j) dz[j] = dz_next[j], bd[j] = bd_next[j];
        fetch(it + 1);
        bool ok = clb_tma::mbar_wait(&full[warp][st], (it / ST) & 1);
        ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
        if (!ok) {
            failed = true;
            break;
        }
        const float *xs = reinterpret_cast<const float *>(wbase + (size_t)st * stage_bytes);
        float tg[WPT][8];
        int cell[WPT][8];
#pragma unroll
        for (int j = 0; j < WPT; ++j) {
            const int base = woff[j] + ((bd[j] >> 1) ? s.P : 0) + (bd[j] & 1);
            float a[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                cell[j][k] = base + toff[k];
                a[k] = xs[cell[j][k]];
            }
            const float d = dz[j];
            const float g0 = gate_eval<float>(g[0], a[0], a[1]), g1 = gate_eval<float>(g[1], a[2], a[3]);
            const float g2 = gate_eval<float>(g[2], a[4], a[5]), g3 = gate_eval<float>(g[3], a[6], a[7]);
            const float t0 = gate_eval<float>(g[4], g0, g1), t1 = gate_eval<float>(g[5], g2, g3);
            const float dt0 = d * gate_da<float>(g[6], t1), dt1 = d * gate_db<float>(g[6], t0);
            float dg[4];
            dg[0] = dt0 * gate_da<float>(g[4], g1), dg[1] = dt0 * gate_db<float>(g[4], g0);
            dg[2] = dt1 * gate_da<float>(g[5], g3), dg[3] = dt1 * gate_db<float>(g[5], g2);
            acc[24] = fmaf(d, t0 * t1, acc[24]), acc[25] = fmaf(d, t0, acc[25]), acc[26] = fmaf(d, t1, acc[26]), acc[27] += d;
            acc[16] = fmaf(dt0, g0 * g1, acc[16]), acc[17] = fmaf(dt0, g0, acc[17]), acc[18] = fmaf(dt0, g1, acc[18]), acc[19] += dt0;
            acc[20] = fmaf(dt1, g2 * g3, acc[20]), acc[21] = fmaf(dt1, g2, acc[21]), acc[22] = fmaf(dt1, g3, acc[22]), acc[23] += dt1;
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                acc[4 * p] = fmaf(dg[p], a[2 * p] * a[2 * p + 1], acc[4 * p]);
                acc[4 * p + 1] = fmaf(dg[p], a[2 * p], acc[4 * p + 1]);
                acc[4 * p + 2] = fmaf(dg[p], a[2 * p + 1], acc[4 * p + 2]);
                acc[4 * p + 3] += dg[p];
                tg[j][2 * p] = dg[p] * gate_da<float>(g[p], a[2 * p + 1]);
                tg[j][2 * p + 1] = dg[p] * gate_db<float>(g[p], a[2 * p]);
            }
        }
        // the input planes of this stage have been read by every lane: refill it
        __syncwarp();
        if (lane == 0 && it + ST < iters) issue(it + ST);
        // tap gradients into the gradient planes, one tap at a time (windows of one tap hit distinct pixels; a pixel
        // outside the image is a halo cell that is never written out)
#pragma unroll
        for (int k = 0; k < 8; ++k) {
#pragma unroll
            for (int j = 0; j < WPT; ++j) gt[cell[j][k]] += tg[j][k];
            __syncwarp();
        }
        // write the interior of the gradient planes out and clear it for the next iteration
        const int nb0 = n_lo + (it * 4 + warp) * s.IPW;
        for (int u = lane; u < units; u += 32) {
            const int col4 = u % w4;
            int r = u / w4;
            const int row = r % s.H;
            r /= s.H;
            const int slot = r & 1, img = r >> 1;
            float *src = gt + slot * s.slot_floats + img * s.img_floats + (row + s.ph) * s.P + kPlaneLead + col4 * 4;
            const float4 v = *reinterpret_cast<float4 *>(src);
            *reinterpret_cast<float4 *>(src) = make_float4(0.f, 0.f, 0.f, 0.f);
            if (nb0 + img < n_hi)
                *reinterpret_cast<float4 *>(planes + (((size_t)(nb0 + img) * s.C + c) * 2 + slot) * HW + row * s.W + col4 * 4) = v;
        }
        __syncwarp();
    }
    if (failed && lane == 0) {
        g_plane_error = 1;
        for (int j = it + 1; j < iters && j < it + ST; ++j) clb_tma::mbar_wait(&full[warp][j % ST], (j / ST) & 1);
    }
    if (!usable && tid == 0) g_plane_error = 2;

#pragma unroll
    for (int i = 0; i < 28; ++i) {
        const float v = warp_sum<float>(acc[i]);
        if (lane == 0) red[warp][i] = v;
    }
    __syncthreads();
    if (tid < 28) partial[((size_t)blockIdx.x * s.C + c) * 28 + tid] = (red[0][tid] + red[1][tid]) + (red[2][tid] + red[3][tid]);
}

// Pass 2: gx[n][ch] = sum of the gradient planes (c, slot) that belong to input channel ch, in list order.
// `start` [Ci + 1], `entry` [..] = 2*c + slot.  One float4 per thread; grid-stride over N * Ci * HW / 4.
__global__ void __launch_bounds__(256) plane_sum_kernel(const float *__restrict__ planes, const int32_t *__restrict__ start,
                                                        const int32_t *__restrict__ entry, float *__restrict__ gx, int N, int Ci, int C, int HW4)
{
    const long long total = (long long)N * Ci * HW4;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int e = (int)(i % HW4);
        const long long r = i / HW4;
        const int ch = (int)(r % Ci);
        const long long n = r / Ci;
        const int lo = start[ch], hi = start[ch + 1];
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 *base = reinterpret_cast<const float4 *>(planes) + (size_t)n * C * 2 * HW4 + e;
        int l = lo;
        for (; l + 1 < hi; l += 2) { // two loads in flight
            const float4 a = __ldg(base + (size_t)entry[l] * HW4), b = __ldg(base + (size_t)entry[l + 1] * HW4);
            acc.x += a.x, acc.y += a.y, acc.z += a.z, acc.w += a.w;
            acc.x += b.x, acc.y += b.y, acc.z += b.z, acc.w += b.w;
        }
        if (l < hi) {
            const float4 a = __ldg(base + (size_t)entry[l] * HW4);
            acc.x += a.x, acc.y += a.y, acc.z += a.z, acc.w += a.w;
        }
        reinterpret_cast<float4 *>(gx)[i] = acc;
    }
}

// One thread per gate: adds the per-part basis sums in part order and writes the 16 gradients.
__global__ void plane_gate_finalize_kernel(const float *__restrict__ partial, const float *__restrict__ w, float *__restrict__ gw, int parts,
                                           long long ngates, int wmode)
{
    const long long gi = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gi >= ngates) return;
    float sums[4] = {0.f, 0.f, 0.f, 0.f};
    for (int p = 0; p < parts; ++p) {
        const float4 q = *reinterpret_cast<const float4 *>(partial + ((size_t)p * ngates + gi) * 4);
        sums[0] += q.x, sums[1] += q.y, sums[2] += q.z, sums[3] += q.w;
    }
    gate_grad_store<float>(sums, w + gi * 16, wmode, gw + gi * 16);
}

} // namespace clb

// ================================================================================== host side ====
using namespace clb;
using namespace clb_host;

namespace {

// Row pitch: the smallest multiple of 4 floats that holds lead + image + right halo and keeps the pooled rows (and
// images) one warp covers in disjoint shared-memory banks; the smallest that fits when no such pitch exists nearby.
int pick_pitch(int W, int pw, int R, int lanes_per_row, int rows_per_image, int images_per_warp)
{
    const int need = (W + pw + kPlaneLead + 3) / 4 * 4;
    const int rows = lanes_per_row > 0 ? 32 / lanes_per_row : 1;
    for (int P = need; P < need + 32; P += 4) {
        unsigned used = 0;
        bool ok = true;
        for (int j = 0; j < rows && ok; ++j) {
            const int img = rows_per_image > 0 ? j / rows_per_image : 0, py = rows_per_image > 0 ? j % rows_per_image : j;
            if (img >= images_per_warp) break;
            const int off = (img * R * P + 2 * P * py) & 31;
            for (int l = 0; l < lanes_per_row; ++l) {
                const unsigned bit = 1u << ((off + l) & 31);
                if (used & bit) ok = false;
                used |= bit;
            }
        }
        if (ok) return P;
    }
    return need;
}

// Geometry shared by the forward and backward plans; false when the plane kernels do not cover the shape.
bool plane_geometry(PlaneShape &s, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int wmode)
{
    if (sh != 1 || sw != 1 || N <= 0 || C <= 0 || C > 65535 || (W & 3) || pw > kPlaneLead || Ci > 65535) return false;
    if (tune_get(CLB_TUNE_PLANE_KERNELS) == 0 || clb_tma::encode_tiled_fn() == nullptr) return false;
    s.N = N, s.Ci = Ci, s.H = H, s.W = W, s.C = C, s.ph = ph, s.pw = pw, s.kh = kh, s.kw = kw, s.wmode = wmode;
    const int Ho = conv_out(H, ph, kh, 1), Wo = conv_out(W, pw, kw, 1);
    if (Ho <= 0 || Wo <= 0 || (Ho & 1) || (Wo & 1)) return false;
    // every tap (row < kh, col < kw) of every position must stay inside the staged rows and columns
    if (Ho - 1 + kh - 1 > H + 2 * ph - 1 || Wo - 1 + kw - 1 - pw > W + pw - 1) return false;
    s.Hp = Ho / 2, s.Wp = Wo / 2, s.Wo = Wo;
    s.R = H + 2 * ph;
    return s.R <= 256;
}

bool plan_fwd(PlaneShape &s, size_t &smem, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int wmode)
{
    if (!plane_geometry(s, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, wmode)) return false;
    s.TPI = s.Hp * s.Wo;
    if (s.TPI == kPlaneThreads && s.Wo <= 32)
        s.IPW = 1;
    else if (s.TPI <= 32 && 32 % s.TPI == 0)
        s.IPW = 32 / s.TPI;
    else
        return false;
    s.P = pick_pitch(W, pw, s.R, s.Wo, s.TPI >= 32 ? 0 : s.Hp, s.IPW);
    if (s.P > 256) return false;
    s.img_floats = s.R * s.P;
    s.slot_floats = (s.IPW * s.img_floats + 31) / 32 * 32;
    const int groups = s.TPI >= kPlaneThreads ? 1 : kPlaneThreads / 32;
    smem = (size_t)groups * kPlaneStages * 2 * s.slot_floats * 4;
    return smem <= 100 * 1024;
}

bool plan_bwd(PlaneShape &s, size_t &smem, int &wpt, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int wmode)
{
    if (!plane_geometry(s, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, wmode)) return false;
    const int I = s.Hp * s.Wp;
    if (I >= 32) {
        if (I % 32 || I / 32 > 2) return false;
        wpt = I / 32, s.IPW = 1;
    } else {
        if (32 % I) return false;
        wpt = 1, s.IPW = 32 / I;
    }
    s.TPI = I;
    s.P = (W + pw + kPlaneLead + 3) / 4 * 4;
    s.img_floats = s.R * s.P;
    s.slot_floats = (s.IPW * s.img_floats + 31) / 32 * 32;
    smem = (size_t)(kPlaneThreads / 32) * kPlaneStages * 2 * s.slot_floats * 4; // per warp: 3 input stages + 1 gradient tile
    return smem <= 100 * 1024;
}

int plane_parts(int N, int C, int images_per_block_iteration)
{
    long long parts = ((long long)sm_count() * 16 + C - 1) / C;
    const long long most = N / (4LL * images_per_block_iteration); // at least four iterations per group
    if (parts > most) parts = most;
    if (parts < 1) parts = 1;
    return (int)parts;
}

} // namespace

// Forward of a many-channel layer through the plane kernels; CLB_ERR_SHAPE when they do not cover the shape.
int clb_convtree_fwd_plane_f32(const float *x, const float *w, const int32_t *sel, float *y, uint8_t *amax, int N, int Ci, int H, int W, int C,
                               int sh, int sw, int ph, int pw, int kh, int kw, int wmode, cudaStream_t st)
{
    PlaneShape s;
    size_t smem;
    if (!plan_fwd(s, smem, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, wmode)) return CLB_ERR_SHAPE;
    CUtensorMap map;
    if (!clb_tma::make_plane_map(&map, x, N, Ci, H, W, s.P, s.R, s.IPW)) return CLB_ERR_SHAPE;
    auto k = convtree_fwd_plane_kernel;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return check_launch(0);
    const int groups = s.TPI >= kPlaneThreads ? 1 : kPlaneThreads / 32;
    const int parts = plane_parts(N, C, groups * s.IPW);
    CLB_TRACED("convtree_fwd_plane_kernel", st, k<<<dim3(parts, C), kPlaneThreads, smem, st>>>(map, x, w, sel, y, amax, s));
    return check_launch();
}

// For every input channel the (output channel, slot) planes that hold its gradient: start [Ci + 1], entry = 2*c + slot,
// output channels ascending.  Slot numbering as in fill_slots: the first distinct channel of an output channel's taps is
// slot 0, the second slot 1.  Returns the number of entries, or CLB_ERR_SHAPE when some output channel names more than
// two channels or a tap outside the kh x kw window (such selections take the general kernels), CLB_ERR_ARG on bad input.
extern "C" int clb_conv_channel_lists(const int32_t *sel_host, int C, int Ci, int kh, int kw, int32_t *start, int32_t *entry, int entry_cap)
{
    if (!sel_host || !start || (!entry && entry_cap > 0) || C < 0 || Ci <= 0) return CLB_ERR_ARG;
    for (int ch = 0; ch <= Ci; ++ch) start[ch] = 0;
    // pass 1: count; pass 2: fill (output channels ascending within a channel's list)
    for (int pass = 0; pass < 2; ++pass) {
        for (int c = 0; c < C; ++c) {
            int n = 0, chs[2] = {0, 0};
            for (int k = 0; k < 8; ++k) {
                const int32_t word = sel_host[c * 8 + k];
                const int ch = (word >> 16) & 0xFFFF;
                if (word < 0 || ch >= Ci || ((word >> 8) & 0xFF) >= kh || (word & 0xFF) >= kw) return CLB_ERR_SHAPE;
                bool seen = false;
                for (int j = 0; j < n; ++j) seen = seen || chs[j] == ch;
                if (!seen) {
                    if (n == 2) return CLB_ERR_SHAPE;
                    chs[n++] = ch;
                }
            }
            for (int j = 0; j < n; ++j) {
                if (pass == 0)
                    ++start[chs[j] + 1];
                else {
                    const int at = start[chs[j]]++;
                    if (at >= entry_cap) return CLB_ERR_SCRATCH;
                    entry[at] = 2 * c + j;
                }
            }
        }
        if (pass == 0) {
            for (int ch = 0; ch < Ci; ++ch) start[ch + 1] += start[ch]; // counts -> start[ch] = begin of channel ch's list
        } else {
            for (int ch = Ci; ch > 0; --ch) start[ch] = start[ch - 1];   // the fill advanced every begin to its end: shift back
            start[0] = 0;
        }
    }
    return start[Ci];
}

extern "C" size_t clb_convtree_bwd_plane_scratch_bytes(int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int dtype)
{
    PlaneShape s;
    size_t smem;
    int wpt;
    if (dtype != CLB_F32 || !conv_args_ok(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw) || !plan_bwd(s, smem, wpt, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, 0))
        return 0;
    const int parts = plane_parts(N, C, (kPlaneThreads / 32) * s.IPW);
    const size_t partial = ((size_t)parts * C * 28 * sizeof(float) + 255) / 256 * 256;
    return partial + (size_t)N * C * 2 * H * W * sizeof(float);
}

extern "C" int clb_convtree_bwd_plane(const void *gy, const void *x, const void *w, const int32_t *sel, const uint8_t *amax, void *gx, void *gw,
                                      const int32_t *ch_start, const int32_t *ch_entry, void *scratch, size_t scratch_bytes, int N, int Ci, int H,
                                      int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int wmode, int dtype, void *stream)
{
    if (!gy || !x || !w || !sel || !amax || !gx || !ch_start || !ch_entry || !scratch || wmode < 0 || wmode > 2) return CLB_ERR_ARG;
    if (dtype != CLB_F32 || !conv_args_ok(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw)) return CLB_ERR_SHAPE;
    PlaneShape s;
    size_t smem;
    int wpt;
    if (!plan_bwd(s, smem, wpt, N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, wmode)) return CLB_ERR_SHAPE;
    const size_t need = clb_convtree_bwd_plane_scratch_bytes(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, dtype);
    if (scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 15) || (reinterpret_cast<uintptr_t>(gx) & 15)) return CLB_ERR_SCRATCH;
    CUtensorMap map;
    if (!clb_tma::make_plane_map(&map, (const float *)x, N, Ci, H, W, s.P, s.R, s.IPW)) return CLB_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    const int parts = plane_parts(N, C, (kPlaneThreads / 32) * s.IPW);
    float *partial = (float *)scratch;
    float *planes = (float *)((unsigned char *)scratch + ((size_t)parts * C * 28 * sizeof(float) + 255) / 256 * 256);
    auto go = [&](auto k) {
        if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return false;
        CLB_TRACED("convtree_bwd_plane_kernel", st,
                   k<<<dim3(parts, C), kPlaneThreads, smem, st>>>(map, (const float *)gy, (const float *)w, sel, amax, partial, planes, s));
        return true;
    };
    if (!(wpt == 1 ? go(convtree_bwd_plane_kernel<1>) : go(convtree_bwd_plane_kernel<2>))) return check_launch(0);
    int launched = 1;
    const int HW4 = H * W / 4;
    const long long total = (long long)N * Ci * HW4;
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)sm_count() * 32;
    if (blocks > cap) blocks = cap;
    CLB_TRACED("plane_sum_kernel", st, plane_sum_kernel<<<(unsigned)blocks, 256, 0, st>>>(planes, ch_start, ch_entry, (float *)gx, N, Ci, C, HW4));
    ++launched;
    if (gw) {
        const long long ngates = (long long)C * 7;
        CLB_TRACED("plane_gate_finalize_kernel", st,
                   plane_gate_finalize_kernel<<<(int)((ngates + 127) / 128), 128, 0, st>>>(partial, (const float *)w, (float *)gw, parts, ngates, wmode));
        ++launched;
    }
    return check_launch(launched);
}

// Diagnostic: the device-side flag a plane kernel sets when one of its bounded waits ran out (0 = never).  Synchronises.
extern "C" int clb_plane_error(int *flag)
{
    if (!flag) return CLB_ERR_ARG;
    if (cudaMemcpyFromSymbol(flag, g_plane_error, sizeof(int)) != cudaSuccess) return check_launch(0);
    return CLB_OK;
}
