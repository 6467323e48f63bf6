// Fused ConvLogic block for layers with many input channels (blocks 2-4 of the CIFAR stacks): fp32, stride 1,
// 3x3 window, padding 1, square images of 16, 8 or 4 pixels (other shapes take the kernels of convtree_fast.cu /
// convtree.cu).
//
// An output channel reads only the (normally two) input channels its 8 taps name, so a block owns ONE output
// channel and streams, image by image, just those two channel planes through shared memory.  The planes are
// fetched by the copy engine (TMA, cp.async.bulk.tensor): one elected thread issues a 4-D box load per plane,
//     box = (P columns starting at column -4, R = H + 2 rows starting at row -1, 1 channel, NIMG images),
// whose out-of-image elements arrive as zeros -- the padding halo costs no instruction and no bounds test -- into
// a ring of buffers; arrival is signalled on an mbarrier the consumers poll (bounded).  No thread spends an
// instruction on staging, and the loads of the next images are in flight while one is evaluated.  The geometry is
// a template parameter, so every shared-memory access is  [per-thread register + immediate].
//
// Forward: a thread owns one COLUMN position ox of one pooled row py of an image PAIR, i.e. the conv positions
// (2py, ox) and (2py+1, ox) of two images.  The lanes of a warp are consecutive ox (then py), so a tap is a
// row-major, stride-1, conflict-free shared load (the row pitch P keeps the pooled rows of a warp in disjoint banks);
// the two images of a pair are packed into one 64-bit register and the gate polynomials run as packed two-float FMAs
// (fma.rn.f32x2: two independent IEEE FMAs, so the values are the scalar kernels' bit for bit).  The 2x2 pool is
// finished with a shuffle between the lanes ox and ox^1.
//
// Backward, pass 1: a thread owns pooled windows, a warp whole images.  The gate chain is recomputed at the saved
// arg-max position from the staged planes; the 28 gate-gradient basis sums stay in registers until the end; the
// gradient w.r.t. the 8 taps is ADDED INTO a shared-memory copy of the two planes (one tap after the other, __syncwarp
// between them: within one tap the map window -> pixel is injective), and the two gradient planes of (image, output
// channel) are written out with 128-bit stores.  Pass 2 (plane_sum_kernel) adds, for every input channel, the planes of
// the output channels that read it, in a fixed order: a pure streaming kernel.  Deterministic, no float atomics.
#include "clb_common.cuh"
#include "clb_tma.cuh"

namespace clb {
namespace plane {

constexpr int kThreads = 128;
constexpr int kLead = 4; // columns in front of the image in a staged row: 16 bytes, so that the box starts aligned

// Geometry of a square S x S layer (3x3 window, padding 1): staged pitch P, rows R, images per box.
template <int S> struct Geo;
// The forward kernel's tile may have its own pitch and plane size (FWD_P, FWD_IMG >= R * FWD_P): a warp's lanes are
// (image pair, pooled row, column), and the pitch and the distance between pairs are chosen so that the 32 lanes of a tap
// load fall into 32 different banks.  16x16: 2 rows x 16 columns, rows 48 floats apart (bank 16).  8x8: 4 rows x 8 columns,
// rows 40 apart (banks 0, 8, 16, 24).  4x4: 4 pairs x 2 rows x 4 columns; rows 16 apart (pitch 8: the right halo of a row is
// the always-zero lead cell of the next one), pairs 68 apart (banks 0, 4, 8, 12), a pair being images p and p + 4 of the
// warp's eight.
template <> struct Geo<16> {
    static constexpr int P = 24, R = 18, FWD_NIMG = 2, BWD_NIMG = 1, BWD_WPT = 2, FWD_P = 24, FWD_IMG = 18 * 24;
};
template <> struct Geo<8> {
    static constexpr int P = 20, R = 10, FWD_NIMG = 2, BWD_NIMG = 2, BWD_WPT = 1, FWD_P = 20, FWD_IMG = 10 * 20;
};
template <> struct Geo<4> {
    static constexpr int P = 12, R = 6, FWD_NIMG = 8, BWD_NIMG = 8, BWD_WPT = 1, FWD_P = 8, FWD_IMG = 68;
};

struct Args {
    int N, Ci, C, wmode;
    int parts; // the batch is split into this many contiguous parts; a (channel, part) pair is one task
    int y_fm;  // the block's output (forward) / upstream gradient (backward) is feature-major: [C][windows][N] instead of
               // [N][C][windows] -- the layout the flat layers behind the last block work in; the arg-max bytes keep [N][C][windows]
};

__device__ int g_plane_error; // set when a bounded wait gave up (never expected); read by clb_plane_error()

struct SlotInfo {
    int slot[8];
    int ch[2];
    int nslot; // 3 = the selection does not fit two staged planes (more channels, or taps outside the 3x3 window)
};

// channel -> slot map of output channel c's taps (one thread fills it)
__device__ __forceinline__ void fill_slots(SlotInfo &si, const int32_t *__restrict__ sel, int c, int Ci)
{
    int n = 0, chs[8];
    bool inside = true;
    for (int k = 0; k < 8; ++k) {
        const int word = sel[c * 8 + k];
        const int ch = (word >> 16) & 0xFFFF;
        inside = inside && word >= 0 && ch < Ci && ((word >> 8) & 0xFF) < 3 && (word & 0xFF) < 3;
        int slot = -1;
        for (int j = 0; j < n; ++j)
            if (chs[j] == ch) slot = j;
        if (slot < 0) {
            slot = n;
            chs[n++] = ch;
        }
        si.slot[k] = slot;
    }
    si.ch[0] = min(chs[0], Ci - 1);
    si.ch[1] = min(chs[n > 1 ? 1 : 0], Ci - 1);
    si.nslot = (inside && n <= 2) ? n : 3;
}

typedef unsigned long long f32x2; // two floats in one 64-bit register
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c)
{
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
// volatile: computed once and kept, never re-materialised in front of every use
__device__ __forceinline__ f32x2 dup2(float v)
{
    f32x2 d;
    asm volatile("mov.b64 %0, {%1, %1};" : "=l"(d) : "r"(__float_as_uint(v)));
    return d;
}
struct Gate2 {
    f32x2 k1, ka, kb, kab;
};
__device__ __forceinline__ f32x2 gate_eval2(const Gate2 &g, f32x2 a, f32x2 b) { return fma2(a, fma2(g.kab, b, g.ka), fma2(g.kb, b, g.k1)); }
__device__ __forceinline__ float lo_of(f32x2 v) { return __uint_as_float((unsigned)v); }
__device__ __forceinline__ float hi_of(f32x2 v) { return __uint_as_float((unsigned)(v >> 32)); }

// {shared[addr + OFF], shared[addr + OFF + SECOND]} as one packed pair; addr is a 32-bit shared-memory address
template <int OFF, int SECOND> __device__ __forceinline__ f32x2 lds_pair(uint32_t addr)
{
    f32x2 v;
    asm volatile("{\n\t.reg .b32 a, b;\n\tld.shared.b32 a, [%1+%2];\n\tld.shared.b32 b, [%1+%3];\n\tmov.b64 %0, {a, b};\n\t}"
                 : "=l"(v)
                 : "r"(addr), "n"(OFF), "n"(OFF + SECOND));
    return v;
}
template <int OFF> __device__ __forceinline__ float lds_f32(uint32_t addr)
{
    float v;
    asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF> __device__ __forceinline__ void sts_f32(uint32_t addr, float v)
{
    asm volatile("st.shared.f32 [%0+%1], %2;" ::"r"(addr), "n"(OFF), "f"(v) : "memory");
}

template <int OFF> __device__ __forceinline__ float4 lds_v4(uint32_t addr)
{
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4+%5];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF> __device__ __forceinline__ void sts_v4_zero(uint32_t addr)
{
    asm volatile("st.shared.v4.f32 [%0+%1], {%2, %2, %2, %2};" ::"r"(addr), "n"(OFF), "f"(0.f) : "memory");
}

// 16-byte asynchronous copy global -> shared (L2 only), commit / wait of the calling thread's copy groups
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
template <int OFF> __device__ __forceinline__ void cp_async16_off(uint32_t dst, const void *src)
{
    asm volatile("cp.async.cg.shared.global [%0+%2], [%1], 16;" ::"r"(dst), "l"(src), "n"(OFF) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory"); }

// How the planes reach shared memory.  16x16 images: TMA box loads (one elected thread, halo zero-filled by the copy
// engine).  8x8 and 4x4 images: the copy engine handles a box row by row at a few cycles per row, and rows of 32 or 16
// useful bytes make it the bottleneck (measured: 290-300 us per layer against 230-240 us for register staging); there
// every thread of the group issues two 16-byte cp.async copies per iteration into the interior of a tile whose halo was
// zeroed once.
template <int S> struct UseTma {
    static constexpr bool value = S >= 16;
};

// =========================================================================================== forward
template <int S> struct FwdCfg {
    using G = Geo<S>;
    static constexpr int P = G::FWD_P, R = G::R, NIMG = G::FWD_NIMG;
    static constexpr int WO = S, HP = S / 2, WP = S / 2, I = HP * WP;
    static constexpr int TPI = HP * WO;                          // threads per image pair
    static constexpr bool WIDE = TPI >= kThreads;                // one group of 128 threads, else four warps on their own
    static constexpr int GROUPS = WIDE ? 1 : kThreads / 32;
    static constexpr int IMG = G::FWD_IMG;                       // floats of one staged plane (R * P + padding)
    static constexpr int SLOT = (NIMG * IMG + 31) / 32 * 32;     // floats of one slot (NIMG planes of one channel)
    static constexpr int STAGE_BYTES = 2 * SLOT * 4;
    static constexpr bool TMA = UseTma<S>::value;
    // pair p of a group = images (2p, 2p + 1) of its batch, or (p, p + NIMG / 2) when several pairs share a warp
    static constexpr bool SPLIT_PAIRS = NIMG > 2;
    static constexpr int PAIR_STRIDE = SPLIT_PAIRS ? IMG : 2 * IMG, SECOND = SPLIT_PAIRS ? (NIMG / 2) * IMG : IMG;
    static_assert(IMG >= R * P && IMG % 4 == 0 && P % 4 == 0 && (!TMA || IMG == R * P), "tile geometry");
    static constexpr int STAGES = TMA ? 4 : 3;
    static constexpr int SMEM = GROUPS * STAGES * STAGE_BYTES;
    static constexpr int GSIZE = WIDE ? kThreads : 32;
    static constexpr int CPQ = NIMG * 2 * S * (S / 4) / GSIZE;   // 16-byte copies per thread and iteration (cp.async staging)
    static_assert(WIDE ? (TPI == kThreads && NIMG == 2) : (32 % TPI == 0 && NIMG == 2 * (32 / TPI)), "thread mapping");
    static_assert(NIMG * 2 * S * (S / 4) % GSIZE == 0, "copies per thread");
};

// One stage of the ring: both conv rows of both images of the thread's pair.
template <int S, int ST> __device__ __forceinline__ void fwd_stage(const uint32_t (&toff)[8], const Gate2 (&g)[7], f32x2 (&z)[2])
{
    using Cf = FwdCfg<S>;
    constexpr int B = ST * Cf::STAGE_BYTES, ROWB = Cf::P * 4, IMGB = Cf::SECOND * 4;
    {
        f32x2 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = lds_pair<B, IMGB>(toff[k]);
        const f32x2 g0 = gate_eval2(g[0], v[0], v[1]), g1 = gate_eval2(g[1], v[2], v[3]);
        const f32x2 g2 = gate_eval2(g[2], v[4], v[5]), g3 = gate_eval2(g[3], v[6], v[7]);
        z[0] = gate_eval2(g[6], gate_eval2(g[4], g0, g1), gate_eval2(g[5], g2, g3));
    }
    {
        f32x2 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = lds_pair<B + ROWB, IMGB>(toff[k]);
        const f32x2 g0 = gate_eval2(g[0], v[0], v[1]), g1 = gate_eval2(g[1], v[2], v[3]);
        const f32x2 g2 = gate_eval2(g[2], v[4], v[5]), g3 = gate_eval2(g[3], v[6], v[7]);
        z[1] = gate_eval2(g[6], gate_eval2(g[4], g0, g1), gate_eval2(g[5], g2, g3));
    }
}

template <int S>
__global__ void __launch_bounds__(kThreads) convtree_fwd_plane_kernel(const __grid_constant__ CUtensorMap xmap, const float *__restrict__ x,
                                                                      const float *__restrict__ w, const int32_t *__restrict__ sel,
                                                                      float *__restrict__ y, uint8_t *__restrict__ amax, Args s)
{
    using Cf = FwdCfg<S>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full[Cf::GROUPS][Cf::STAGES];
    __shared__ Gate<float> sgs[Cf::GROUPS][7];
    __shared__ SlotInfo sis[Cf::GROUPS];
    __shared__ int saborts[Cf::GROUPS];

    // A group is the unit that shares a ring of staged planes: the whole block (16x16 images: 128 threads per image
    // pair) or one warp (smaller images).  Every group works on its own task = (output channel, part of the batch),
    // so with warp groups nothing in this kernel synchronises the block.
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int HW = S * S, I = Cf::I;
    const int gid = Cf::WIDE ? 0 : warp;
    const int gt = Cf::WIDE ? tid : lane;                 // thread index inside the group
    constexpr int GSIZE = Cf::WIDE ? kThreads : 32;
    const bool leader = gt == 0;
    const long long task = (long long)blockIdx.x * Cf::GROUPS + gid;
    if (task >= (long long)s.C * s.parts) return;         // a whole group leaves together
    const int c = (int)(task % s.C), part = (int)(task / s.C);
    auto group_sync = [&]() {
        if (Cf::WIDE)
            __syncthreads();
        else
            __syncwarp();
    };
    Gate<float> *sg = sgs[gid];
    SlotInfo &si = sis[gid];

    if (gt < 7) sg[gt] = gate_load<float>(w + ((size_t)c * 7 + gt) * 16, s.wmode);
    if (gt == (Cf::WIDE ? 32 : 8)) fill_slots(si, sel, c, s.Ci);
    if (gt == (Cf::WIDE ? 64 : 9)) {
        for (int st = 0; st < Cf::STAGES; ++st) clb_tma::mbar_init(&full[gid][st], 1);
        clb_tma::mbar_init_fence();
        saborts[gid] = *reinterpret_cast<volatile int *>(&g_plane_error);
    }
    group_sync();
    if (saborts[gid]) return; // an earlier wait ran out: do not queue more work behind a copy engine that does not answer

    const int n_lo = (int)((long long)s.N * part / s.parts), n_hi = (int)((long long)s.N * (part + 1) / s.parts);

    if (si.nslot > 2) {
        // Hand-made selection (more than two channels, or taps outside the window): every tap is a bounds-checked
        // global load.  Block-uniform branch; nothing has been issued to the copy engine.
        Gate<float> g[7];
#pragma unroll
        for (int i = 0; i < 7; ++i) g[i] = sg[i];
        for (int f = gt; f < (n_hi - n_lo) * I; f += GSIZE) {
            const int img = f / I, win = f - img * I;
            const int py = win / Cf::WP, px = win - py * Cf::WP;
            const float *ximg = x + (size_t)(n_lo + img) * s.Ci * HW;
            float best = 0.f;
            int bd = 0;
            for (int d = 0; d < 4; ++d) {
                float a[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const Tap tp = unpack_tap(sel[c * 8 + k], 1, 1);
                    const int iy = 2 * py + (d >> 1) + tp.dy, ix = 2 * px + (d & 1) + tp.dx;
                    a[k] = ((unsigned)iy < (unsigned)S && (unsigned)ix < (unsigned)S && tp.ch < s.Ci) ? __ldg(ximg + tp.ch * HW + iy * S + ix) : 0.f;
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
            y[s.y_fm ? ((size_t)c * I + win) * s.N + (n_lo + img) : o] = best;
            if (amax != nullptr) amax[o] = (uint8_t)bd;
        }
        return;
    }

    Gate2 g[7];
#pragma unroll
    for (int i = 0; i < 7; ++i) g[i].k1 = dup2(sg[i].k1), g[i].ka = dup2(sg[i].ka), g[i].kb = dup2(sg[i].kb), g[i].kab = dup2(sg[i].kab);

    // this thread's place: pair `pair_local` of the group's batch, pooled row py, column position ox
    const int pair_local = gt / Cf::TPI;
    const int t = gt - pair_local * Cf::TPI;
    const int py = t / Cf::WO, ox = t - py * Cf::WO;
    unsigned char *gbase = smem_raw + (size_t)gid * Cf::STAGES * Cf::STAGE_BYTES;
    const uint32_t thr = clb_tma::smem_addr(gbase) + 4u * (uint32_t)(pair_local * Cf::PAIR_STRIDE + 2 * py * Cf::P + ox);
    uint32_t toff[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int word = sel[c * 8 + k];
        toff[k] = thr + 4u * (uint32_t)(si.slot[k] * Cf::SLOT + ((word >> 8) & 0xFF) * Cf::P + (word & 0xFF) + kLead - 1);
    }
    const int ch_a = si.ch[0], ch_b = si.ch[1];

    const int iters = (n_hi - n_lo + Cf::NIMG - 1) / Cf::NIMG;
    constexpr uint32_t tx_bytes = 2u * (uint32_t)(Cf::NIMG * Cf::IMG * 4);
    auto issue = [&](int it) {
        const int st = it % Cf::STAGES;
        const int n0 = n_lo + it * Cf::NIMG;
        unsigned char *dst = gbase + (size_t)st * Cf::STAGE_BYTES;
        clb_tma::mbar_expect_tx(&full[gid][st], tx_bytes);
        clb_tma::load_box_4d(dst, &xmap, -kLead, -1, ch_a, n0, &full[gid][st]);
        clb_tma::load_box_4d(dst + Cf::SLOT * 4, &xmap, -kLead, -1, ch_b, n0, &full[gid][st]);
    };
    // cp.async staging: which 16-byte pieces this thread moves is the same for every iteration; the source pointers run
    // along with the iterations (NIMG images further each time), cp_iters = iterations in which the piece's image exists
    const float *csrc[Cf::CPQ];
    int cp_iters[Cf::CPQ];
    uint32_t cdst[Cf::CPQ];
#pragma unroll
    for (int q = 0; q < Cf::CPQ; ++q) {
        const int u = gt + q * Cf::GSIZE;
        constexpr int W4 = S / 4;
        const int col4 = u % W4, row = (u / W4) % S, slot = (u / (W4 * S)) & 1, img = u / (W4 * S * 2);
        csrc[q] = x + ((size_t)(n_lo + img) * s.Ci + (slot ? ch_b : ch_a)) * HW + row * S + col4 * 4;
        cp_iters[q] = (n_hi - n_lo - img + Cf::NIMG - 1) / Cf::NIMG;
        cdst[q] = clb_tma::smem_addr(gbase) + 4u * (uint32_t)(slot * Cf::SLOT + img * Cf::IMG + (row + 1) * Cf::P + kLead + col4 * 4);
    }
    const size_t cstep = (size_t)Cf::NIMG * s.Ci * HW;
    // Called once per iteration in rising order (the pointers advance); always commits, so that the group counts stay
    // aligned.  An image past the end of the part is not fetched: its slot keeps older (finite) data that is never stored.
#define CLB_FWD_ISSUE_CP(ST, IT)                                                                                          \
    {                                                                                                                     \
        _Pragma("unroll") for (int q = 0; q < Cf::CPQ; ++q)                                                               \
        {                                                                                                                 \
            if ((IT) < cp_iters[q]) cp_async16_off<(ST) * Cf::STAGE_BYTES>(cdst[q], csrc[q]);                             \
            csrc[q] += cstep;                                                                                             \
        }                                                                                                                 \
        cp_async_commit();                                                                                                \
    }
    if (Cf::TMA) {
        if (leader)
            for (int it = 0; it < Cf::STAGES && it < iters; ++it) issue(it);
    } else {
        // the halo is zeroed once; the copies only ever write the interior
        for (int i = gt * 4; i < Cf::STAGES * Cf::STAGE_BYTES / 4; i += Cf::GSIZE * 4)
            *reinterpret_cast<float4 *>(reinterpret_cast<float *>(gbase) + i) = make_float4(0.f, 0.f, 0.f, 0.f);
        group_sync();
        CLB_FWD_ISSUE_CP(0, 0)
        CLB_FWD_ISSUE_CP(1, 1)
        CLB_FWD_ISSUE_CP(2, 2)
        static_assert(Cf::TMA || Cf::STAGES == 3, "prologue of the cp.async ring");
    }

    // 2x2 pool: lanes ox and ox^1 hold the two columns of a window, each for both images of the pair.  The even lane
    // pools and stores the pair's first image, the odd lane the second; each hands the other the half it does not need.
    const bool odd = ox & 1;
    const int my_img = Cf::SPLIT_PAIRS ? pair_local + (odd ? Cf::NIMG / 2 : 0) : 2 * pair_local + (odd ? 1 : 0);
    const int my_iters = (n_hi - n_lo - my_img + Cf::NIMG - 1) / Cf::NIMG;   // iterations in which that image exists
    const size_t o0 = ((size_t)(n_lo + my_img) * s.C + c) * I + py * Cf::WP + (ox >> 1);
    const size_t ostep = (size_t)Cf::NIMG * s.C * I;
    const bool want_amax = amax != nullptr;
    float *yp = y + (s.y_fm ? ((size_t)c * I + py * Cf::WP + (ox >> 1)) * s.N + (n_lo + my_img) : o0); // run along with the iterations
    const size_t ystep = s.y_fm ? (size_t)Cf::NIMG : ostep;
    uint8_t *ap = want_amax ? amax + o0 : nullptr;
    bool failed = false;
    int it = 0;
    auto pool_store = [&](const f32x2(&z)[2]) {
        const float m0 = odd ? hi_of(z[0]) : lo_of(z[0]), m1 = odd ? hi_of(z[1]) : lo_of(z[1]);   // my image, my column
        const float t0 = odd ? lo_of(z[0]) : hi_of(z[0]), t1 = odd ? lo_of(z[1]) : hi_of(z[1]);   // the other lane's image
        const float r0 = __shfl_xor_sync(0xffffffffu, t0, 1), r1 = __shfl_xor_sync(0xffffffffu, t1, 1); // my image, other column
        // candidates in scan order (0,0),(0,1),(1,0),(1,1); the even lane holds the even column
        const float c0 = odd ? r0 : m0, c1 = odd ? m0 : r0, c2 = odd ? r1 : m1, c3 = odd ? m1 : r1;
        float best = c0;
        int bd = 0;
        if (c1 > best) best = c1, bd = 1; // strict '>' in scan order keeps the first maximum
        if (c2 > best) best = c2, bd = 2;
        if (c3 > best) best = c3, bd = 3;
        if (it < my_iters) {
            *yp = best;
            if (want_amax) *ap = (uint8_t)bd;
        }
        yp += ystep;
        if (want_amax) ap += ostep;
    };
    // the ring is walked with the stage index as a compile-time constant: every load is [register + immediate]
    while (it < iters && !failed) {
        const uint32_t parity = (it / Cf::STAGES) & 1;
#define CLB_FWD_STAGE(ST)                                                                                                 \
    if (it < iters && !failed) {                                                                                          \
        bool ok = true;                                                                                                   \
        if constexpr (Cf::TMA) {                                                                                          \
            ok = clb_tma::mbar_wait(&full[gid][ST], parity);                                                              \
        } else {                                                                                                          \
            cp_async_wait<Cf::STAGES - 1>();                                                                              \
            group_sync(); /* the other threads' pieces of this stage are visible */                                      \
        }                                                                                                                 \
        f32x2 z[2];                                                                                                       \
        fwd_stage<S, ST>(toff, g, z);                                                                                     \
        /* The tile has been read by the whole group: refill this stage.  With TMA the same vote tells every thread    */ \
        /* whether anyone's wait ran out (never expected): then nothing of this iteration is stored.                   */ \
        if constexpr (Cf::TMA) {                                                                                          \
            ok = Cf::WIDE ? (__syncthreads_and(ok ? 1 : 0) != 0) : (__all_sync(0xffffffffu, ok ? 1 : 0) != 0);            \
            if (!ok)                                                                                                      \
                failed = true;                                                                                            \
            else if (leader && it + Cf::STAGES < iters)                                                                   \
                issue(it + Cf::STAGES);                                                                                   \
        } else {                                                                                                          \
            group_sync();                                                                                                 \
            CLB_FWD_ISSUE_CP(ST, it + Cf::STAGES)                                                                         \
        }                                                                                                                 \
        if (!failed) {                                                                                                    \
            pool_store(z);                                                                                                \
            ++it;                                                                                                         \
        }                                                                                                                 \
    }
        CLB_FWD_STAGE(0)
        CLB_FWD_STAGE(1)
        CLB_FWD_STAGE(2)
        if constexpr (Cf::STAGES > 3) {
            CLB_FWD_STAGE(3)
        }
#undef CLB_FWD_STAGE
#undef CLB_FWD_ISSUE_CP
    }
    if (failed && leader) {
        g_plane_error = 1;
        // copies issued for later stages may still be in flight into this block's shared memory: give them a bounded
        // time to land before the block retires
        for (int j = it + 1; j < iters && j < it + Cf::STAGES; ++j) clb_tma::mbar_wait(&full[gid][j % Cf::STAGES], (j / Cf::STAGES) & 1);
    }
}

// ================================================================================== backward, pass 1
// 4 warps per block, every warp with its own task = (output channel, part of the batch), its own ring of staged
// planes and its own gradient tile: nothing synchronises the block.  A warp works on NIMG whole images per iteration
// (32 / I of them when an image has I < 32 pooled windows, else one image with WPT = I / 32 windows per lane).
// Per warp: [XST stages x (2 slots of x planes)] + [2 slots of gradient planes].
template <int S> struct BwdCfg {
    using G = Geo<S>;
    static constexpr int P = G::P, R = G::R, NIMG = G::BWD_NIMG, WPT = G::BWD_WPT;
    static constexpr int HP = S / 2, WP = S / 2, I = HP * WP;
    static constexpr int IMG = R * P;
    static constexpr int SLOT = (NIMG * IMG + 31) / 32 * 32;
    static constexpr int STAGE_FLOATS = 2 * SLOT, STAGE_BYTES = STAGE_FLOATS * 4;
    static constexpr int XST = 3;                       // stages of input planes
    static constexpr int GT_BYTES = XST * STAGE_BYTES;  // byte distance from stage 0 to the gradient tile: the same cell offsets
    static constexpr int WARP_BYTES = (XST + 1) * STAGE_BYTES;
    static constexpr int SMEM = (kThreads / 32) * WARP_BYTES;
    static constexpr int UNITS = NIMG * 2 * S * (S / 4); // float4 units of the interior of the gradient tile (and of a stage)
    static constexpr bool TMA = UseTma<S>::value;
    static_assert(I >= 32 ? (NIMG == 1 && WPT * 32 == I) : (WPT == 1 && NIMG * I == 32), "thread mapping");
    static_assert(UNITS % 32 == 0, "write-out units per lane");
};

// The lane's WPT windows at their arg-max positions: gate chain, basis sums, tap gradients added into the gradient tile.
template <int S, int ST, int WPT>
__device__ __forceinline__ void bwd_windows(const uint32_t (&base)[WPT], const uint32_t (&toff)[8], const Gate<float> (&g)[7],
                                            const float (&dz)[WPT], float (&acc)[28])
{
    using Cf = BwdCfg<S>;
    constexpr int B = ST * Cf::STAGE_BYTES, GT = Cf::GT_BYTES;
    uint32_t cell[WPT][8];
    float tg[WPT][8];
#pragma unroll
    for (int j = 0; j < WPT; ++j) {
        float a[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            cell[j][k] = base[j] + toff[k];
            a[k] = lds_f32<B>(cell[j][k]);
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
    // (Skipping the accesses of taps that repeat an earlier tap's cell -- about one tap in six with 8 taps over 18 cells --
    // was measured slower in both forms tried: warp-uniform branches around each access break the batching of the loads,
    // 0.78 -> 0.92 ms per step at batch 256; predicated accesses with select chains cost a block per SM in registers, 1.00 ms.)
    // One tap at a time: all windows of a warp (both of a lane included) hit distinct pixels within one tap -- the map
    // window -> pixel is a translation of the window grid -- and a pixel outside the image is a halo cell that is never
    // written out.  The order of additions into a pixel is the tap order: fixed.
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        float cur[WPT];
#pragma unroll
        for (int j = 0; j < WPT; ++j) cur[j] = lds_f32<GT>(cell[j][k]);
#pragma unroll
        for (int j = 0; j < WPT; ++j) sts_f32<GT>(cell[j][k], cur[j] + tg[j][k]);
        __syncwarp();
    }
}

template <int S, bool FM>
__global__ void __launch_bounds__(kThreads) convtree_bwd_plane_kernel(const __grid_constant__ CUtensorMap xmap, const float *__restrict__ gy,
                                                                      const float *__restrict__ x, const float *__restrict__ w,
                                                                      const int32_t *__restrict__ sel, const uint8_t *__restrict__ amax,
                                                                      float *__restrict__ partial, float *__restrict__ planes, Args s)
{
    using Cf = BwdCfg<S>;
    constexpr int XST = Cf::XST, WPT = Cf::WPT, I = Cf::I, HW = S * S;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full[4][XST];
    __shared__ Gate<float> sgs[4][7];
    __shared__ SlotInfo sis[4];
    __shared__ int saborts[4];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long task = (long long)blockIdx.x * 4 + warp;
    if (task >= (long long)s.C * s.parts) return;
    const int c = (int)(task % s.C), part = (int)(task / s.C);
    Gate<float> *sg = sgs[warp];
    SlotInfo &si = sis[warp];
    if (lane < 7) sg[lane] = gate_load<float>(w + ((size_t)c * 7 + lane) * 16, s.wmode);
    if (lane == 8) fill_slots(si, sel, c, s.Ci);
    if (lane == 9) {
        for (int st = 0; st < XST; ++st) clb_tma::mbar_init(&full[warp][st], 1);
        clb_tma::mbar_init_fence();
        saborts[warp] = *reinterpret_cast<volatile int *>(&g_plane_error);
    }
    __syncwarp();
    if (saborts[warp]) return;
    Gate<float> g[7];
#pragma unroll
    for (int i = 0; i < 7; ++i) g[i] = sg[i];
    float acc[28];
#pragma unroll
    for (int i = 0; i < 28; ++i) acc[i] = 0.f;

    const int n_lo = (int)((long long)s.N * part / s.parts), n_hi = (int)((long long)s.N * (part + 1) / s.parts);
    unsigned char *wbase = smem_raw + (size_t)warp * Cf::WARP_BYTES;
    float *gt = reinterpret_cast<float *>(wbase + Cf::GT_BYTES);
    for (int i = lane * 4; i < Cf::STAGE_FLOATS; i += 128) *reinterpret_cast<float4 *>(gt + i) = make_float4(0.f, 0.f, 0.f, 0.f);

    // the lane's windows: slot j = lane + 32*j of the warp's (image, window) space
    int img_local[WPT], win[WPT];
    uint32_t woff[WPT]; // shared address of the window's first position in stage 0, slot 0, tap (0, 0)
#pragma unroll
    for (int j = 0; j < WPT; ++j) {
        const int f = lane + 32 * j;
        img_local[j] = f / I;
        win[j] = f - img_local[j] * I;
        const int py = win[j] / Cf::WP, px = win[j] - py * Cf::WP;
        woff[j] = clb_tma::smem_addr(wbase) + 4u * (uint32_t)(img_local[j] * Cf::IMG + 2 * py * Cf::P + 2 * px);
    }
    uint32_t toff[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int word = sel[c * 8 + k];
        toff[k] = 4u * (uint32_t)(si.slot[k] * Cf::SLOT + ((word >> 8) & 0xFF) * Cf::P + (word & 0xFF) + kLead - 1);
    }
    const int ch_a = si.ch[0], ch_b = si.ch[1];
    const bool usable = si.nslot <= 2; // the host only routes selections here that fit two planes

    const int iters = usable ? (n_hi - n_lo + Cf::NIMG - 1) / Cf::NIMG : 0;
    constexpr uint32_t tx_bytes = 2u * (uint32_t)(Cf::NIMG * Cf::IMG * 4);
    auto issue = [&](int it) {
        const int st = it % XST;
        const int n0 = n_lo + it * Cf::NIMG;
        unsigned char *dst = wbase + (size_t)st * Cf::STAGE_BYTES;
        clb_tma::mbar_expect_tx(&full[warp][st], tx_bytes);
        clb_tma::load_box_4d(dst, &xmap, -kLead, -1, ch_a, n0, &full[warp][st]);
        clb_tma::load_box_4d(dst + Cf::SLOT * 4, &xmap, -kLead, -1, ch_b, n0, &full[warp][st]);
    };
    // cp.async staging (small images): the 16-byte pieces this lane moves, the same for every iteration; the source
    // pointers run along with the iterations, cp_iters = iterations in which the piece's image exists
    constexpr int CPQ = Cf::UNITS / 32;
    const float *csrc[CPQ];
    int cp_iters[CPQ];
    uint32_t cdst[CPQ];
#pragma unroll
    for (int q = 0; q < CPQ; ++q) {
        const int u = lane + 32 * q;
        constexpr int W4 = S / 4;
        const int col4 = u % W4, row = (u / W4) % S, slot = (u / (W4 * S)) & 1, img = u / (W4 * S * 2);
        csrc[q] = x + ((size_t)(n_lo + img) * s.Ci + (slot ? ch_b : ch_a)) * HW + row * S + col4 * 4;
        cp_iters[q] = usable ? (n_hi - n_lo - img + Cf::NIMG - 1) / Cf::NIMG : 0;
        cdst[q] = clb_tma::smem_addr(wbase) + 4u * (uint32_t)(slot * Cf::SLOT + img * Cf::IMG + (row + 1) * Cf::P + kLead + col4 * 4);
    }
    const size_t cstep = (size_t)Cf::NIMG * s.Ci * HW;
    // once per iteration in rising order; always commits, so that the group counts stay aligned; an image past the end of
    // the part is not fetched (its upstream gradient reads as zero)
#define CLB_BWD_ISSUE_CP(ST, IT)                                                                                          \
    {                                                                                                                     \
        _Pragma("unroll") for (int q = 0; q < CPQ; ++q)                                                                   \
        {                                                                                                                 \
            if ((IT) < cp_iters[q]) cp_async16_off<(ST) * Cf::STAGE_BYTES>(cdst[q], csrc[q]);                             \
            csrc[q] += cstep;                                                                                             \
        }                                                                                                                 \
        cp_async_commit();                                                                                                \
    }
    if (Cf::TMA) {
        if (lane == 0)
            for (int it = 0; it < XST && it < iters; ++it) issue(it);
    } else {
        for (int i = lane * 4; i < XST * Cf::STAGE_FLOATS; i += 128)   // the halo is zeroed once; copies write the interior
            *reinterpret_cast<float4 *>(reinterpret_cast<float *>(wbase) + i) = make_float4(0.f, 0.f, 0.f, 0.f);
        __syncwarp();
        CLB_BWD_ISSUE_CP(0, 0)
        CLB_BWD_ISSUE_CP(1, 1)
        CLB_BWD_ISSUE_CP(2, 2)
        static_assert(XST == 3, "prologue of the cp.async ring");
    }

    // upstream gradient and arg-max: fetched one iteration ahead
    float dz_next[WPT];
    int bd_next[WPT];
    auto fetch = [&](int it) {
#pragma unroll
        for (int j = 0; j < WPT; ++j) {
            const int n = n_lo + it * Cf::NIMG + img_local[j];
            const bool live = it < iters && n < n_hi;
            const size_t o = ((size_t)n * s.C + c) * I + win[j];
            if constexpr (FM) // gy is [C][windows][N] (compile-time: the flag in the index arithmetic cost the 8x8 kernel 7 %)
                dz_next[j] = live ? __ldg(gy + ((size_t)c * I + win[j]) * s.N + n) : 0.f;
            else
                dz_next[j] = live ? __ldg(gy + o) : 0.f;
            bd_next[j] = live ? (int)__ldg(amax + o) : 0;
        }
    };
    fetch(0);

    bool failed = false;
    int it = 0;
    __syncwarp();
    // write-out: the lane's float4 units of the gradient tile are the cells its cp.async pieces have in a stage
    float *pdst[CPQ];
#pragma unroll
    for (int q = 0; q < CPQ; ++q) {
        const int u = lane + 32 * q;
        constexpr int W4 = S / 4;
        const int col4 = u % W4, row = (u / W4) % S, slot = (u / (W4 * S)) & 1, img = u / (W4 * S * 2);
        pdst[q] = planes + (((size_t)(n_lo + img) * s.C + c) * 2 + slot) * HW + row * S + col4 * 4;
    }
    const size_t pstep = (size_t)Cf::NIMG * s.C * 2 * HW;
    auto finish = [&]() {
        // write the interior of the gradient planes out and clear it for the next iteration
#pragma unroll
        for (int q = 0; q < CPQ; ++q) {
            const float4 v = lds_v4<Cf::GT_BYTES>(cdst[q]);
            sts_v4_zero<Cf::GT_BYTES>(cdst[q]);
            if (it < cp_iters[q]) *reinterpret_cast<float4 *>(pdst[q]) = v;
            pdst[q] += pstep;
        }
        __syncwarp();
    };
    while (it < iters && !failed) {
        const uint32_t parity = (it / XST) & 1;
#define CLB_BWD_STAGE(ST)                                                                                                 \
    if (it < iters && !failed) {                                                                                          \
        float dz[WPT];                                                                                                    \
        int bd[WPT];                                                                                                      \
        _Pragma("unroll") for (int j = 0; j < WPT; ++j) dz[j] = dz_next[j], bd[j] = bd_next[j];                            \
        fetch(it + 1);                                                                                                    \
        bool ok = true;                                                                                                   \
        if (Cf::TMA) {                                                                                                    \
            ok = clb_tma::mbar_wait(&full[warp][ST], parity);                                                             \
        } else {                                                                                                          \
            cp_async_wait<XST - 1>();                                                                                     \
        }                                                                                                                 \
        ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0; /* also: the other lanes' pieces of this stage are visible */     \
        if (!ok) {                                                                                                        \
            failed = true;                                                                                                \
        } else {                                                                                                          \
            uint32_t base[WPT];                                                                                           \
            _Pragma("unroll") for (int j = 0; j < WPT; ++j) base[j] = woff[j] + 4u * (uint32_t)(((bd[j] >> 1) ? Cf::P : 0) + (bd[j] & 1)); \
            bwd_windows<S, ST, WPT>(base, toff, g, dz, acc);                                                              \
            /* the input planes of this stage have been read by every lane (the taps' __syncwarp): refill it */           \
            if (Cf::TMA) {                                                                                                \
                if (lane == 0 && it + XST < iters) issue(it + XST);                                                       \
            } else {                                                                                                      \
                CLB_BWD_ISSUE_CP(ST, it + XST)                                                                            \
            }                                                                                                             \
            finish();                                                                                                     \
            ++it;                                                                                                         \
        }                                                                                                                 \
    }
        CLB_BWD_STAGE(0)
        CLB_BWD_STAGE(1)
        CLB_BWD_STAGE(2)
#undef CLB_BWD_STAGE
#undef CLB_BWD_ISSUE_CP
    }
    if (failed && lane == 0) {
        g_plane_error = 1;
        for (int j = it + 1; j < iters && j < it + XST; ++j) clb_tma::mbar_wait(&full[warp][j % XST], (j / XST) & 1);
    }
    if (!usable && lane == 0) g_plane_error = 2;

    // the warp's 28 basis sums: lane i ends up with sum i (a transposed butterfly over the 32 lanes)
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = i < 28 ? acc[i] : 0.f;
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
    if (lane < 28) partial[((size_t)part * s.C + c) * 28 + lane] = v[0];
}

// ======================================================================= gate gradient alone, 32x32 images
// The first block of a stack needs no input gradient.  A block of 128 threads owns one (output channel, batch part)
// task and walks its images one at a time through a ring of TMA-staged planes (32x32 planes are 4 KB: rows of 160
// bytes suit the copy engine); a thread owns two pooled windows of the image, recomputes the gate chain at the saved
// arg-max and keeps the 28 basis sums in registers for ALL its images: one block reduction at the very end instead of
// one per (image group, channel).
struct BwdW32 {
    static constexpr int S = 32, P = 40, R = 34, WP = 16, I = 256, WPT = 2;
    static constexpr int IMG = R * P, SLOT = (IMG + 31) / 32 * 32, STAGE_BYTES = 2 * SLOT * 4, STAGES = 3;
    static constexpr int SMEM = STAGES * STAGE_BYTES;
};

template <int ST> __device__ __forceinline__ void bww_window(uint32_t base, const uint32_t (&toff)[8], const Gate<float> (&g)[7], float d, float (&acc)[28])
{
    constexpr int B = ST * BwdW32::STAGE_BYTES;
    float a[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) a[k] = lds_f32<B>(base + toff[k]);
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
    }
}

__global__ void __launch_bounds__(kThreads) convtree_bwd_w_plane32_kernel(const __grid_constant__ CUtensorMap xmap, const float *__restrict__ gy,
                                                                          const float *__restrict__ w, const int32_t *__restrict__ sel,
                                                                          const uint8_t *__restrict__ amax, float *__restrict__ partial, Args s)
{
    using Cf = BwdW32;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full[Cf::STAGES];
    __shared__ Gate<float> sg[7];
    __shared__ SlotInfo si;
    __shared__ float red[4][28];
    __shared__ int sabort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int c = blockIdx.x % s.C, part = blockIdx.x / s.C;
    if (tid < 7) sg[tid] = gate_load<float>(w + ((size_t)c * 7 + tid) * 16, s.wmode);
    if (tid == 32) fill_slots(si, sel, c, s.Ci);
    if (tid == 64) {
        for (int st = 0; st < Cf::STAGES; ++st) clb_tma::mbar_init(&full[st], 1);
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
    const int n_lo = (int)((long long)s.N * part / s.parts), n_hi = (int)((long long)s.N * (part + 1) / s.parts);
    const bool usable = si.nslot <= 2; // the host only routes selections here that fit two planes

    int win[Cf::WPT];
    uint32_t woff[Cf::WPT];
#pragma unroll
    for (int j = 0; j < Cf::WPT; ++j) {
        win[j] = tid + kThreads * j;
        const int py = win[j] / Cf::WP, px = win[j] - py * Cf::WP;
        woff[j] = clb_tma::smem_addr(smem_raw) + 4u * (uint32_t)(2 * py * Cf::P + 2 * px);
    }
    uint32_t toff[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int word = sel[c * 8 + k];
        toff[k] = 4u * (uint32_t)(si.slot[k] * Cf::SLOT + ((word >> 8) & 0xFF) * Cf::P + (word & 0xFF) + kLead - 1);
    }
    const int ch_a = si.ch[0], ch_b = si.ch[1];
    const int iters = usable ? n_hi - n_lo : 0;
    constexpr uint32_t tx_bytes = 2u * (uint32_t)(Cf::IMG * 4);
    auto issue = [&](int it) {
        const int st = it % Cf::STAGES;
        unsigned char *dst = smem_raw + (size_t)st * Cf::STAGE_BYTES;
        clb_tma::mbar_expect_tx(&full[st], tx_bytes);
        clb_tma::load_box_4d(dst, &xmap, -kLead, -1, ch_a, n_lo + it, &full[st]);
        clb_tma::load_box_4d(dst + Cf::SLOT * 4, &xmap, -kLead, -1, ch_b, n_lo + it, &full[st]);
    };
    if (tid == 0)
        for (int it = 0; it < Cf::STAGES && it < iters; ++it) issue(it);

    float dz_next[Cf::WPT];
    int bd_next[Cf::WPT];
    auto fetch = [&](int it) {
#pragma unroll
        for (int j = 0; j < Cf::WPT; ++j) {
            const bool live = it < iters;
            const size_t o = ((size_t)(n_lo + it) * s.C + c) * Cf::I + win[j];
            dz_next[j] = live ? __ldg(gy + o) : 0.f;
            bd_next[j] = live ? (int)__ldg(amax + o) : 0;
        }
    };
    fetch(0);
    bool failed = false;
    int it = 0;
    while (it < iters && !failed) {
        const uint32_t parity = (it / Cf::STAGES) & 1;
#define CLB_BWW_STAGE(ST)                                                                                                 \
    if (it < iters && !failed) {                                                                                          \
        float dz[Cf::WPT];                                                                                                \
        int bd[Cf::WPT];                                                                                                  \
        _Pragma("unroll") for (int j = 0; j < Cf::WPT; ++j) dz[j] = dz_next[j], bd[j] = bd_next[j];                        \
        fetch(it + 1);                                                                                                    \
        bool ok = clb_tma::mbar_wait(&full[ST], parity);                                                                  \
        if (ok) {                                                                                                         \
            _Pragma("unroll") for (int j = 0; j < Cf::WPT; ++j)                                                            \
                bww_window<ST>(woff[j] + 4u * (uint32_t)(((bd[j] >> 1) ? Cf::P : 0) + (bd[j] & 1)), toff, g, dz[j], acc);  \
        }                                                                                                                 \
        ok = __syncthreads_and(ok ? 1 : 0) != 0; /* the stage has been read by the whole block */                        \
        if (!ok) {                                                                                                        \
            failed = true;                                                                                                \
        } else {                                                                                                          \
            if (tid == 0 && it + Cf::STAGES < iters) issue(it + Cf::STAGES);                                              \
            ++it;                                                                                                         \
        }                                                                                                                 \
    }
        CLB_BWW_STAGE(0)
        CLB_BWW_STAGE(1)
        CLB_BWW_STAGE(2)
#undef CLB_BWW_STAGE
    }
    if (failed && tid == 0) {
        g_plane_error = 1;
        for (int j = it + 1; j < iters && j < it + Cf::STAGES; ++j) clb_tma::mbar_wait(&full[j % Cf::STAGES], (j / Cf::STAGES) & 1);
    }
    if (!usable && tid == 0) g_plane_error = 2;

    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = i < 28 ? acc[i] : 0.f;
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
    if (lane < 28) red[warp][lane] = v[0];
    __syncthreads();
    if (tid < 28) partial[((size_t)part * s.C + c) * 28 + tid] = (red[0][tid] + red[1][tid]) + (red[2][tid] + red[3][tid]);
}

// Pass 2: gx[n][ch] = sum of the gradient planes (c, slot) that belong to input channel ch, in list order.
// `start` [Ci + 1], `entry` [..] = 2*c + slot.  One float4 per thread; grid-stride over N * Ci * HW / 4.
// The first fin.blocks blocks of the same launch finish the gate gradient instead (one thread per gate: the per-part basis
// sums added in part order, then the 16 gradients): one launch less per layer and step.
struct GateFinish {
    const float *partial, *w;
    float *gw;
    int parts, wmode, blocks;
    long long ngates;
};
__device__ __forceinline__ void gate_finish_thread(const GateFinish &fin, long long gi)
{
    if (gi >= fin.ngates) return;
    float sums[4] = {0.f, 0.f, 0.f, 0.f};
    for (int p = 0; p < fin.parts; ++p) {
        const float4 q = *reinterpret_cast<const float4 *>(fin.partial + ((size_t)p * fin.ngates + gi) * 4);
        sums[0] += q.x, sums[1] += q.y, sums[2] += q.z, sums[3] += q.w;
    }
    gate_grad_store<float>(sums, fin.w + gi * 16, fin.wmode, fin.gw + gi * 16);
}

template <typename IDX>
__global__ void __launch_bounds__(256) plane_sum_kernel(const float *__restrict__ planes, const int32_t *__restrict__ start,
                                                        const int32_t *__restrict__ entry, float *__restrict__ gx, int N, int Ci, int C, int HW4,
                                                        GateFinish fin)
{
    if ((int)blockIdx.x < fin.blocks) {
        gate_finish_thread(fin, (long long)blockIdx.x * blockDim.x + threadIdx.x);
        return;
    }
    // IDX: 32-bit when the output has fewer than 2^31 float4 units (the three index divisions per unit are then cheap)
    const IDX block = (IDX)blockIdx.x - (IDX)fin.blocks, nblocks = (IDX)gridDim.x - (IDX)fin.blocks;
    // (Measured slower at batch 256: two units per thread a grid stride apart with eight streaming loads in flight,
    // 0.32 -> 0.40 ms per step; walking the images last to first to catch what pass 1 left in L2, 0.32 -> 0.33 ms.)
    const IDX total = (IDX)N * (IDX)Ci * (IDX)HW4;
    for (IDX i = block * (IDX)blockDim.x + (IDX)threadIdx.x; i < total; i += nblocks * (IDX)blockDim.x) {
        const int e = (int)(i % (IDX)HW4);
        const IDX r = i / (IDX)HW4;
        const int ch = (int)(r % (IDX)Ci);
        const IDX n = r / (IDX)Ci;
        const int lo = start[ch], hi = start[ch + 1];
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 *base = reinterpret_cast<const float4 *>(planes) + (size_t)n * C * 2 * HW4 + e;
        int l = lo;
        for (; l + 3 < hi; l += 4) { // four loads in flight
            const float4 a = __ldg(base + (size_t)entry[l] * HW4), b = __ldg(base + (size_t)entry[l + 1] * HW4);
            const float4 p = __ldg(base + (size_t)entry[l + 2] * HW4), q = __ldg(base + (size_t)entry[l + 3] * HW4);
            acc.x += a.x, acc.y += a.y, acc.z += a.z, acc.w += a.w;
            acc.x += b.x, acc.y += b.y, acc.z += b.z, acc.w += b.w;
            acc.x += p.x, acc.y += p.y, acc.z += p.z, acc.w += p.w;
            acc.x += q.x, acc.y += q.y, acc.z += q.z, acc.w += q.w;
        }
        for (; l < hi; ++l) {
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

} // namespace plane
} // namespace clb

// ================================================================================== host side ====
using namespace clb;
using namespace clb_host;
using namespace clb::plane;

namespace {

// The plane kernels cover: fp32, stride 1, 3x3 window, padding 1, square images of 16, 8 or 4 pixels.
int plane_side(int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw)
{
    if (sh != 1 || sw != 1 || ph != 1 || pw != 1 || kh != 3 || kw != 3 || H != W || N <= 0 || C <= 0 || C > 65535 || Ci > 65535) return 0;
    if (tune_get(CLB_TUNE_PLANE_KERNELS) == 0 || clb_tma::encode_tiled_fn() == nullptr) return 0;
    return (H == 32 || H == 16 || H == 8 || H == 4) ? H : 0; // 32: the gate gradient alone (clb_convtree_bwd_plane without gx)
}

// Parts of the batch per output channel: enough (channel, part) tasks for about three waves of resident groups, but
// at least eight iterations per task so that a task's set-up (soft-max of 7 gates, tap table) stays a small share.
int plane_parts(int N, int C, int images_per_iteration, int resident_groups_per_sm)
{
    long long parts = ((long long)sm_count() * resident_groups_per_sm * 3 + C - 1) / C;
    const long long most = N / (8LL * images_per_iteration);
    if (parts > most) parts = most;
    if (parts < 1) parts = 1;
    return (int)parts;
}

template <int S>
int launch_fwd(const float *x, const float *w, const int32_t *sel, float *y, uint8_t *amax, int N, int Ci, int C, int wmode, cudaStream_t st)
{
    using Cf = FwdCfg<S>;
    CUtensorMap map;
    if (!clb_tma::make_plane_map(&map, x, N, Ci, S, S, Cf::P, Cf::R, Cf::NIMG)) return CLB_ERR_SHAPE;
    auto k = convtree_fwd_plane_kernel<S>;
    if (clb_host::ensure_dynamic_smem(k, Cf::SMEM) != cudaSuccess) return check_launch(0);
    const int parts = plane_parts(N, C, Cf::NIMG, Cf::WIDE ? 6 : 12);
    const Args a{N, Ci, C, wmode & 0xff, parts, (wmode & CLB_Y_FEATURE_MAJOR) ? 1 : 0};
    const long long tasks = (long long)C * parts;
    CLB_TRACED("convtree_fwd_plane_kernel", st,
               k<<<(unsigned)((tasks + Cf::GROUPS - 1) / Cf::GROUPS), kThreads, Cf::SMEM, st>>>(map, x, w, sel, y, amax, a));
    return check_launch();
}

template <int S> int bwd_parts(int N, int C) { return plane_parts(N, C, BwdCfg<S>::NIMG, 12); }

template <int S>
int launch_bwd(const float *gy, const float *x, const float *w, const int32_t *sel, const uint8_t *amax, float *partial, float *planes, int N,
               int Ci, int C, int wmode, cudaStream_t st)
{
    using Cf = BwdCfg<S>;
    CUtensorMap map;
    if (!clb_tma::make_plane_map(&map, x, N, Ci, S, S, Cf::P, Cf::R, Cf::NIMG)) return CLB_ERR_SHAPE;
    const bool fm = (wmode & CLB_Y_FEATURE_MAJOR) != 0;
    auto k = fm ? convtree_bwd_plane_kernel<S, true> : convtree_bwd_plane_kernel<S, false>;
    if (clb_host::ensure_dynamic_smem(k, Cf::SMEM) != cudaSuccess) return check_launch(0);
    const int parts = bwd_parts<S>(N, C);
    const Args a{N, Ci, C, wmode & 0xff, parts, fm ? 1 : 0};
    const long long tasks = (long long)C * parts;
    CLB_TRACED("convtree_bwd_plane_kernel", st, k<<<(unsigned)((tasks + 3) / 4), kThreads, Cf::SMEM, st>>>(map, gy, x, w, sel, amax, partial, planes, a));
    return CLB_OK;
}

int bwd_parts_for(int side, int N, int C)
{
    if (side == 32) return plane_parts(N, C, 1, 5);
    return side == 16 ? bwd_parts<16>(N, C) : side == 8 ? bwd_parts<8>(N, C) : bwd_parts<4>(N, C);
}

} // namespace

// Forward of a many-channel layer through the plane kernels; CLB_ERR_SHAPE when they do not cover the shape.
int clb_convtree_fwd_plane_f32(const float *x, const float *w, const int32_t *sel, float *y, uint8_t *amax, int N, int Ci, int H, int W, int C,
                               int sh, int sw, int ph, int pw, int kh, int kw, int wmode, cudaStream_t st)
{
    const int side = plane_side(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw);
    if (side == 16) return launch_fwd<16>(x, w, sel, y, amax, N, Ci, C, wmode, st);
    if (side == 8) return launch_fwd<8>(x, w, sel, y, amax, N, Ci, C, wmode, st);
    if (side == 4) return launch_fwd<4>(x, w, sel, y, amax, N, Ci, C, wmode, st);
    return CLB_ERR_SHAPE;
}

// For every input channel the (output channel, slot) planes that hold its gradient: start [Ci + 1], entry = 2*c + slot,
// output channels ascending.  Slot numbering as in fill_slots: the first distinct channel of an output channel's taps is
// slot 0, the second slot 1.  Returns the number of entries, or CLB_ERR_SHAPE when some output channel names more than
// two channels or a tap outside the kh x kw window (such selections take the general kernels), CLB_ERR_ARG on bad input.
extern "C" int clb_conv_channel_lists(const int32_t *sel_host, int C, int Ci, int kh, int kw, int32_t *start, int32_t *entry, int entry_cap)
{
    if (!sel_host || !start || (!entry && entry_cap > 0) || C < 0 || Ci <= 0) return CLB_ERR_ARG;
    for (int ch = 0; ch <= Ci; ++ch) start[ch] = 0;
    // pass 0: count; pass 1: fill (output channels ascending within a channel's list)
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
    if (dtype != CLB_F32 || !conv_args_ok(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw)) return 0;
    const int side = plane_side(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw);
    if (!side) return 0;
    const size_t partial = ((size_t)bwd_parts_for(side, N, C) * C * 28 * sizeof(float) + 255) / 256 * 256;
    if (side == 32) return partial; // gate gradient alone: no gradient planes
    return partial + (size_t)N * C * 2 * H * W * sizeof(float);
}

extern "C" int clb_convtree_bwd_plane(const void *gy, const void *x, const void *w, const int32_t *sel, const uint8_t *amax, void *gx, void *gw,
                                      const int32_t *ch_start, const int32_t *ch_entry, void *scratch, size_t scratch_bytes, int N, int Ci, int H,
                                      int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int wmode, int dtype, void *stream)
{
    const int wmode_in = wmode; // may carry CLB_Y_FEATURE_MAJOR: gy is [C][windows][N]
    wmode &= ~CLB_Y_FEATURE_MAJOR;
    if (!gy || !x || !w || !sel || !amax || (!gx && !gw) || !scratch || wmode < 0 || wmode > 2) return CLB_ERR_ARG;
    if (gx && (!ch_start || !ch_entry)) return CLB_ERR_ARG;
    if (dtype != CLB_F32 || !conv_args_ok(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw)) return CLB_ERR_SHAPE;
    const int side = plane_side(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw);
    if (!side || (side == 32) != (gx == nullptr)) return CLB_ERR_SHAPE; // 32x32: gate gradient alone; smaller: both gradients
    if (side == 32 && wmode_in != wmode) return CLB_ERR_SHAPE;          // the 32x32 kernel reads gy as [N][C][windows] only
    if (side == 32) {
        const int parts32 = bwd_parts_for(32, N, C);
        if (scratch_bytes < (size_t)parts32 * C * 28 * sizeof(float) || (reinterpret_cast<uintptr_t>(scratch) & 15)) return CLB_ERR_SCRATCH;
        CUtensorMap map32;
        if (!clb_tma::make_plane_map(&map32, (const float *)x, N, Ci, 32, 32, BwdW32::P, BwdW32::R, 1)) return CLB_ERR_SHAPE;
        auto k32 = convtree_bwd_w_plane32_kernel;
        if (clb_host::ensure_dynamic_smem(k32, BwdW32::SMEM) != cudaSuccess) return check_launch(0);
        cudaStream_t st32 = (cudaStream_t)stream;
        const Args a32{N, Ci, C, wmode, parts32, 0};
        CLB_TRACED("convtree_bwd_w_plane32_kernel", st32,
                   k32<<<(unsigned)((long long)C * parts32), kThreads, BwdW32::SMEM, st32>>>(map32, (const float *)gy, (const float *)w, sel, amax,
                                                                                           (float *)scratch, a32));
        const long long ngates32 = (long long)C * 7;
        CLB_TRACED("plane_gate_finalize_kernel", st32,
                   plane_gate_finalize_kernel<<<(int)((ngates32 + 127) / 128), 128, 0, st32>>>((const float *)scratch, (const float *)w, (float *)gw,
                                                                                              parts32, ngates32, wmode));
        return check_launch(2);
    }
    const size_t need = clb_convtree_bwd_plane_scratch_bytes(N, Ci, H, W, C, sh, sw, ph, pw, kh, kw, dtype);
    if (scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 15) || (reinterpret_cast<uintptr_t>(gx) & 15)) return CLB_ERR_SCRATCH;
    cudaStream_t st = (cudaStream_t)stream;
    const int parts = bwd_parts_for(side, N, C);
    float *partial = (float *)scratch;
    float *planes = (float *)((unsigned char *)scratch + ((size_t)parts * C * 28 * sizeof(float) + 255) / 256 * 256);
    const float *gyf = (const float *)gy, *xf = (const float *)x, *wf = (const float *)w;
    const int rc = side == 16  ? launch_bwd<16>(gyf, xf, wf, sel, amax, partial, planes, N, Ci, C, wmode_in, st)
                   : side == 8 ? launch_bwd<8>(gyf, xf, wf, sel, amax, partial, planes, N, Ci, C, wmode_in, st)
                               : launch_bwd<4>(gyf, xf, wf, sel, amax, partial, planes, N, Ci, C, wmode_in, st);
    if (rc != CLB_OK) return rc;
    int launched = 1;
    const int HW4 = H * W / 4;
    const long long total = (long long)N * Ci * HW4;
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)sm_count() * 32;
    if (blocks > cap) blocks = cap;
    GateFinish fin{partial, wf, (float *)gw, parts, wmode, 0, (long long)C * 7};
    if (gw) fin.blocks = (int)((fin.ngates + 255) / 256);
    if (total + (blocks + fin.blocks) * 256 < 0x7fffffffLL)
        CLB_TRACED("plane_sum_kernel", st,
                   plane_sum_kernel<unsigned><<<(unsigned)(blocks + fin.blocks), 256, 0, st>>>(planes, ch_start, ch_entry, (float *)gx, N, Ci, C, HW4, fin));
    else
        CLB_TRACED("plane_sum_kernel", st,
                   plane_sum_kernel<long long><<<(unsigned)(blocks + fin.blocks), 256, 0, st>>>(planes, ch_start, ch_entry, (float *)gx, N, Ci, C, HW4, fin));
    ++launched;
    return check_launch(launched);
}

// Diagnostic: the device-side flag a plane kernel sets when one of its bounded waits ran out (0 = never).  Synchronises.
extern "C" int clb_plane_error(int *flag)
{
    if (!flag) return CLB_ERR_ARG;
    if (cudaMemcpyFromSymbol(flag, g_plane_error, sizeof(int)) != cudaSuccess) return check_launch(0);
    return CLB_OK;
}
