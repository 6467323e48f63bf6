// Packed (discretised) inference kernels: every bit of a word is one sample.
//
// A packed tensor is [rows, words] of `bits`-wide integers, sample bits*word + i in bit i.  On a
// little-endian machine that is the same as a row of ceil(B/bits)*bits/8 BYTES with sample s in bit
// (s & 7) of byte (s >> 3), whatever `bits` is; bitwise gates do not care about the word width either.
// The kernels therefore see rows of bytes and move them in the widest unit the row length and the
// pointers allow (8 bytes when the row length is a multiple of 8 and the bases are 8-byte aligned,
// single bytes otherwise); `bits` only fixes how many pad samples a row ends with.
//
// A 2-input gate with truth table (f00, f01, f10, f11), given as four all-ones/all-zero masks, is the
// two-level multiplexer  y = a ? (b ? m11 : m10) : (b ? m01 : m00): three 3-input logic operations per
// 32 bits, branch-free, with the masks uniform over the thread block.
#include "clb_common.cuh"

namespace clb {

template <typename U> struct OpMasks {
    U m00, m01, m10, m11;
};
template <typename U> __device__ __forceinline__ OpMasks<U> op_masks(int op)
{
    OpMasks<U> m;
    const U ones = ~U(0);
    m.m00 = (op & 8) ? ones : U(0);
    m.m01 = (op & 4) ? ones : U(0);
    m.m10 = (op & 2) ? ones : U(0);
    m.m11 = (op & 1) ? ones : U(0);
    return m;
}
template <typename U> __device__ __forceinline__ U op_apply(const OpMasks<U> &m, U a, U b)
{
    const U r1 = (b & m.m11) | (~b & m.m10);
    const U r0 = (b & m.m01) | (~b & m.m00);
    return (a & r1) | (~a & r0);
}

// ------------------------------------------------------------------------------------- pack bits
// feature-major source t [F,B]; one thread builds one output byte from 8 consecutive samples.
__global__ void pack_bits_kernel(const uint8_t *__restrict__ t, uint8_t *__restrict__ out, long long F, long long B, long long rowbytes)
{
    const long long total = F * rowbytes;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long f = i / rowbytes, q = i % rowbytes;
        const uint8_t *src = t + f * B + q * 8;
        unsigned v = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (q * 8 + k < B) v |= (src[k] != 0 ? 1u : 0u) << k;
        out[i] = (uint8_t)v;
    }
}

// sample-major source t [N,F]: thread <-> feature, loops over 8*BY samples and writes BY bytes of its row.
template <int BY>
__global__ void __launch_bounds__(256) pack_bits_nmajor_kernel(const uint8_t *__restrict__ t, uint8_t *__restrict__ out, long long N,
                                                               long long F, long long rowbytes)
{
    const long long f = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (f >= F) return;
    for (long long q0 = (long long)blockIdx.y * BY; q0 < rowbytes; q0 += (long long)gridDim.y * BY) {
        uint8_t bytes[BY];
#pragma unroll
        for (int q = 0; q < BY; ++q) {
            unsigned v = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const long long n = (q0 + q) * 8 + k;
                if (n < N) v |= (__ldg(t + n * F + f) != 0 ? 1u : 0u) << k;
            }
            bytes[q] = (uint8_t)v;
        }
        uint8_t *dst = out + f * rowbytes + q0;
        if (BY == 32 && q0 + BY <= rowbytes && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
            const uint4 *b4 = reinterpret_cast<const uint4 *>(bytes);
            reinterpret_cast<uint4 *>(dst)[0] = b4[0];
            reinterpret_cast<uint4 *>(dst)[1] = b4[1];
        } else {
#pragma unroll
            for (int q = 0; q < BY; ++q)
                if (q0 + q < rowbytes) dst[q] = bytes[q];
        }
    }
}

// ---------------------------------------------------------------------------- thermometer + pack
// Fused input stage of packed inference: pixels [N][P] (P = channels * H * W, fp32 in [0,1] or uint8 that is
// divided by 255 as torchvision's ToTensor does) -> the L*P thermometer features "pixel > threshold[i]",
// threshold-major (feature i*P + p), bit-packed along the batch, without the [N, L*P] byte tensor in between.
// Block: 32 pixel positions (lanes: coalesced 128-byte reads of one sample) x 256 samples (8 warps x 32);
// a thread builds, for its position, the 32-sample word of every level in registers; the words go through
// shared memory so that each feature row receives 32 contiguous bytes (rows layout) or each (feature, slab)
// 512 contiguous bytes (slab layout, one 16-byte unit per position).
constexpr int kThermoLevels = 32; // levels handled per pass over the pixels

template <typename PIX>
__device__ __forceinline__ float pixel_value(const PIX *p);
template <>
__device__ __forceinline__ float pixel_value<float>(const float *p)
{
    return __ldg(p);
}
template <>
__device__ __forceinline__ float pixel_value<uint8_t>(const uint8_t *p)
{
    return __fdiv_rn((float)__ldg(p), 255.0f);
}

template <typename PIX>
__global__ void __launch_bounds__(256) thermometer_pack_kernel(const PIX *__restrict__ pix, const float *__restrict__ thr, int L,
                                                               unsigned *__restrict__ out, long long N, int P, int HW,
                                                               long long words32, int to_slab)
{
    __shared__ unsigned sm[kThermoLevels * 32 * 9];
    __shared__ unsigned lut[256]; // uint8 pixels: level mask of every pixel value
    const int lane = threadIdx.x & 31, wv = threadIdx.x >> 5;
    const int p = blockIdx.x * 32 + lane;
    const long long n0 = (long long)blockIdx.y * 256;
    for (int l0 = 0; l0 < L; l0 += kThermoLevels) {
        const int nl = min(kThermoLevels, L - l0);
        float th[kThermoLevels];
#pragma unroll
        for (int i = 0; i < kThermoLevels; ++i) th[i] = i < nl ? __ldg(thr + l0 + i) : 0.f;
        unsigned word[kThermoLevels];
        if constexpr (sizeof(PIX) == 1) {
            // uint8 pixels take 256 values: thread t builds the level mask of value t once per block (the same float
            // expression as below, so the bits are the same), a sample is then one byte load and one table look-up,
            // and a 32x32 bit transpose in registers turns the 32 samples' level masks into the 32 levels' sample words.
            __syncthreads(); // the previous pass no longer reads the table
            {
                const float v = __fdiv_rn((float)threadIdx.x, 255.0f);
                unsigned m = 0u;
#pragma unroll
                for (int i = 0; i < kThermoLevels; ++i) m |= ((i < nl && v > th[i]) ? 1u : 0u) << i;
                lut[threadIdx.x] = m;
            }
            __syncthreads();
            {
                const long long nb = n0 + wv * 32;                  // first of the warp's 32 samples
                const int live = p < P ? (int)min((long long)32, N - nb) : 0; // how many of them exist (<= 0: none)
                const uint8_t *src = reinterpret_cast<const uint8_t *>(pix) + nb * P + p;
#pragma unroll
                for (int j = 0; j < 32; ++j) word[j] = j < live ? lut[__ldg(src + (long long)j * P)] : 0u;
            }
            unsigned m = 0x0000FFFFu;
#pragma unroll
            for (int j = 16; j != 0; j >>= 1) {
#pragma unroll
                for (int k = 0; k < 32; k = (k + j + 1) & ~j) {
                    const unsigned t = ((word[k] >> j) ^ word[k + j]) & m;
                    word[k + j] ^= t;
                    word[k] ^= t << j;
                }
                m ^= m << (j >> 1);
            }
        } else {
#pragma unroll
            for (int i = 0; i < kThermoLevels; ++i) word[i] = 0u;
#pragma unroll 4
            for (int j = 0; j < 32; ++j) {
                const long long n = n0 + wv * 32 + j;
                if (n < N && p < P) {
                    const float v = pixel_value<PIX>(pix + n * P + p);
#pragma unroll
                    for (int i = 0; i < kThermoLevels; ++i) word[i] |= (v > th[i] ? 1u : 0u) << j;
                }
            }
        }
        __syncthreads(); // the previous pass has been written out
#pragma unroll
        for (int i = 0; i < kThermoLevels; ++i) sm[(i * 32 + lane) * 9 + wv] = word[i];
        __syncthreads();
        const long long w0 = n0 / 32; // first 32-bit word of this block in a row
        // Write-out: element e = thread + 256 * level, so a thread's (position, word) never changes and only the level
        // walks: one shared load, one store and two additions per level.
        if (!to_slab) {
            // (level, position, word): 8 consecutive lanes write the 32 bytes of one row
            const int w = threadIdx.x & 7, pos = (threadIdx.x >> 3) & 31;
            const int pp = blockIdx.x * 32 + pos;
            if (pp < P && w0 + w < words32) {
                unsigned *dst = out + ((long long)l0 * P + pp) * words32 + w0 + w;
                const unsigned *srcw = sm + pos * 9 + w;
                const long long dstep = (long long)P * words32;
                for (int i = 0; i < nl; ++i) dst[i * dstep] = srcw[i * 32 * 9];
            }
        } else {
            // slab layout [feature channel][U][HW] of 16-byte units: 4 consecutive lanes write one unit
            const long long U = words32 / 4;
            const int q = threadIdx.x & 3, pos = (threadIdx.x >> 2) & 31, u2 = (threadIdx.x >> 7) & 1;
            const int pp = blockIdx.x * 32 + pos;
            const long long u = w0 / 4 + u2;
            if (pp < P && u < U) {
                const int c = pp / HW, yx = pp - c * HW;
                unsigned *dst = out + ((((long long)l0 * (P / HW) + c) * U + u) * HW + yx) * 4 + q;
                const unsigned *srcw = sm + pos * 9 + u2 * 4 + q;
                const long long dstep = (long long)(P / HW) * U * HW * 4;
                for (int i = 0; i < nl; ++i) dst[i * dstep] = srcw[i * 32 * 9];
            }
        }
    }
}

// ----------------------------------------------------------------------------------- flat layer
// U = transfer unit; units = units per row.  thread <-> (neuron, unit), unit fastest.
template <typename U>
__global__ void __launch_bounds__(256) packed_logic_kernel(const U *__restrict__ x, const int64_t *__restrict__ ia,
                                                           const int64_t *__restrict__ ib, const uint8_t *__restrict__ ops,
                                                           U *__restrict__ y, long long out_dim, long long units)
{
    // (neuron, unit) of the thread's items by carried additions: one 64-bit division per thread, none per item
    const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
    const long long dj = stride / units, du = stride - dj * units;
    long long j = i0 / units, u = i0 - j * units;
    for (long long i = i0; j < out_dim; i += stride, j += dj, u += du) {
        if (u >= units) u -= units, ++j;
        if (j >= out_dim) break;
        const OpMasks<U> m = op_masks<U>(ops[j]);
        y[i] = op_apply<U>(m, x[ia[j] * units + u], x[ib[j] * units + u]);
    }
}

// 16-byte variant: one thread moves a uint4 (two 64-bit units) per operand.
__global__ void __launch_bounds__(256) packed_logic_v4_kernel(const uint4 *__restrict__ x, const int64_t *__restrict__ ia,
                                                              const int64_t *__restrict__ ib, const uint8_t *__restrict__ ops,
                                                              uint4 *__restrict__ y, long long out_dim, long long units)
{
    // (neuron, unit) of the thread's items by carried additions: one 64-bit division per thread, none per item
    const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
    const long long dj = stride / units, du = stride - dj * units;
    long long j = i0 / units, u = i0 - j * units;
    for (long long i = i0; j < out_dim; i += stride, j += dj, u += du) {
        if (u >= units) u -= units, ++j;
        if (j >= out_dim) break;
        const OpMasks<unsigned> m = op_masks<unsigned>(ops[j]);
        const uint4 a = __ldg(x + ia[j] * units + u), b = __ldg(x + ib[j] * units + u);
        uint4 r;
        r.x = op_apply<unsigned>(m, a.x, b.x);
        r.y = op_apply<unsigned>(m, a.y, b.y);
        r.z = op_apply<unsigned>(m, a.z, b.z);
        r.w = op_apply<unsigned>(m, a.w, b.w);
        y[i] = r;
    }
}

// Two or three consecutive flat layers as one pass.  When a layer's outputs are each read about once by the next
// layer (the stacks halve their width from layer to layer, and `randperm(2*out) % in` then uses every output
// exactly once), a neuron of the last layer is a gate tree over 2^M rows of the FIRST layer's input: the
// intermediate activations (the largest tensors of the stack) are never written or read.  leaf [out][2^M] are the
// input rows in tree order (gate p of the first level reads leaves 2p and 2p+1), ops [out][2^M - 1] the gate ids
// level by level (first level, ..., root).  Rows move in 8- or 16-byte units like the single layer.
template <typename V4, int M, typename IDX>
__global__ void __launch_bounds__(256) packed_tree_kernel(const V4 *__restrict__ x, const int32_t *__restrict__ leaf,
                                                          const uint8_t *__restrict__ ops, V4 *__restrict__ y, long long out_dim,
                                                          long long units, long long u_lo, long long u_n)
{
    // one launch covers units [u_lo, u_lo + u_n) of every row
    constexpr int L = 1 << M, G = L - 1;
    constexpr int W = sizeof(V4) / 4;
    // (tree, unit) of the thread's items by carried additions: one 64-bit division per thread instead of two per item
    const long long t0 = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
    const long long dj = stride / u_n, du = stride - dj * u_n;
    long long j = t0 / u_n, ur = t0 - j * u_n;
    for (; j < out_dim; j += dj, ur += du) {
        if (ur >= u_n) ur -= u_n, ++j;
        if (j >= out_dim) break;
        const long long u = u_lo + ur, i = j * units + u;
        unsigned v[L][W];
#pragma unroll
        for (int k = 0; k < L; ++k) {
            const V4 q = __ldg(x + ((IDX)__ldg(leaf + j * L + k) * (IDX)units + (IDX)u)); // IDX: 32 bits when the input has < 2^32 units
            const unsigned *qw = reinterpret_cast<const unsigned *>(&q);
#pragma unroll
            for (int w = 0; w < W; ++w) v[k][w] = qw[w];
        }
        int g = 0;
#pragma unroll
        for (int n = L / 2; n >= 1; n /= 2) { // n gates on this level
#pragma unroll
            for (int p = 0; p < n; ++p) {
                const OpMasks<unsigned> m = op_masks<unsigned>(__ldg(ops + j * G + g + p));
#pragma unroll
                for (int w = 0; w < W; ++w) v[p][w] = op_apply<unsigned>(m, v[2 * p][w], v[2 * p + 1][w]);
            }
            g += n;
        }
        V4 r;
        unsigned *rw = reinterpret_cast<unsigned *>(&r);
#pragma unroll
        for (int w = 0; w < W; ++w) rw[w] = v[0][w];
        y[i] = r;
    }
}

// ----------------------------------------------------------------------------------- group sum
// x rows as 32-bit units (32 samples each).  thread <-> (class, row split, unit).  Rows are added 16 at
// a time into bit-sliced counters (carry-save adders: ones, twos, fours, eights + ripple counter for
// the sixteens), so a row costs a handful of logic operations per 32 samples; the per-sample integers
// are only extracted once at the end.  With more than one row split the partial counts are combined
// with integer atomics (exact, order-independent) into a zeroed output.
__device__ __forceinline__ void csa(unsigned &hi, unsigned &lo, unsigned a, unsigned b, unsigned c)
{
    const unsigned u = a ^ b;
    hi = (a & b) | (u & c);
    lo = u ^ c;
}

// PLANES bit planes above the sixteens: a thread can count 16 * 2^PLANES rows (8 planes when its share of the rows
// allows it: the ripple through the planes is most of the work per 16 rows)
template <int PLANES>
__global__ void __launch_bounds__(128) group_popcount_kernel(const unsigned *__restrict__ x, int *__restrict__ counts, long long S,
                                                             long long units, long long B, int k, int splits)
{
    const long long total = (long long)k * splits * units;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long u = i % units;
        const int sp = (int)((i / units) % splits);
        const int cls = (int)(i / (units * splits));
        const long long per = ((S + splits - 1) / splits + 15) / 16 * 16;
        const long long r_lo = per * sp, r_hi = min(S, r_lo + per);
        const unsigned *base = x + ((long long)cls * S) * units + u;
        unsigned ones = 0, twos = 0, fours = 0, eights = 0;
        unsigned up[PLANES];
#pragma unroll
        for (int p = 0; p < PLANES; ++p) up[p] = 0;
        const unsigned *pr = base + r_lo * units; // walks down the rows: one addition per load, no multiplication
        for (long long r = r_lo; r < r_hi; r += 16) {
            unsigned v[16];
            if (r + 16 <= r_hi) {
#pragma unroll
                for (int q = 0; q < 16; ++q) v[q] = __ldg(pr), pr += units;
            } else {
#pragma unroll
                for (int q = 0; q < 16; ++q) v[q] = (r + q < r_hi) ? __ldg(pr + q * units) : 0u;
            }
            unsigned t2a, t2b, t4a, t4b, t8a, t8b, t16;
            csa(t2a, ones, ones, v[0], v[1]);
            csa(t2b, ones, ones, v[2], v[3]);
            csa(t4a, twos, twos, t2a, t2b);
            csa(t2a, ones, ones, v[4], v[5]);
            csa(t2b, ones, ones, v[6], v[7]);
            csa(t4b, twos, twos, t2a, t2b);
            csa(t8a, fours, fours, t4a, t4b);
            csa(t2a, ones, ones, v[8], v[9]);
            csa(t2b, ones, ones, v[10], v[11]);
            csa(t4a, twos, twos, t2a, t2b);
            csa(t2a, ones, ones, v[12], v[13]);
            csa(t2b, ones, ones, v[14], v[15]);
            csa(t4b, twos, twos, t2a, t2b);
            csa(t8b, fours, fours, t4a, t4b);
            csa(t16, eights, eights, t8a, t8b);
            // ripple the sixteens into the upper counter
            unsigned carry = t16;
#pragma unroll
            for (int p = 0; p < PLANES; ++p) {
                const unsigned nc = up[p] & carry;
                up[p] ^= carry;
                carry = nc;
            }
        }
#pragma unroll 1
        for (int bit = 0; bit < 32; ++bit) {
            const long long s = u * 32 + bit;
            if (s >= B) break;
            int c = ((ones >> bit) & 1) + 2 * ((twos >> bit) & 1) + 4 * ((fours >> bit) & 1) + 8 * ((eights >> bit) & 1);
#pragma unroll
            for (int p = 0; p < PLANES; ++p) c += (int)((up[p] >> bit) & 1u) << (4 + p);
            if (splits == 1)
                counts[s * k + cls] = c;
            else if (c)
                atomicAdd(counts + s * k + cls, c);
        }
    }
}

// byte-unit fallback for rows whose length is not a multiple of 4 bytes: thread <-> (sample, class)
__global__ void group_popcount_bytes_kernel(const uint8_t *__restrict__ x, int *__restrict__ counts, long long S, long long rowbytes,
                                            long long B, int k)
{
    const long long total = B * k;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long s = i / k;
        const int cls = (int)(i % k);
        const uint8_t *base = x + (long long)cls * S * rowbytes + (s >> 3);
        int c = 0;
        for (long long r = 0; r < S; ++r) c += (base[r * rowbytes] >> (s & 7)) & 1;
        counts[i] = c;
    }
}

// --------------------------------------------------------------------------- packed ConvLogic block
struct PackedShape {
    int Ci, H, W, C, Ho, Wo, sh, sw, ph, pw;
};

// grid (chunks over (py, px, unit), C); thread <-> (py, px, unit) with unit fastest.
template <typename U>
__global__ void __launch_bounds__(256) packed_convtree_kernel(const U *__restrict__ x, const uint8_t *__restrict__ ops,
                                                              const int32_t *__restrict__ sel, U *__restrict__ y, PackedShape s,
                                                              long long units)
{
    __shared__ OpMasks<U> sm[7];
    __shared__ Tap stap[8];
    const int c = blockIdx.y;
    if (threadIdx.x < 7) sm[threadIdx.x] = op_masks<U>(ops[c * 7 + threadIdx.x]);
    if (threadIdx.x >= 32 && threadIdx.x < 40) stap[threadIdx.x - 32] = unpack_tap(sel[c * 8 + threadIdx.x - 32], s.ph, s.pw);
    __syncthreads();
    const int Hp = s.Ho / 2, Wp = s.Wo / 2;
    const long long total = (long long)Hp * Wp * units;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long u = i % units;
        const int win = (int)(i / units);
        const int py = win / Wp, px = win % Wp;
        U acc = U(0);
#pragma unroll
        for (int d = 0; d < 4; ++d) {
            const int oy = 2 * py + (d >> 1), ox = 2 * px + (d & 1);
            U a[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                const int iy = oy * s.sh + stap[t].dy, ix = ox * s.sw + stap[t].dx;
                a[t] = ((unsigned)iy < (unsigned)s.H && (unsigned)ix < (unsigned)s.W)
                           ? __ldg(x + (((long long)stap[t].ch * s.H + iy) * s.W + ix) * units + u)
                           : U(0);
            }
            const U g0 = op_apply<U>(sm[0], a[0], a[1]), g1 = op_apply<U>(sm[1], a[2], a[3]);
            const U g2 = op_apply<U>(sm[2], a[4], a[5]), g3 = op_apply<U>(sm[3], a[6], a[7]);
            const U t0 = op_apply<U>(sm[4], g0, g1), t1 = op_apply<U>(sm[5], g2, g3);
            acc |= op_apply<U>(sm[6], t0, t1);
        }
        y[((long long)c * Hp * Wp + win) * units + u] = acc;
    }
}

// 16-byte variant for rows that are a multiple of 16 bytes (the usual case: 64-bit words, batches that
// are a multiple of 128).  One thread produces one uint4 (128 samples) of one pooled output.  Everything
// block-uniform (the 7 gates as 32-bit multiplexer masks, the 8 tap offsets) sits in registers; a window
// whose 4 x 8 taps all fall inside the image takes a path without bounds tests; indices are 32-bit.
struct Masks32 {
    unsigned m00, m01, m10, m11;
};
__device__ __forceinline__ unsigned mux32(const Masks32 &m, unsigned a, unsigned b)
{
    const unsigned r1 = (b & m.m11) | (~b & m.m10);
    const unsigned r0 = (b & m.m01) | (~b & m.m00);
    return (a & r1) | (~a & r0);
}
__device__ __forceinline__ uint4 mux128(const Masks32 &m, const uint4 &a, const uint4 &b)
{
    return make_uint4(mux32(m, a.x, b.x), mux32(m, a.y, b.y), mux32(m, a.z, b.z), mux32(m, a.w, b.w));
}

__global__ void __launch_bounds__(256) packed_convtree_v4_kernel(const uint4 *__restrict__ x, const uint8_t *__restrict__ ops,
                                                                 const int32_t *__restrict__ sel, uint4 *__restrict__ y, PackedShape s,
                                                                 int units)
{
    const int c = blockIdx.y;
    Masks32 gm[7];
#pragma unroll
    for (int g = 0; g < 7; ++g) {
        const int op = ops[c * 7 + g];
        gm[g].m00 = (op & 8) ? ~0u : 0u, gm[g].m01 = (op & 4) ? ~0u : 0u, gm[g].m10 = (op & 2) ? ~0u : 0u, gm[g].m11 = (op & 1) ? ~0u : 0u;
    }
    int tb[8], tdy[8], tdx[8]; // tap: element offset (in units) relative to the position, row / col displacement
    int ymin = 0, ymax = 0, xmin = 0, xmax = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const Tap t = unpack_tap(sel[c * 8 + k], s.ph, s.pw);
        tdy[k] = t.dy, tdx[k] = t.dx;
        tb[k] = ((t.ch * s.H + t.dy) * s.W + t.dx) * units;
        ymin = min(ymin, t.dy), ymax = max(ymax, t.dy), xmin = min(xmin, t.dx), xmax = max(xmax, t.dx);
    }
    const int Hp = s.Ho / 2, Wp = s.Wo / 2;
    const int total = Hp * Wp * units;
    const int rowstep = s.sh * s.W * units, colstep = s.sw * units;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int win = i / units, u = i - win * units;
        const int py = win / Wp, px = win - py * Wp;
        const int oy0 = 2 * py * s.sh, ox0 = 2 * px * s.sw;
        const int p0 = (oy0 * s.W + ox0) * units + u; // first position of the window
        const bool interior = oy0 + ymin >= 0 && oy0 + s.sh + ymax < s.H && ox0 + xmin >= 0 && ox0 + s.sw + xmax < s.W;
        uint4 acc = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int d = 0; d < 4; ++d) {
            const int pd = p0 + ((d >> 1) ? rowstep : 0) + ((d & 1) ? colstep : 0);
            uint4 a[8];
            if (interior) {
#pragma unroll
                for (int k = 0; k < 8; ++k) a[k] = __ldg(x + (pd + tb[k]));
            } else {
                const int oy = oy0 + (d >> 1) * s.sh, ox = ox0 + (d & 1) * s.sw;
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    a[k] = ((unsigned)(oy + tdy[k]) < (unsigned)s.H && (unsigned)(ox + tdx[k]) < (unsigned)s.W) ? __ldg(x + (pd + tb[k]))
                                                                                                              : make_uint4(0u, 0u, 0u, 0u);
            }
            const uint4 g0 = mux128(gm[0], a[0], a[1]), g1 = mux128(gm[1], a[2], a[3]);
            const uint4 g2 = mux128(gm[2], a[4], a[5]), g3 = mux128(gm[3], a[6], a[7]);
            const uint4 t0 = mux128(gm[4], g0, g1), t1 = mux128(gm[5], g2, g3);
            const uint4 z = mux128(gm[6], t0, t1);
            acc.x |= z.x, acc.y |= z.y, acc.z |= z.z, acc.w |= z.w;
        }
        y[(c * Hp * Wp + win) * units + u] = acc;
    }
}

// ---- slab layout --------------------------------------------------------------------------------
// The [C][H][W][words] layout makes a pixel's words contiguous, which suits the flat layers but forces the
// conv block to gather 32 scattered 16-byte pieces per output piece through L1/L2.  In the slab layout
// [C][U][H][W] of uint4 (U = words/2; one uint4 = 128 samples) the image of one (channel, sample slab) is
// contiguous.  A persistent block walks (output channel, group of UB slabs) items; for each it copies the two
// channel planes the output channel reads into a shared tile (halo zeroed once, columns de-interleaved as in
// the float forward so that window columns are consecutive 16-byte slots) with cp.async into the buffer the
// previous item is not using, so the copy of item i+1 runs under the gate tree of item i.  Every tap is then a
// conflict-free 128-bit shared-memory load.  The per-item bookkeeping (tap offsets, gate ids, the two
// channels) is parsed two items ahead by eight threads into a small shared record, and a gate is applied by a
// block-uniform switch over its id to eight words at a time: one LOP3 per word instead of the three a
// multiplexer with run-time masks needs.  UB * windows-per-image <= 256 threads.  An output channel with a tap
// on a third channel or outside the kernel window (hand-made selections only) takes a global-memory path.
struct SlabShape {
    int Ci, H, W, C, Ho, Wo, ph, pw, kh, kw;
    int U, UB;       // slabs in total / per block
    int PH, pwh;     // padded rows, uint4 slots per column-parity plane of a padded row
    int CS, SS;      // plane stride (one channel slot) and slab stride in the tile, in uint4
    int n_ug, items; // slab groups per channel, items = C * n_ug
    int per_thread;  // copies per thread and channel plane group: ceil(UB*H*W / threads)
};

struct __align__(16) SlabRec {
    int tb0[8], tb1[8]; // tile offsets (bytes) of tap k for the left / right conv column of a window
    int op[8];          // gate ids (7 used)
    int ch[2], nst, all_in_tile;
    int word[8];        // the raw selection words (global path)
};

__device__ __forceinline__ void cp_async16(uint4 *dst_shared, const uint4 *src)
{
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst_shared);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// a[w] = gate(a[w], b[w]) for eight words; `op` is uniform over the block.  Every case is ONE lop3 per word written IN PLACE
// (the "+r" constraint): with plain C expressions the sixteen cases end in different registers and the compiler reconciles
// them with moves at the join -- more moves than logic operations.  Truth-table immediates for (A, B) = (0xF0, 0xCC); the
// third operand is unused (every table is symmetric in it).
// The sixteen cases sit behind ONE indexed branch (brx.idx over a table of the sixteen case labels) instead of the
// compare-and-branch tree a C switch compiles to (13 control instructions per gate, more than its 8 lop3).  `op` is uniform
// over the block, so the branch is declared uniform.  Eight words, in place.
__device__ __forceinline__ void gate_words_brx(int op, unsigned (&a)[8], const unsigned (&b)[8])
{
    asm(
        "{\n\t.reg .u32 gi;\n\tand.b32 gi, %16, 15;\n\t"
        "gtab: .branchtargets G0, G1, G2, G3, G4, G5, G6, G7, G8, G9, G10, G11, G12, G13, G14, G15;\n\t"
        "brx.idx.uni gi, gtab;\n"
        "G0: lop3.b32 %0, %0, %8, %8, 0x00; lop3.b32 %1, %1, %9, %9, 0x00; lop3.b32 %2, %2, %10, %10, 0x00; lop3.b32 %3, %3, %11, %11, 0x00; lop3.b32 %4, %4, %12, %12, 0x00; lop3.b32 %5, %5, %13, %13, 0x00; lop3.b32 %6, %6, %14, %14, 0x00; lop3.b32 %7, %7, %15, %15, 0x00; bra.uni GDONE;\n"
        "G1: lop3.b32 %0, %0, %8, %8, 0xC0; lop3.b32 %1, %1, %9, %9, 0xC0; lop3.b32 %2, %2, %10, %10, 0xC0; lop3.b32 %3, %3, %11, %11, 0xC0; lop3.b32 %4, %4, %12, %12, 0xC0; lop3.b32 %5, %5, %13, %13, 0xC0; lop3.b32 %6, %6, %14, %14, 0xC0; lop3.b32 %7, %7, %15, %15, 0xC0; bra.uni GDONE;\n"
        "G2: lop3.b32 %0, %0, %8, %8, 0x30; lop3.b32 %1, %1, %9, %9, 0x30; lop3.b32 %2, %2, %10, %10, 0x30; lop3.b32 %3, %3, %11, %11, 0x30; lop3.b32 %4, %4, %12, %12, 0x30; lop3.b32 %5, %5, %13, %13, 0x30; lop3.b32 %6, %6, %14, %14, 0x30; lop3.b32 %7, %7, %15, %15, 0x30; bra.uni GDONE;\n"
        "G3: lop3.b32 %0, %0, %8, %8, 0xF0; lop3.b32 %1, %1, %9, %9, 0xF0; lop3.b32 %2, %2, %10, %10, 0xF0; lop3.b32 %3, %3, %11, %11, 0xF0; lop3.b32 %4, %4, %12, %12, 0xF0; lop3.b32 %5, %5, %13, %13, 0xF0; lop3.b32 %6, %6, %14, %14, 0xF0; lop3.b32 %7, %7, %15, %15, 0xF0; bra.uni GDONE;\n"
        "G4: lop3.b32 %0, %0, %8, %8, 0x0C; lop3.b32 %1, %1, %9, %9, 0x0C; lop3.b32 %2, %2, %10, %10, 0x0C; lop3.b32 %3, %3, %11, %11, 0x0C; lop3.b32 %4, %4, %12, %12, 0x0C; lop3.b32 %5, %5, %13, %13, 0x0C; lop3.b32 %6, %6, %14, %14, 0x0C; lop3.b32 %7, %7, %15, %15, 0x0C; bra.uni GDONE;\n"
        "G5: lop3.b32 %0, %0, %8, %8, 0xCC; lop3.b32 %1, %1, %9, %9, 0xCC; lop3.b32 %2, %2, %10, %10, 0xCC; lop3.b32 %3, %3, %11, %11, 0xCC; lop3.b32 %4, %4, %12, %12, 0xCC; lop3.b32 %5, %5, %13, %13, 0xCC; lop3.b32 %6, %6, %14, %14, 0xCC; lop3.b32 %7, %7, %15, %15, 0xCC; bra.uni GDONE;\n"
        "G6: lop3.b32 %0, %0, %8, %8, 0x3C; lop3.b32 %1, %1, %9, %9, 0x3C; lop3.b32 %2, %2, %10, %10, 0x3C; lop3.b32 %3, %3, %11, %11, 0x3C; lop3.b32 %4, %4, %12, %12, 0x3C; lop3.b32 %5, %5, %13, %13, 0x3C; lop3.b32 %6, %6, %14, %14, 0x3C; lop3.b32 %7, %7, %15, %15, 0x3C; bra.uni GDONE;\n"
        "G7: lop3.b32 %0, %0, %8, %8, 0xFC; lop3.b32 %1, %1, %9, %9, 0xFC; lop3.b32 %2, %2, %10, %10, 0xFC; lop3.b32 %3, %3, %11, %11, 0xFC; lop3.b32 %4, %4, %12, %12, 0xFC; lop3.b32 %5, %5, %13, %13, 0xFC; lop3.b32 %6, %6, %14, %14, 0xFC; lop3.b32 %7, %7, %15, %15, 0xFC; bra.uni GDONE;\n"
        "G8: lop3.b32 %0, %0, %8, %8, 0x03; lop3.b32 %1, %1, %9, %9, 0x03; lop3.b32 %2, %2, %10, %10, 0x03; lop3.b32 %3, %3, %11, %11, 0x03; lop3.b32 %4, %4, %12, %12, 0x03; lop3.b32 %5, %5, %13, %13, 0x03; lop3.b32 %6, %6, %14, %14, 0x03; lop3.b32 %7, %7, %15, %15, 0x03; bra.uni GDONE;\n"
        "G9: lop3.b32 %0, %0, %8, %8, 0xC3; lop3.b32 %1, %1, %9, %9, 0xC3; lop3.b32 %2, %2, %10, %10, 0xC3; lop3.b32 %3, %3, %11, %11, 0xC3; lop3.b32 %4, %4, %12, %12, 0xC3; lop3.b32 %5, %5, %13, %13, 0xC3; lop3.b32 %6, %6, %14, %14, 0xC3; lop3.b32 %7, %7, %15, %15, 0xC3; bra.uni GDONE;\n"
        "G10: lop3.b32 %0, %0, %8, %8, 0x33; lop3.b32 %1, %1, %9, %9, 0x33; lop3.b32 %2, %2, %10, %10, 0x33; lop3.b32 %3, %3, %11, %11, 0x33; lop3.b32 %4, %4, %12, %12, 0x33; lop3.b32 %5, %5, %13, %13, 0x33; lop3.b32 %6, %6, %14, %14, 0x33; lop3.b32 %7, %7, %15, %15, 0x33; bra.uni GDONE;\n"
        "G11: lop3.b32 %0, %0, %8, %8, 0xF3; lop3.b32 %1, %1, %9, %9, 0xF3; lop3.b32 %2, %2, %10, %10, 0xF3; lop3.b32 %3, %3, %11, %11, 0xF3; lop3.b32 %4, %4, %12, %12, 0xF3; lop3.b32 %5, %5, %13, %13, 0xF3; lop3.b32 %6, %6, %14, %14, 0xF3; lop3.b32 %7, %7, %15, %15, 0xF3; bra.uni GDONE;\n"
        "G12: lop3.b32 %0, %0, %8, %8, 0x0F; lop3.b32 %1, %1, %9, %9, 0x0F; lop3.b32 %2, %2, %10, %10, 0x0F; lop3.b32 %3, %3, %11, %11, 0x0F; lop3.b32 %4, %4, %12, %12, 0x0F; lop3.b32 %5, %5, %13, %13, 0x0F; lop3.b32 %6, %6, %14, %14, 0x0F; lop3.b32 %7, %7, %15, %15, 0x0F; bra.uni GDONE;\n"
        "G13: lop3.b32 %0, %0, %8, %8, 0xCF; lop3.b32 %1, %1, %9, %9, 0xCF; lop3.b32 %2, %2, %10, %10, 0xCF; lop3.b32 %3, %3, %11, %11, 0xCF; lop3.b32 %4, %4, %12, %12, 0xCF; lop3.b32 %5, %5, %13, %13, 0xCF; lop3.b32 %6, %6, %14, %14, 0xCF; lop3.b32 %7, %7, %15, %15, 0xCF; bra.uni GDONE;\n"
        "G14: lop3.b32 %0, %0, %8, %8, 0x3F; lop3.b32 %1, %1, %9, %9, 0x3F; lop3.b32 %2, %2, %10, %10, 0x3F; lop3.b32 %3, %3, %11, %11, 0x3F; lop3.b32 %4, %4, %12, %12, 0x3F; lop3.b32 %5, %5, %13, %13, 0x3F; lop3.b32 %6, %6, %14, %14, 0x3F; lop3.b32 %7, %7, %15, %15, 0x3F; bra.uni GDONE;\n"
        "G15: lop3.b32 %0, %0, %8, %8, 0xFF; lop3.b32 %1, %1, %9, %9, 0xFF; lop3.b32 %2, %2, %10, %10, 0xFF; lop3.b32 %3, %3, %11, %11, 0xFF; lop3.b32 %4, %4, %12, %12, 0xFF; lop3.b32 %5, %5, %13, %13, 0xFF; lop3.b32 %6, %6, %14, %14, 0xFF; lop3.b32 %7, %7, %15, %15, 0xFF; bra.uni GDONE;\n"
        "GDONE:\n\t}"
        : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7])
        : "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(b[4]), "r"(b[5]), "r"(b[6]), "r"(b[7]), "r"(op));
}

// Branch-free form of the same: the gate as a two-level multiplexer over four block-uniform masks, three lop3 per word
// (0xCA = a ? b : c) and no switch.  MUX selects it at compile time.
template <int N>
__device__ __forceinline__ void gate_words_mux(int op, unsigned (&a)[N], const unsigned (&b)[N])
{
    const unsigned m00 = (op & 8) ? ~0u : 0u, m01 = (op & 4) ? ~0u : 0u, m10 = (op & 2) ? ~0u : 0u, m11 = (op & 1) ? ~0u : 0u;
#pragma unroll
    for (int w = 0; w < N; ++w) {
        unsigned r1, r0;
        asm("lop3.b32 %0, %1, %2, %3, 0xCA;" : "=r"(r1) : "r"(b[w]), "r"(m11), "r"(m10));
        asm("lop3.b32 %0, %1, %2, %3, 0xCA;" : "=r"(r0) : "r"(b[w]), "r"(m01), "r"(m00));
        asm("lop3.b32 %0, %0, %1, %2, 0xCA;" : "+r"(a[w]) : "r"(r1), "r"(r0));
    }
}
template <bool MUX, int N> __device__ __forceinline__ void gate_apply(int op, unsigned (&a)[N], const unsigned (&b)[N])
{
    if (MUX)
        gate_words_mux<N>(op, a, b);
    else
        gate_words_brx(op, a, b);
}

// two 16-byte shared-memory loads (left and right conv column of a tap) into eight words
__device__ __forceinline__ void lds_pair(unsigned (&d)[8], unsigned addr0, unsigned addr1)
{
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(addr0));
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]) : "r"(addr1));
}

// one pooled output piece straight from global memory, for selections the tile does not cover
__device__ __noinline__ uint4 slab_window_global(const uint4 *__restrict__ xg, const SlabRec &R, const SlabShape &s, int py, int px)
{
    const int HW = s.H * s.W;
    Masks32 gm[7];
    for (int g = 0; g < 7; ++g) {
        const int op = R.op[g];
        gm[g].m00 = (op & 8) ? ~0u : 0u, gm[g].m01 = (op & 4) ? ~0u : 0u, gm[g].m10 = (op & 2) ? ~0u : 0u, gm[g].m11 = (op & 1) ? ~0u : 0u;
    }
    uint4 acc = make_uint4(0u, 0u, 0u, 0u);
    for (int d = 0; d < 4; ++d) {
        uint4 a[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int word = R.word[k];
            const int ch = min((word >> 16) & 0xFFFF, s.Ci - 1);
            const int iy = 2 * py + (d >> 1) + ((word >> 8) & 0xFF) - s.ph, ix = 2 * px + (d & 1) + (word & 0xFF) - s.pw;
            a[k] = ((unsigned)iy < (unsigned)s.H && (unsigned)ix < (unsigned)s.W) ? __ldg(xg + (size_t)ch * s.U * HW + iy * s.W + ix)
                                                                                : make_uint4(0u, 0u, 0u, 0u);
        }
        const uint4 g0 = mux128(gm[0], a[0], a[1]), g1 = mux128(gm[1], a[2], a[3]);
        const uint4 g2 = mux128(gm[2], a[4], a[5]), g3 = mux128(gm[3], a[6], a[7]);
        const uint4 t0 = mux128(gm[4], g0, g1), t1 = mux128(gm[5], g2, g3);
        const uint4 z = mux128(gm[6], t0, t1);
        acc.x |= z.x, acc.y |= z.y, acc.z |= z.z, acc.w |= z.w;
    }
    return acc;
}

// one record per output channel
__global__ void packed_slab_records_kernel(const uint8_t *__restrict__ ops, const int32_t *__restrict__ sel, SlabRec *__restrict__ recs,
                                           SlabShape s)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= s.C) return;
    SlabRec R;
    int ch0 = 0, ch1 = -1;
    bool all = true;
    for (int k = 0; k < 8; ++k) {
        const int w = sel[c * 8 + k];
        const int ch = min((w >> 16) & 0xFFFF, s.Ci - 1), r = (w >> 8) & 0xFF, sx = w & 0xFF;
        if (k == 0) ch0 = ch;
        if (ch1 < 0 && ch != ch0) ch1 = ch;
        all = all && (ch == ch0 || ch == ch1) && r < s.kh && sx < s.kw;
        const int rr = min(r, s.kh - 1), sc = min(sx, s.kw - 1);
        const int base = (ch == ch0 ? 0 : s.CS) + rr * 2 * s.pwh;
        R.tb0[k] = 16 * (base + (sc & 1) * s.pwh + (sc >> 1));
        R.tb1[k] = 16 * (base + ((sc + 1) & 1) * s.pwh + ((sc + 1) >> 1));
        R.word[k] = w;
        R.op[k] = k < 7 ? ops[c * 7 + k] : 0;
    }
    R.ch[0] = ch0, R.ch[1] = ch1 < 0 ? ch0 : ch1, R.nst = ch1 < 0 ? 1 : 2, R.all_in_tile = all;
    recs[c] = R;
}

template <bool MUX>
__global__ void __launch_bounds__(256, 2) packed_convtree_slab_kernel(const uint4 *__restrict__ x,
                                                                      const SlabRec *__restrict__ recs, uint4 *__restrict__ y,
                                                                      SlabShape s)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ __align__(16) SlabRec rec[3];
    uint4 *tile = reinterpret_cast<uint4 *>(smem_raw);
    const int tid = threadIdx.x, nt = blockDim.x;
    const int HW = s.H * s.W;
    const int buf_elems = s.UB * s.SS;
    int *copy_off = reinterpret_cast<int *>(tile + 2 * buf_elems); // [per_thread][nt] tile offsets of a thread's copies
    for (int i = tid; i < 2 * buf_elems; i += nt) tile[i] = make_uint4(0u, 0u, 0u, 0u);
    for (int q = tid; q < s.per_thread * nt; q += nt) {
        const int ub = q / HW, p = q - ub * HW, row = p / s.W, xp = p - row * s.W + s.pw;
        copy_off[q] = ub * s.SS + (row + s.ph) * 2 * s.pwh + (xp & 1) * s.pwh + (xp >> 1);
    }

    // the record of an item's output channel: 9 x 16 bytes from the table the record kernel wrote
    auto fetch_rec = [&](int c, SlabRec &R) {
        for (int j = tid; j < (int)(sizeof(SlabRec) / 16); j += nt) // a block may have fewer threads than pieces
            cp_async16(reinterpret_cast<uint4 *>(&R) + j, reinterpret_cast<const uint4 *>(recs + c) + j);
    };
    // copies of the planes of an item whose record is already visible
    auto stage = [&](int ug, const SlabRec &R, uint4 *dst) {
        const int u0 = ug * s.UB;
        const int n = min(s.UB, s.U - u0) * HW;
        if (!R.all_in_tile) return;
        for (int slot = 0; slot < R.nst; ++slot) {
            const uint4 *src = x + ((size_t)R.ch[slot] * s.U + u0) * HW;
            uint4 *d = dst + slot * s.CS;
            for (int j = 0, q = tid; j < s.per_thread && q < n; ++j, q += nt) cp_async16(d + copy_off[q], src + q);
        }
    };

    const int Hp = s.Ho / 2, Wp = s.Wo / 2, I = Hp * Wp;
    const int ub = tid / I, win = tid - ub * I;
    const int py = win / Wp, px = win - py * Wp;
    const int toff = ub * s.SS + 2 * py * 2 * s.pwh + px;
    const int RS = 2 * s.pwh;

    // items are (slab group ug, output channel c), c fastest: the blocks that run at the same time work on the same
    // few slabs of ALL input channels (a few MB, L2-resident) instead of all slabs of a few channels, so the planes are
    // fetched from DRAM once although every input channel is read by several output channels.  A block takes every
    // gridDim.x-th item and keeps the (c, ug) of its current and next two items by carrying additions instead of dividing.
    const int first = blockIdx.x, stride = gridDim.x;
    const int dug = stride / s.C, dc = stride - dug * s.C;
    auto advance = [&](int &c, int &ug) {
        c += dc, ug += dug;
        if (c >= s.C) c -= s.C, ++ug;
    };
    int ug0 = first / s.C, c0 = first - ug0 * s.C, c1 = c0, ug1 = ug0;
    advance(c1, ug1);
    int c2 = c1, ug2 = ug1;
    advance(c2, ug2);
    if (ug0 < s.n_ug) fetch_rec(c0, rec[0]);
    if (ug1 < s.n_ug) fetch_rec(c1, rec[1]);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads(); // records, copy offsets and halo zeros in place
    if (ug0 < s.n_ug) stage(ug0, rec[0], tile);
    cp_async_commit();
    int cur = 0, r0 = 0; // tile buffer and record slot of the current item
    for (; ug0 < s.n_ug; cur ^= 1, r0 = r0 == 2 ? 0 : r0 + 1) {
        const int r1 = r0 == 2 ? 0 : r0 + 1, r2 = r1 == 2 ? 0 : r1 + 1;
        // one barrier per item: this item's planes and the next item's record have landed, and every thread is
        // done with the previous item, whose tile buffer and whose predecessor's record slot are refilled now
        cp_async_wait<0>();
        __syncthreads();
        if (ug2 < s.n_ug) fetch_rec(c2, rec[r2]);
        if (ug1 < s.n_ug) stage(ug1, rec[r1], tile + (cur ^ 1) * buf_elems);
        cp_async_commit();
        const int c = c0, u0 = ug0 * s.UB;
        c0 = c1, ug0 = ug1, c1 = c2, ug1 = ug2;
        advance(c2, ug2);

        const SlabRec &R = rec[r0];
        if (ub < min(s.UB, s.U - u0)) {
            uint4 out;
            if (R.all_in_tile) {
                // tile offsets in the record are in bytes; a tap's two columns for the two conv rows of the window
                const unsigned t0 = (unsigned)__cvta_generic_to_shared(tile + cur * buf_elems + toff);
                const int4 o0a = *reinterpret_cast<const int4 *>(&R.tb0[0]), o0b = *reinterpret_cast<const int4 *>(&R.tb0[4]);
                const int4 o1a = *reinterpret_cast<const int4 *>(&R.tb1[0]), o1b = *reinterpret_cast<const int4 *>(&R.tb1[4]);
                const int4 opa = *reinterpret_cast<const int4 *>(&R.op[0]), opb = *reinterpret_cast<const int4 *>(&R.op[4]);
                const int o0[8] = {o0a.x, o0a.y, o0a.z, o0a.w, o0b.x, o0b.y, o0b.z, o0b.w};
                const int o1[8] = {o1a.x, o1a.y, o1a.z, o1a.w, o1b.x, o1b.y, o1b.z, o1b.w};
                const int op[7] = {opa.x, opa.y, opa.z, opa.w, opb.x, opb.y, opb.z};
                unsigned acc[4] = {0u, 0u, 0u, 0u};
                // The two conv rows of the window run through ONE copy of the code (the loop is not unrolled): the seven
                // 16-way gate switches are about 150 instructions each, and with fourteen of them the kernel did not fit
                // the instruction cache (stall reason "no instruction").  Inside a row the taps of the next gate are
                // fetched before the current gate's switch, so that the shared-memory latency runs under it (fetching all
                // sixteen loads of a row up front instead was measured slower: 2.49 -> 2.79 ms over the four c4 blocks).
#pragma unroll 1
                for (int dy = 0; dy < 2; ++dy) {
                    const unsigned tn = t0 + dy * RS * 16;
                    unsigned g[4][8], b[4][8];
                    lds_pair(g[0], tn + o0[0], tn + o1[0]);
                    lds_pair(b[0], tn + o0[1], tn + o1[1]);
#pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        if (p < 3) {
                            lds_pair(g[p + 1], tn + o0[2 * p + 2], tn + o1[2 * p + 2]);
                            lds_pair(b[p + 1], tn + o0[2 * p + 3], tn + o1[2 * p + 3]);
                        }
                        gate_apply<MUX, 8>(op[p], g[p], b[p]);
                    }
                    gate_apply<MUX, 8>(op[4], g[0], g[1]);
                    gate_apply<MUX, 8>(op[5], g[2], g[3]);
                    gate_apply<MUX, 8>(op[6], g[0], g[2]);
#pragma unroll
                    for (int w = 0; w < 4; ++w) acc[w] |= g[0][w] | g[0][w + 4];
                }
                out = make_uint4(acc[0], acc[1], acc[2], acc[3]);
            } else {
                out = slab_window_global(x + (size_t)(u0 + ub) * HW, R, s, py, px);
            }
            y[((size_t)c * s.U + u0 + ub) * I + win] = out;
        }
    }
    cp_async_wait<0>();
}

// rows [F][2U] of 64-bit words  <->  slab [C][U][HW] of uint4, F = C*HW (pure data movement)
__global__ void packed_rows_to_slab_kernel(const uint4 *__restrict__ rows, uint4 *__restrict__ slab, int C, int HW, int U, int to_slab)
{
    const long long total = (long long)C * HW * U;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        // i enumerates the rows layout: ((c*HW + p)*U + u)
        const int u = (int)(i % U);
        const long long cp = i / U;
        const int p = (int)(cp % HW);
        const long long c = cp / HW;
        const long long j = (c * U + u) * HW + p;
        if (to_slab)
            slab[j] = rows[i];
        else
            slab[i] = rows[j]; // here `rows` is the slab tensor and `slab` the rows tensor
    }
}

} // namespace clb

using namespace clb;
using namespace clb_host;

static bool bits_ok(int bits) { return bits == 8 || bits == 16 || bits == 32 || bits == 64; }
static bool aligned_to(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
static int flat_grid(long long items, int threads)
{
    long long blocks = (items + threads - 1) / threads;
    const long long cap = (long long)sm_count() * 32;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

extern "C" int clb_pack_bits(const uint8_t *t, void *packed, int64_t F, int64_t B, int bits, void *stream)
{
    if (!t || !packed || F < 0 || B < 0 || !bits_ok(bits)) return CLB_ERR_ARG;
    const long long words = (B + bits - 1) / bits, rowbytes = words * (bits / 8);
    if (F == 0 || rowbytes == 0) return CLB_OK;
    CLB_TRACED("pack_bits_kernel", (cudaStream_t)stream, pack_bits_kernel<<<flat_grid(F * rowbytes, 256), 256, 0, (cudaStream_t)stream>>>(t, (uint8_t *)packed, F, B, rowbytes));
    return check_launch();
}

extern "C" int clb_pack_bits_nmajor(const uint8_t *t, void *packed, int64_t N, int64_t F, int bits, void *stream)
{
    if (!t || !packed || F < 0 || N < 0 || !bits_ok(bits)) return CLB_ERR_ARG;
    const long long words = (N + bits - 1) / bits, rowbytes = words * (bits / 8);
    if (F == 0 || rowbytes == 0) return CLB_OK;
    long long gy = (rowbytes + 31) / 32;
    if (gy > 4096) gy = 4096;
    dim3 grid((unsigned)((F + 255) / 256), (unsigned)gy);
    CLB_TRACED("pack_bits_nmajor_kernel", (cudaStream_t)stream, pack_bits_nmajor_kernel<32><<<grid, 256, 0, (cudaStream_t)stream>>>(t, (uint8_t *)packed, N, F, rowbytes));
    return check_launch();
}

extern "C" int clb_thermometer_pack(const void *pixels, int pixels_u8, const float *thresholds, int levels, void *packed, int64_t N,
                                    int64_t channels, int64_t HW, int64_t words, int to_slab, void *stream)
{
    if (!pixels || !thresholds || !packed || levels <= 0 || N < 0 || channels <= 0 || HW <= 0 || words < 0) return CLB_ERR_ARG;
    const long long P = channels * HW;
    if (P > 0x7fffffff || (long long)levels * P > 0x7fffffffLL * 16) return CLB_ERR_SHAPE;
    const long long need = (N + 63) / 64;
    if (words == 0) words = need;
    if (words < need || words > need + 1) return CLB_ERR_SHAPE; // rows of ceil(N/64) words, or one more to reach an even count
    if (words == 0) return CLB_OK;
    const long long words32 = words * 2;
    if (to_slab && (words32 % 4)) return CLB_ERR_SHAPE; // a slab unit is 128 samples
    if (!aligned_to(packed, 16)) return CLB_ERR_ARG;
    const long long gy = (words32 + 7) / 8; // a block writes 8 half-words of every row: all of them are written, bits beyond N as zeros
    if (gy > 65535) return CLB_ERR_SHAPE;
    dim3 grid((unsigned)((P + 31) / 32), (unsigned)gy);
    cudaStream_t st = (cudaStream_t)stream;
    if (pixels_u8)
        CLB_TRACED("thermometer_pack_kernel", st, thermometer_pack_kernel<uint8_t><<<grid, 256, 0, st>>>((const uint8_t *)pixels, thresholds, levels, (unsigned *)packed, N, (int)P,
                                                                (int)HW, words32, to_slab));
    else
        CLB_TRACED("thermometer_pack_kernel", st, thermometer_pack_kernel<float><<<grid, 256, 0, st>>>((const float *)pixels, thresholds, levels, (unsigned *)packed, N, (int)P, (int)HW,
                                                              words32, to_slab));
    return check_launch();
}

extern "C" int clb_packed_logic(const void *x, const int64_t *a, const int64_t *b, const uint8_t *ops, void *y, int64_t in_dim,
                                int64_t out_dim, int64_t words, int bits, void *stream)
{
    if (!x || !a || !b || !ops || !y || in_dim <= 0 || out_dim < 0 || words < 0 || !bits_ok(bits)) return CLB_ERR_ARG;
    const long long rowbytes = words * (bits / 8);
    if (out_dim == 0 || rowbytes == 0) return CLB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (rowbytes % 16 == 0 && aligned_to(x, 16) && aligned_to(y, 16)) {
        const long long units = rowbytes / 16;
        CLB_TRACED("packed_logic_v4_kernel", st, packed_logic_v4_kernel<<<flat_grid(out_dim * units, 256), 256, 0, st>>>((const uint4 *)x, a, b, ops, (uint4 *)y, out_dim, units));
    } else if (rowbytes % 8 == 0 && aligned_to(x, 8) && aligned_to(y, 8)) {
        const long long units = rowbytes / 8;
        CLB_TRACED("packed_logic_kernel", st, packed_logic_kernel<unsigned long long><<<flat_grid(out_dim * units, 256), 256, 0, st>>>(
            (const unsigned long long *)x, a, b, ops, (unsigned long long *)y, out_dim, units));
    } else {
        CLB_TRACED("packed_logic_kernel", st, packed_logic_kernel<uint8_t><<<flat_grid(out_dim * rowbytes, 256), 256, 0, st>>>((const uint8_t *)x, a, b, ops, (uint8_t *)y,
                                                                                        out_dim, rowbytes));
    }
    return check_launch();
}

extern "C" int clb_packed_tree(const void *x, const int32_t *leaf, const uint8_t *ops, void *y, int64_t in_dim, int64_t out_dim, int levels,
                               int64_t words, int bits, void *stream)
{
    if (!x || !leaf || !ops || !y || in_dim <= 0 || out_dim < 0 || words < 0 || !bits_ok(bits) || (levels != 2 && levels != 3))
        return CLB_ERR_ARG;
    if (in_dim > 0x7fffffffLL) return CLB_ERR_SHAPE;
    const long long rowbytes = words * (bits / 8);
    if (out_dim == 0 || rowbytes == 0) return CLB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (rowbytes % 16 == 0 && aligned_to(x, 16) && aligned_to(y, 16)) {
        const long long units = rowbytes / 16;
        // The leaves are gathered from all over the input: when it is larger than about three quarters of the 126 MB L2, the
        // rows are walked in pieces (a range of units = a range of samples at a time), so that the piece of the input in
        // use stays cached.  Measured on a 134 MB input: 0.64 ms in one piece, 0.50 in two or four, 0.56 in eight.
        long long pieces = 1;
        while (in_dim * rowbytes / pieces > (96LL << 20) && units % (pieces * 2) == 0 && units / (pieces * 2) >= 8) pieces *= 2;
        const long long u_n = units / pieces;
        const int grid = flat_grid(out_dim * u_n, 256);
        for (long long pc = 0; pc < pieces; ++pc) {
            if (levels == 2)
                CLB_TRACED("packed_tree_kernel", st,
                           packed_tree_kernel<uint4, 2, long long><<<grid, 256, 0, st>>>((const uint4 *)x, leaf, ops, (uint4 *)y, out_dim, units, pc * u_n, u_n));
            else
                if (in_dim * units < 0xffffffffLL)
                    CLB_TRACED("packed_tree_kernel", st,
                               packed_tree_kernel<uint4, 3, unsigned><<<grid, 256, 0, st>>>((const uint4 *)x, leaf, ops, (uint4 *)y, out_dim, units, pc * u_n, u_n));
                else
                    CLB_TRACED("packed_tree_kernel", st,
                               packed_tree_kernel<uint4, 3, long long><<<grid, 256, 0, st>>>((const uint4 *)x, leaf, ops, (uint4 *)y, out_dim, units, pc * u_n, u_n));
        }
        return check_launch((int)pieces);
    } else if (rowbytes % 8 == 0 && aligned_to(x, 8) && aligned_to(y, 8)) {
        const long long units = rowbytes / 8;
        const int grid = flat_grid(out_dim * units, 256);
        if (levels == 2)
            CLB_TRACED("packed_tree_kernel", st, packed_tree_kernel<uint2, 2, long long><<<grid, 256, 0, st>>>((const uint2 *)x, leaf, ops, (uint2 *)y, out_dim, units, 0, units));
        else
            CLB_TRACED("packed_tree_kernel", st, packed_tree_kernel<uint2, 3, long long><<<grid, 256, 0, st>>>((const uint2 *)x, leaf, ops, (uint2 *)y, out_dim, units, 0, units));
    } else {
        return CLB_ERR_SHAPE; // rows of 64-bit words only
    }
    return check_launch();
}

extern "C" int clb_group_popcount(const void *x, int32_t *counts, int64_t F, int64_t words, int bits, int pad_len, int k,
                                  void *stream)
{
    if (!x || !counts || F < 0 || words < 0 || !bits_ok(bits) || k <= 0 || pad_len < 0 || pad_len >= bits) return CLB_ERR_ARG;
    if (F % k) return CLB_ERR_SHAPE;
    const long long rowbytes = words * (bits / 8);
    const long long B = words * bits - pad_len;
    if (B <= 0) return CLB_OK;
    const long long S = F / k;
    cudaStream_t st = (cudaStream_t)stream;
    if (rowbytes % 4 == 0 && aligned_to(x, 4)) {
        const long long units = rowbytes / 4;
        long long splits = 1;
        while ((long long)k * splits * units < (long long)sm_count() * 128 * 16 && S / (splits * 2) >= 64) splits *= 2; // 16 resident blocks per SM: the row loop is latency-bound
        if (splits > 1) {
            if (cudaMemsetAsync(counts, 0, (size_t)B * k * sizeof(int32_t), st) != cudaSuccess) return check_launch();
        }
        const long long per = ((S + splits - 1) / splits + 15) / 16 * 16; // rows per thread, as the kernel computes it
        if (per <= 16 * 256)
            CLB_TRACED("group_popcount_kernel", st, group_popcount_kernel<8><<<flat_grid((long long)k * splits * units, 128), 128, 0, st>>>((const unsigned *)x, counts, S, units, B, k,
                                                                                                    (int)splits));
        else
            CLB_TRACED("group_popcount_kernel", st, group_popcount_kernel<27><<<flat_grid((long long)k * splits * units, 128), 128, 0, st>>>((const unsigned *)x, counts, S, units, B,
                                                                                                     k, (int)splits));
    } else {
        CLB_TRACED("group_popcount_bytes_kernel", st, group_popcount_bytes_kernel<<<flat_grid(B * k, 256), 256, 0, st>>>((const uint8_t *)x, counts, S, rowbytes, B, k));
    }
    return check_launch();
}

extern "C" int clb_packed_convtree(const void *x, const uint8_t *ops, const int32_t *sel, void *y, int Ci, int H, int W, int C,
                                   int sh, int sw, int ph, int pw, int kh, int kw, int64_t words, int bits, void *stream)
{
    if (!conv_args_ok(1, Ci, H, W, C, sh, sw, ph, pw, kh, kw) || !x || !ops || !sel || !y || words < 0 || !bits_ok(bits))
        return CLB_ERR_ARG;
    PackedShape s{Ci, H, W, C, conv_out(H, ph, kh, sh), conv_out(W, pw, kw, sw), sh, sw, ph, pw};
    if (s.Ho <= 0 || s.Wo <= 0) return CLB_ERR_SHAPE;
    if ((s.Ho & 1) || (s.Wo & 1)) return CLB_ERR_ODD_OUTPUT;
    if (C > 65535) return CLB_ERR_SHAPE;
    const long long rowbytes = words * (bits / 8);
    if (C == 0 || rowbytes == 0) return CLB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const long long wins = (long long)(s.Ho / 2) * (s.Wo / 2);
    const long long in_units16 = (long long)Ci * H * W * (rowbytes / 16), out_units16 = (long long)C * wins * (rowbytes / 16);
    if (rowbytes % 16 == 0 && aligned_to(x, 16) && aligned_to(y, 16) && in_units16 < (1LL << 30) && out_units16 < (1LL << 30)) {
        const int units = (int)(rowbytes / 16);
        long long gx = (wins * units + 255) / 256;
        const long long cap = ((long long)sm_count() * 32 + C - 1) / C;
        if (gx > cap) gx = cap;
        dim3 grid((unsigned)(gx < 1 ? 1 : gx), C);
        CLB_TRACED("packed_convtree_v4_kernel", st, packed_convtree_v4_kernel<<<grid, 256, 0, st>>>((const uint4 *)x, ops, sel, (uint4 *)y, s, units));
    } else if (rowbytes % 8 == 0 && aligned_to(x, 8) && aligned_to(y, 8)) {
        const long long units = rowbytes / 8;
        long long gx = (wins * units + 255) / 256;
        const long long cap = ((long long)sm_count() * 32 + C - 1) / C;
        if (gx > cap) gx = cap;
        dim3 grid((unsigned)(gx < 1 ? 1 : gx), C);
        CLB_TRACED("packed_convtree_kernel", st, packed_convtree_kernel<unsigned long long><<<grid, 256, 0, st>>>((const unsigned long long *)x, ops, sel,
                                                                         (unsigned long long *)y, s, units));
    } else {
        long long gx = (wins * rowbytes + 255) / 256;
        const long long cap = ((long long)sm_count() * 32 + C - 1) / C;
        if (gx > cap) gx = cap;
        dim3 grid((unsigned)(gx < 1 ? 1 : gx), C);
        CLB_TRACED("packed_convtree_kernel", st, packed_convtree_kernel<uint8_t><<<grid, 256, 0, st>>>((const uint8_t *)x, ops, sel, (uint8_t *)y, s, rowbytes));
    }
    return check_launch();
}

extern "C" int clb_packed_layout(const void *src, void *dst, int64_t C, int64_t HW, int64_t U, int to_slab, void *stream)
{
    if (!src || !dst || C < 0 || HW < 0 || U < 0) return CLB_ERR_ARG;
    if (!aligned_to(src, 16) || !aligned_to(dst, 16)) return CLB_ERR_ARG;
    if (C > 0x7fffffff || HW > 0x7fffffff || U > 0x7fffffff) return CLB_ERR_SHAPE;
    const long long total = C * HW * U;
    if (total == 0) return CLB_OK;
    CLB_TRACED("packed_rows_to_slab_kernel", (cudaStream_t)stream, packed_rows_to_slab_kernel<<<flat_grid(total, 256), 256, 0, (cudaStream_t)stream>>>((const uint4 *)src, (uint4 *)dst, (int)C, (int)HW,
                                                                                        (int)U, to_slab));
    return check_launch();
}

extern "C" int64_t clb_packed_convtree_slab_scratch_bytes(int C) { return C < 0 ? 0 : (int64_t)C * (int64_t)sizeof(SlabRec); }

extern "C" int clb_packed_convtree_slab(const void *x, const uint8_t *ops, const int32_t *sel, void *y, void *scratch, int Ci, int H,
                                        int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int64_t U, void *stream)
{
    if (!conv_args_ok(1, Ci, H, W, C, sh, sw, ph, pw, kh, kw) || !x || !ops || !sel || !y || U < 0) return CLB_ERR_ARG;
    if (!aligned_to(x, 16) || !aligned_to(y, 16) || (C > 0 && (!scratch || !aligned_to(scratch, 16)))) return CLB_ERR_ARG;
    if (sh != 1 || sw != 1) return CLB_ERR_SHAPE; // the rows layout serves other strides
    SlabShape s;
    s.Ci = Ci, s.H = H, s.W = W, s.C = C, s.ph = ph, s.pw = pw, s.kh = kh, s.kw = kw;
    s.Ho = conv_out(H, ph, kh, 1), s.Wo = conv_out(W, pw, kw, 1);
    if (s.Ho <= 0 || s.Wo <= 0) return CLB_ERR_SHAPE;
    if ((s.Ho & 1) || (s.Wo & 1)) return CLB_ERR_ODD_OUTPUT;
    const int I = (s.Ho / 2) * (s.Wo / 2);
    if (C > 65535 || I > 256 || U > 0x7fffffff) return CLB_ERR_SHAPE;
    if ((long long)Ci * U * H * W >= (1LL << 31) || (long long)C * U * I >= (1LL << 31)) return CLB_ERR_SHAPE;
    if (C == 0 || U == 0) return CLB_OK;
    s.U = (int)U;
    s.UB = 256 / I;
    if (s.UB > s.U) s.UB = s.U;
    s.PH = H + 2 * ph;
    s.pwh = (W + 2 * pw + 1) / 2;
    s.CS = s.PH * 2 * s.pwh;
    s.SS = 2 * s.CS;
    auto smem_of = [&](int ub) { // two buffers + copy offsets
        const int th = ub * I;
        return 2 * (size_t)ub * s.SS * 16 + (size_t)((ub * H * W + th - 1) / th) * th * 4;
    };
    while (s.UB > 1 && smem_of(s.UB) > 110 * 1024) s.UB = (s.UB + 1) / 2; // small images: the halo doubles the tile; keep two blocks per SM
    const int threads = s.UB * I;
    s.per_thread = (s.UB * H * W + threads - 1) / threads;
    const size_t smem = smem_of(s.UB);
    if (smem > 200 * 1024) return CLB_ERR_SHAPE;
    s.n_ug = (s.U + s.UB - 1) / s.UB;
    s.items = C * s.n_ug;
    const bool mux = tune_get(CLB_TUNE_SLAB_MUX) != 0;
    auto k = mux ? packed_convtree_slab_kernel<true> : packed_convtree_slab_kernel<false>;
    if (clb_host::ensure_dynamic_smem(k, (int)smem) != cudaSuccess) return check_launch(0);
    int bps = (int)((227 * 1024) / (smem + 1024));
    const int by_regs = 512 / threads < 2 ? 2 : (512 / threads > 8 ? 8 : 512 / threads); // 112 registers per thread
    if (bps > by_regs) bps = by_regs;
    if (bps < 1) bps = 1;
    int grid = sm_count() * bps;
    if (grid > s.items) grid = s.items;
    CLB_TRACED("packed_slab_records_kernel", (cudaStream_t)stream, packed_slab_records_kernel<<<(C + 127) / 128, 128, 0, (cudaStream_t)stream>>>(ops, sel, (SlabRec *)scratch, s));
    CLB_TRACED("packed_convtree_slab_kernel", (cudaStream_t)stream, k<<<grid, threads, smem, (cudaStream_t)stream>>>((const uint4 *)x, (const SlabRec *)scratch, (uint4 *)y, s));
    return check_launch();
}
