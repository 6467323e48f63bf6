// Compiled network: a discretised stack (fused ConvLogic blocks, flat LogicLayers, GroupSum) serialised into one
// blob and run by a single host call that enqueues the packed kernels of this library back to back.
// It plays the part of the reference's CompiledLogicNet (src/difflogic/compiled_model.py:41-361), which writes
// the gates out as C source and compiles it with gcc for the CPU and which cannot hold conv blocks; here the
// artefact is data (the blob), the code is this library, and the network runs on the GPU from any host
// language that can call C.
//
// Blob, little-endian, every array 16-byte aligned relative to the blob start:
//   header  (64 bytes): "CLBNET01", u32 n_layers, u32 num_classes, u32 in_channels, u32 in_h, u32 in_w,
//                       u32 in_features (flat input: in_channels = 0), u64 total_bytes, zero padding
//   layer i (64 bytes): u32 kind (1 fused conv block, 2 flat layer), u32 p[7], u64 off_a, u64 off_b, u64 off_ops, pad
//       conv: p = {Ci, C, kh, kw, stride, pad_h, pad_w}; off_a -> int32 sel[C][8]; off_ops -> u8 ops[C][7]
//       flat: p = {in_dim (lo), out_dim (lo), in_dim (hi), out_dim (hi)}; off_a / off_b -> int64 idx[out]; off_ops -> u8 ops[out]
//       kind 3, two or three flat layers fused into a gate tree (clb_packed_tree): p = {in_dim (lo), out_dim (lo), in_dim (hi),
//             out_dim (hi), levels}; off_a -> int32 leaf[out][2^levels]; off_ops -> u8 ops[out][2^levels - 1]
//   arrays
// The last flat layer's outputs are summed per class (GroupSum): counts[b][k].
#include "clb_common.cuh"

#include <cstring>
#include <new>
#include <vector>

using namespace clb_host;

namespace {

constexpr char kMagic[8] = {'C', 'L', 'B', 'N', 'E', 'T', '0', '1'};
constexpr size_t kHeaderBytes = 64, kLayerBytes = 64;

struct Header {
    char magic[8];
    uint32_t n_layers, num_classes, in_channels, in_h, in_w, in_features;
    uint64_t total_bytes;
};

struct LayerRec {
    uint32_t kind, p[7];
    uint64_t off_a, off_b, off_ops;
};

struct Layer {
    int kind;
    // conv
    int Ci, C, kh, kw, stride, ph, pw, H, W, Hp, Wp; // input extent and pooled output extent
    // flat (kind 2) and fused flat tree (kind 3)
    long long in_dim, out_dim;
    int levels;
    size_t off_a, off_b, off_ops;
};

} // namespace

struct clb_net {
    std::vector<Layer> layers;
    int num_classes = 0;
    int in_channels = 0, in_h = 0, in_w = 0;
    long long in_features = 0; // features of one sample at the input
    size_t param_bytes = 0;    // the blob is copied to the device as it is
    const unsigned char *dev = nullptr;
    size_t max_conv_channels = 0;
};

static bool parse(const void *blob, size_t bytes, clb_net &net)
{
    if (!blob || bytes < kHeaderBytes) return false;
    Header h;
    std::memcpy(&h, blob, sizeof(Header));
    if (std::memcmp(h.magic, kMagic, 8) != 0 || h.total_bytes != bytes || h.n_layers == 0 || h.n_layers > 4096 || h.num_classes == 0)
        return false;
    if (bytes < kHeaderBytes + (size_t)h.n_layers * kLayerBytes) return false;
    net.num_classes = (int)h.num_classes;
    net.in_channels = (int)h.in_channels, net.in_h = (int)h.in_h, net.in_w = (int)h.in_w;
    net.in_features = h.in_channels ? (long long)h.in_channels * h.in_h * h.in_w : (long long)h.in_features;
    if (net.in_features <= 0) return false;
    net.param_bytes = bytes;
    int C = net.in_channels, H = net.in_h, W = net.in_w; // running conv extent
    long long feat = net.in_features;
    bool flat_seen = false;
    auto in_blob = [&](uint64_t off, unsigned long long n) { return off % 16 == 0 && off <= bytes && n <= bytes - off; };
    const unsigned char *base = (const unsigned char *)blob; // arrays sit at 16-byte aligned offsets of a caller buffer
    for (uint32_t i = 0; i < h.n_layers; ++i) {
        LayerRec r;
        std::memcpy(&r, (const unsigned char *)blob + kHeaderBytes + (size_t)i * kLayerBytes, sizeof(LayerRec));
        Layer L{};
        L.kind = (int)r.kind;
        L.off_a = r.off_a, L.off_b = r.off_b, L.off_ops = r.off_ops;
        if (r.kind == 1) {
            if (flat_seen || C <= 0) return false; // conv blocks come first and need an image input
            L.Ci = (int)r.p[0], L.C = (int)r.p[1], L.kh = (int)r.p[2], L.kw = (int)r.p[3], L.stride = (int)r.p[4], L.ph = (int)r.p[5],
            L.pw = (int)r.p[6];
            if (L.Ci != C || L.C <= 0 || L.C > 65535 || L.stride <= 0 || !conv_args_ok(1, L.Ci, H, W, L.C, L.stride, L.stride, L.ph, L.pw, L.kh, L.kw))
                return false;
            const int Ho = conv_out(H, L.ph, L.kh, L.stride), Wo = conv_out(W, L.pw, L.kw, L.stride);
            if (Ho <= 0 || Wo <= 0 || (Ho & 1) || (Wo & 1)) return false;
            L.H = H, L.W = W, L.Hp = Ho / 2, L.Wp = Wo / 2;
            if (!in_blob(r.off_a, (unsigned long long)L.C * 32) || !in_blob(r.off_ops, (unsigned long long)L.C * 7)) return false;
            { // every tap must name a channel of the input and a cell of the window, every gate id one of the 16 gates
                const int32_t *selw = reinterpret_cast<const int32_t *>(base + r.off_a);
                for (long long t = 0; t < (long long)L.C * 8; ++t) {
                    const int32_t word = selw[t];
                    if (word < 0 || ((word >> 16) & 0xFFFF) >= L.Ci || ((word >> 8) & 0xFF) >= L.kh || (word & 0xFF) >= L.kw) return false;
                }
                const uint8_t *opsb = base + r.off_ops;
                for (long long t = 0; t < (long long)L.C * 7; ++t)
                    if (opsb[t] > 15) return false;
            }
            C = L.C, H = L.Hp, W = L.Wp;
            feat = (long long)C * H * W;
            if ((size_t)L.C > net.max_conv_channels) net.max_conv_channels = (size_t)L.C;
        } else if (r.kind == 2) {
            flat_seen = true;
            L.in_dim = (long long)r.p[0] | ((long long)r.p[2] << 32), L.out_dim = (long long)r.p[1] | ((long long)r.p[3] << 32);
            if (L.in_dim != feat || L.out_dim <= 0) return false;
            if (!in_blob(r.off_a, (unsigned long long)L.out_dim * 8) || !in_blob(r.off_b, (unsigned long long)L.out_dim * 8) ||
                !in_blob(r.off_ops, (unsigned long long)L.out_dim))
                return false;
            { // connection indices must name input features, gate ids one of the 16 gates
                const int64_t *ia = reinterpret_cast<const int64_t *>(base + r.off_a), *ib = reinterpret_cast<const int64_t *>(base + r.off_b);
                const uint8_t *opsb = base + r.off_ops;
                for (long long t = 0; t < L.out_dim; ++t)
                    if (ia[t] < 0 || ia[t] >= L.in_dim || ib[t] < 0 || ib[t] >= L.in_dim || opsb[t] > 15) return false;
            }
            feat = L.out_dim;
        } else if (r.kind == 3) {
            flat_seen = true;
            L.in_dim = (long long)r.p[0] | ((long long)r.p[2] << 32), L.out_dim = (long long)r.p[1] | ((long long)r.p[3] << 32);
            L.levels = (int)r.p[4];
            if (L.in_dim != feat || L.out_dim <= 0 || (L.levels != 2 && L.levels != 3) || L.in_dim > 0x7fffffffLL) return false;
            const unsigned long long leaves = 1ull << L.levels;
            if (!in_blob(r.off_a, (unsigned long long)L.out_dim * leaves * 4) || !in_blob(r.off_ops, (unsigned long long)L.out_dim * (leaves - 1)))
                return false;
            {
                const int32_t *leaf = reinterpret_cast<const int32_t *>(base + r.off_a);
                for (unsigned long long t = 0; t < (unsigned long long)L.out_dim * leaves; ++t)
                    if (leaf[t] < 0 || leaf[t] >= L.in_dim) return false;
                const uint8_t *opsb = base + r.off_ops;
                for (unsigned long long t = 0; t < (unsigned long long)L.out_dim * (leaves - 1); ++t)
                    if (opsb[t] > 15) return false;
            }
            feat = L.out_dim;
        } else {
            return false;
        }
        net.layers.push_back(L);
    }
    return feat % net.num_classes == 0;
}

extern "C" int clb_net_device_bytes(const void *blob, size_t bytes, size_t *device_bytes)
{
    clb_net tmp;
    if (!device_bytes) return CLB_ERR_ARG;
    if (!parse(blob, bytes, tmp)) return CLB_ERR_SHAPE;
    *device_bytes = bytes;
    return CLB_OK;
}

extern "C" int clb_net_create(const void *blob, size_t bytes, void *device_mem, void *stream, clb_net **out)
{
    if (!out || !device_mem || (reinterpret_cast<uintptr_t>(device_mem) & 15)) return CLB_ERR_ARG;
    clb_net *net = new (std::nothrow) clb_net;
    if (!net) return CLB_ERR_ARG;
    if (!parse(blob, bytes, *net)) {
        delete net;
        return CLB_ERR_SHAPE;
    }
    // the parameters travel as one copy; `blob` must stay valid until the stream has run it
    if (cudaMemcpyAsync(device_mem, blob, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream) != cudaSuccess) {
        delete net;
        return check_launch(0);
    }
    net->dev = (const unsigned char *)device_mem;
    *out = net;
    return CLB_OK;
}

extern "C" void clb_net_destroy(clb_net *net) { delete net; }

extern "C" int clb_net_info(const clb_net *net, int64_t *in_features, int *num_classes, int *n_layers)
{
    if (!net) return CLB_ERR_ARG;
    if (in_features) *in_features = net->in_features;
    if (num_classes) *num_classes = net->num_classes;
    if (n_layers) *n_layers = (int)net->layers.size();
    return CLB_OK;
}

// Activations ping-pong between two buffers sized for the widest layer; the batch is padded to 128 samples so
// that every pixel row is a whole number of 16-byte units (slab layout, 128-bit kernels).
static size_t row_bytes(int64_t batch) { return (size_t)((batch + 127) / 128) * 16; }
static size_t align256(size_t v) { return (v + 255) / 256 * 256; }

static size_t widest(const clb_net *net)
{
    long long m = net->in_features;
    for (const Layer &L : net->layers) {
        const long long f = L.kind == 1 ? (long long)L.C * L.Hp * L.Wp : L.out_dim;
        if (f > m) m = f;
    }
    return (size_t)m;
}

extern "C" size_t clb_net_workspace_bytes(const clb_net *net, int64_t batch)
{
    if (!net || batch <= 0) return 0;
    const size_t act = align256(widest(net) * row_bytes(batch));
    return 2 * act + align256((size_t)clb_packed_convtree_slab_scratch_bytes((int)net->max_conv_channels)) + 256;
}

// input_kind: 0 = bool / uint8 bits [batch][in_features]; 1 = float32 pixels, 2 = uint8 pixels [batch][pc][H*W] with
// `levels` thresholds (in_channels == levels * pc); 3 = packed rows [in_features][ceil(batch/128)*2] of 64-bit words.
extern "C" int clb_net_forward(const clb_net *net, int input_kind, const void *input, const float *thresholds, int levels, int64_t batch,
                               int32_t *counts, void *workspace, size_t workspace_bytes, void *stream)
{
    if (!net || !input || !counts || !workspace || batch <= 0 || input_kind < 0 || input_kind > 3) return CLB_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255)) return CLB_ERR_ARG;
    if (workspace_bytes < clb_net_workspace_bytes(net, batch)) return CLB_ERR_SCRATCH;
    const size_t rb = row_bytes(batch);
    const int64_t words = (int64_t)(rb / 8), U = (int64_t)(rb / 16);
    const size_t act = align256(widest(net) * rb);
    unsigned char *buf[2] = {(unsigned char *)workspace, (unsigned char *)workspace + act};
    void *scratch = (unsigned char *)workspace + 2 * act;
    const bool image = net->in_channels > 0;
    const Layer &first = net->layers.front();
    // conv blocks run on the slab layout where the kernel covers them (stride 1, <= 256 pooled outputs per image)
    auto slab_ok = [](const Layer &L) { return L.kind == 1 && L.stride == 1 && L.Hp * L.Wp <= 256; };
    bool slab = image && slab_ok(first);
    int cur = 0, st;

    // ---- input stage
    if (input_kind == 0) {
        if ((batch + 63) / 64 != words) { // pack_bits writes ceil(batch/64) words per row: clear the padding word first
            if (cudaMemsetAsync(buf[0], 0, (size_t)net->in_features * rb, (cudaStream_t)stream) != cudaSuccess) return check_launch(0);
            // rows of `words` words cannot be produced by a kernel that strides ceil(batch/64): pack into buf[1], then widen
            st = clb_pack_bits_nmajor((const uint8_t *)input, buf[1], batch, net->in_features, 64, stream);
            if (st != CLB_OK) return st;
            const size_t narrow = (size_t)((batch + 63) / 64) * 8;
            if (cudaMemcpy2DAsync(buf[0], rb, buf[1], narrow, narrow, (size_t)net->in_features, cudaMemcpyDeviceToDevice,
                                  (cudaStream_t)stream) != cudaSuccess)
                return check_launch(0);
        } else {
            st = clb_pack_bits_nmajor((const uint8_t *)input, buf[0], batch, net->in_features, 64, stream);
            if (st != CLB_OK) return st;
        }
        if (slab) {
            st = clb_packed_layout(buf[0], buf[1], net->in_channels, (int64_t)net->in_h * net->in_w, U, 1, stream);
            if (st != CLB_OK) return st;
            cur = 1;
        }
    } else if (input_kind == 1 || input_kind == 2) {
        if (!image || !thresholds || levels <= 0 || net->in_channels % levels) return CLB_ERR_SHAPE;
        st = clb_thermometer_pack(input, input_kind == 2, thresholds, levels, buf[0], batch, net->in_channels / levels,
                                  (int64_t)net->in_h * net->in_w, words, slab ? 1 : 0, stream);
        if (st != CLB_OK) return st;
    } else {
        if (slab) {
            st = clb_packed_layout(input, buf[0], net->in_channels, (int64_t)net->in_h * net->in_w, U, 1, stream);
            if (st != CLB_OK) return st;
        } else {
            if (cudaMemcpyAsync(buf[0], input, (size_t)net->in_features * rb, cudaMemcpyDeviceToDevice, (cudaStream_t)stream) != cudaSuccess)
                return check_launch(0);
        }
    }

    // ---- layers
    const unsigned char *P = net->dev;
    long long feat = net->in_features;
    for (size_t i = 0; i < net->layers.size(); ++i) {
        const Layer &L = net->layers[i];
        if (L.kind == 1) {
            const bool want_slab = slab_ok(L);
            if (slab != want_slab) { // change of layout between blocks
                st = clb_packed_layout(buf[cur], buf[cur ^ 1], L.Ci, (int64_t)L.H * L.W, U, want_slab ? 1 : 0, stream);
                if (st != CLB_OK) return st;
                cur ^= 1, slab = want_slab;
            }
            if (slab) {
                st = clb_packed_convtree_slab(buf[cur], P + L.off_ops, (const int32_t *)(P + L.off_a), buf[cur ^ 1], scratch, L.Ci, L.H, L.W,
                                              L.C, 1, 1, L.ph, L.pw, L.kh, L.kw, U, stream);
                if (st == CLB_ERR_SHAPE) { // a tile the slab kernel cannot hold: this block runs on the rows layout
                    st = clb_packed_layout(buf[cur], buf[cur ^ 1], L.Ci, (int64_t)L.H * L.W, U, 0, stream);
                    if (st != CLB_OK) return st;
                    cur ^= 1, slab = false;
                }
            }
            if (!slab)
                st = clb_packed_convtree(buf[cur], P + L.off_ops, (const int32_t *)(P + L.off_a), buf[cur ^ 1], L.Ci, L.H, L.W, L.C,
                                         L.stride, L.stride, L.ph, L.pw, L.kh, L.kw, words, 64, stream);
            if (st != CLB_OK) return st;
            cur ^= 1;
            feat = (long long)L.C * L.Hp * L.Wp;
            const bool last_conv = i + 1 == net->layers.size() || net->layers[i + 1].kind != 1;
            if (last_conv && slab) { // Flatten: back to feature rows
                st = clb_packed_layout(buf[cur], buf[cur ^ 1], L.C, (int64_t)L.Hp * L.Wp, U, 0, stream);
                if (st != CLB_OK) return st;
                cur ^= 1, slab = false;
            }
        } else if (L.kind == 2) {
            st = clb_packed_logic(buf[cur], (const int64_t *)(P + L.off_a), (const int64_t *)(P + L.off_b), P + L.off_ops, buf[cur ^ 1],
                                  L.in_dim, L.out_dim, words, 64, stream);
            if (st != CLB_OK) return st;
            cur ^= 1;
            feat = L.out_dim;
        } else {
            st = clb_packed_tree(buf[cur], (const int32_t *)(P + L.off_a), P + L.off_ops, buf[cur ^ 1], L.in_dim, L.out_dim, L.levels, words,
                                 64, stream);
            if (st != CLB_OK) return st;
            cur ^= 1;
            feat = L.out_dim;
        }
    }
    // ---- GroupSum: pad bits are the zero samples of the input, but gates such as NOT turn them on: exclude them
    const int pad = (int)(words * 64 - batch);
    if (pad >= 64) { // the kernel takes a pad below one word: count on the narrower view is not possible, so mask by size
        // rows are [feat][words]; a pad of 64..127 samples means the last word of every row is padding only
        // -> run the count on words-1 words per row through a strided copy
        const size_t narrow = (size_t)(words - 1) * 8;
        if (cudaMemcpy2DAsync(buf[cur ^ 1], narrow, buf[cur], rb, narrow, (size_t)feat, cudaMemcpyDeviceToDevice, (cudaStream_t)stream) !=
            cudaSuccess)
            return check_launch(0);
        return clb_group_popcount(buf[cur ^ 1], counts, feat, words - 1, 64, pad - 64, net->num_classes, stream);
    }
    return clb_group_popcount(buf[cur], counts, feat, words, 64, pad, net->num_classes, stream);
}
