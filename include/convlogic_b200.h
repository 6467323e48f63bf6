/*
 * convlogic_b200 -- C ABI of the B200 (sm_100a) logic-gate kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*,
 * a cudaStream_t), launches on that stream and returns immediately: nothing here allocates,
 * frees, synchronises the device, throws or exits.  The return value is CLB_OK (0) or a negative
 * CLB_ERR_* code; clb_status_string() gives the text.  Inputs are borrowed for the duration of the
 * launched work; outputs and any scratch buffer are supplied by the caller.
 *
 * The citations name the entry point of lkorinek/convlogic that each function stands in for
 * (paths inside that project).
 *
 * Conventions
 *   dtype   CLB_F32 or CLB_F64 for every floating tensor of one call.
 *   wmode   how the gate tensor `w` ([..., 16] per gate) is to be read:
 *             CLB_W_PROB     a mixture over the 16 gates (soft-max already applied, or one-hot);
 *             CLB_W_SOFTMAX  raw logits, soft-max taken inside the kernel;
 *             CLB_W_ARGMAX   raw logits, one-hot of the first arg-max taken inside the kernel.
 *           Backward functions given CLB_W_SOFTMAX return the gradient w.r.t. the logits, given
 *           CLB_W_PROB the gradient w.r.t. the mixture (what the reference's autograd Functions
 *           return).
 *   sel     int32 [C, 8] selection words, (channel << 16) | (row << 8) | col; taps (2p, 2p+1) feed
 *           first-level gate p (src/convlogic/convlogic_layer.py:175-179, 450-451).
 *   gates   slot order of a fused block's 7 gates: 0-3 first level, 4-5 second, 6 third
 *           (src/convlogic/cuda/full_convlogic_kernel.cu:6-8).
 */
#ifndef CONVLOGIC_B200_H
#define CONVLOGIC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CLB_OK 0
#define CLB_ERR_ARG (-1)         /* null pointer, bad enum value, negative size */
#define CLB_ERR_SHAPE (-2)       /* shapes inconsistent or outside what the kernels support */
#define CLB_ERR_LAUNCH (-3)      /* the CUDA runtime refused the launch; see clb_last_cuda_error() */
#define CLB_ERR_SCRATCH (-4)     /* scratch buffer missing or too small */
#define CLB_ERR_ODD_OUTPUT (-5)  /* fused block: conv output height/width must be even (2x2 pool) */
#define CLB_ERR_TOO_LARGE (-6)   /* size beyond a documented fixed maximum */

#define CLB_F32 0
#define CLB_F64 1

#define CLB_W_PROB 0
#define CLB_W_SOFTMAX 1
#define CLB_W_ARGMAX 2
/* OR-ed into wmode of the conv entry points: the selection may hold taps with row >= kh or col >= kw
 * (never produced by the reference's generate_selection, but accepted by its kernels).  Such
 * selections are served by the general kernels only; without this flag the caller guarantees
 * row < kh and col < kw for every tap. */
#define CLB_SEL_UNBOUNDED 0x100
/* OR this into `wmode` of clb_convtree_fwd / clb_convtree_bwd_plane: the block's output y (forward) or the upstream gradient
 * gy (backward) is feature-major, [C][Ho/2 * Wo/2][N] instead of [N][C][Ho/2][Wo/2] -- the layout the flat layers behind a
 * stack's last block work in (no transposed copy in between).  Only the many-channel plane kernels take it (3x3, stride 1,
 * padding 1, images of 16x16 / 8x8 / 4x4, fp32): CLB_ERR_SHAPE otherwise.  The arg-max bytes keep [N][C][windows]. */
#define CLB_Y_FEATURE_MAJOR 0x200

int clb_version(void);
const char *clb_status_string(int status);
/* cudaError_t value of the most recent failed launch made through this library by the calling thread. */
int clb_last_cuda_error(void);
/* Number of kernels this library has launched in the calling process since it was loaded. */
long long clb_kernel_launches(void);
/* Launch tracing, for benchmarks (no counterpart in the reference, which device-synchronises after every
 * launch instead).  clb_trace(1) drops earlier records and turns tracing on: from then on the library
 * brackets each of its main kernels' launches with two CUDA events on the launch's stream (a few
 * microseconds of host time per launch, nothing on the device).  clb_trace_report waits for the recorded
 * events, writes one line per kernel, "name<TAB>launches<TAB>total milliseconds", into buf (NUL-terminated,
 * truncated to cap), drops the records and returns the number of bytes the full text needs.
 * clb_trace(0) turns tracing off.  Not for use during stream capture. */
int clb_trace(int on);
long long clb_trace_report(char *buf, size_t cap);
/* Process-wide tuning knobs (no counterpart in the reference).  Set them before querying scratch sizes: the
 * *_scratch_bytes functions and the launches read the same values.  Returns CLB_ERR_ARG for an unknown key.
 *   CLB_TUNE_TAPGRAD_SLICE_BYTES  the two-pass backward of many-channel blocks (clb_convtree_bwd) can walk the batch
 *       in slices whose tap gradients ([slice][C][8][windows] fp32) fit this many bytes, so that they are still
 *       in the L2 cache when the second pass reads them; 0 = one slice (the whole batch), the default: on B200
 *       both passes are latency-bound, not HBM-bound, and the smaller launches of a sliced walk cost more than the
 *       saved HBM traffic returns (measured: 3.47 ms per cifar10_m step unsliced, 4.4 ms with 80 MiB slices,
 *       5.0 ms with 48 MiB). */
#define CLB_TUNE_TAPGRAD_SLICE_BYTES 1
/*   CLB_TUNE_PLANE_KERNELS  1 (default): many-channel fused blocks (fp32, stride 1, image width a multiple of 4) run on
 *       the kernels that stream two channel planes per output channel through shared memory with TMA loads
 *       (clb_convtree_fwd picks them by itself; clb_convtree_bwd_plane is their backward); 0: never. */
#define CLB_TUNE_PLANE_KERNELS 2
/*   CLB_TUNE_SLAB_MUX  how the packed ConvLogic block on the slab layout applies a gate to its words: 0 = a block-uniform
 *       16-way switch with one lop3 per word, 1 = a branch-free multiplexer over four masks, three lop3 per word. */
#define CLB_TUNE_SLAB_MUX 3
int clb_tune(int key, long long value);
long long clb_tune_get(int key);

/* ------------------------------------------------------------------------------------------------
 * Fused ConvLogic block: 8-tap gather -> 4 gates -> 2 gates -> 1 gate -> 2x2 max pool.
 * Replaces convlogic_cuda.full_convlogic_forward (src/convlogic/cuda/convlogic.cpp:39;
 * full_convlogic_kernel.cu:147-231).
 *   x [N,Ci,H,W]   w [C,7,16]   sel [C,8]   y [N,C,Ho/2,Wo/2],  Ho = (H + 2*ph - kh)/sh + 1.
 * Optional outputs (pass NULL to skip): amax uint8 [N,C,Ho/2,Wo/2] = 2*dy+dx of the first maximum
 * of each window; x2 [N,C,Ho,Wo,4], x3 [N,C,Ho,Wo,2] (the reference's intermediates);
 * idx int32 [N,C,(Ho/2)*(Wo/2)] = in_y*Wo + in_x of the first maximum.
 */
int clb_convtree_fwd(const void *x, const void *w, const int32_t *sel, void *y, uint8_t *amax, void *x2, void *x3,
                     int32_t *idx, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh,
                     int kw, int wmode, int dtype, void *stream);

/* Backward of a fused block with many input channels (both gradients, fp32, stride 1), on the kernels that stream the
 * two channel planes of an output channel through shared memory; stands in for full_convlogic_backward_x +
 * full_convlogic_backward_weight (src/convlogic/cuda/convlogic.cpp:40-44; full_convlogic_kernel.cu:365-461, 616-701)
 * on the layers behind the first one of a stack.  Pass 1 recomputes the gate chain at the saved arg-max, keeps the gate
 * sums and writes, per (image, output channel), the gradient of its two input planes; pass 2 adds, per input channel,
 * the planes of the output channels that read it (lists from clb_conv_channel_lists, built once per selection).
 * Deterministic, no floating-point atomics.  gw may be NULL.  Returns CLB_ERR_SHAPE when the shape is outside these
 * kernels' domain (use clb_convtree_bwd then); clb_convtree_bwd_plane_scratch_bytes returns 0 in that case.
 *   clb_conv_channel_lists: host function; start int32 [Ci + 1], entry int32 [<= 2 * C]; returns the entry count, or
 *   CLB_ERR_SHAPE when an output channel names more than two input channels or a tap outside the kh x kw window. */
int clb_conv_channel_lists(const int32_t *sel_host, int C, int Ci, int kh, int kw, int32_t *start, int32_t *entry, int entry_cap);
size_t clb_convtree_bwd_plane_scratch_bytes(int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw,
                                            int dtype);
int clb_convtree_bwd_plane(const void *gy, const void *x, const void *w, const int32_t *sel, const uint8_t *amax, void *gx, void *gw,
                           const int32_t *ch_start, const int32_t *ch_entry, void *scratch, size_t scratch_bytes, int N, int Ci,
                           int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int wmode, int dtype, void *stream);
/* Diagnostic (synchronises the device): *flag = 0 unless a bounded wait inside one of the plane kernels ever ran out. */
int clb_plane_error(int *flag);

/* Input gradient of the fused block; deterministic (no floating-point atomics).
 * Replaces convlogic_cuda.full_convlogic_backward_x (convlogic.cpp:40-41;
 * full_convlogic_kernel.cu:365-461).  gy like y, gx like x (fully overwritten).
 * amax may be NULL (the arg-max is then recomputed).  The input channels are processed in groups
 * of `cg` consecutive channels; grp_start int32 [G+1] / grp_list int32 [grp_start[G]] list, for each
 * group, the output channels with at least one tap in it (ascending).  Build them with
 * clb_conv_group_plan() + clb_conv_build_groups().
 * scratch is optional: with clb_convtree_bwd_x_scratch_bytes() bytes of it (0 = no use for it) the
 * fp32, stride-1, all-channels-in-shared-memory shapes run a faster tiled kernel that spreads the
 * output channels of an image over several thread blocks and adds their partial tiles in a fixed
 * order; without it (NULL / too small) the general kernel runs.
 */
size_t clb_convtree_bwd_x_scratch_bytes(int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh,
                                        int kw, int dtype);
int clb_convtree_bwd_x(const void *gy, const void *x, const void *w, const int32_t *sel, const uint8_t *amax,
                       void *gx, const int32_t *grp_start, const int32_t *grp_list, int cg, int nb, void *scratch,
                       size_t scratch_bytes, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw,
                       int kh, int kw, int wmode, int dtype, void *stream);

/* Both gradients of the fused block in one call (either output may be NULL).  For the fp32 shapes
 * the tiled kernels cover, one kernel recomputes the gate chain at the arg-max once and produces the
 * input gradient and the per-image-group basis sums of the gate gradient together; other shapes run
 * clb_convtree_bwd_x / clb_convtree_bwd_w one after the other.  scratch: clb_convtree_bwd_scratch_bytes()
 * (16-byte aligned); amax is required for the combined kernel (NULL falls back to the separate ones).
 * Stands in for the pair full_convlogic_backward_x + full_convlogic_backward_weight that the
 * reference's autograd Function calls back to back (src/convlogic/convlogic_layer.py:71-82). */
size_t clb_convtree_bwd_scratch_bytes(int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh,
                                      int kw, int want_gx, int want_gw, int dtype);
int clb_convtree_bwd(const void *gy, const void *x, const void *w, const int32_t *sel, const uint8_t *amax, void *gx,
                     void *gw, const int32_t *grp_start, const int32_t *grp_list, int cg, int nb, void *scratch,
                     size_t scratch_bytes, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh,
                     int kw, int wmode, int dtype, void *stream);

/* Host-side helpers for the tables above (pure CPU, no CUDA call).
 * clb_conv_group_plan: picks cg (channels per group) and nb (images per thread block) for a shape.
 * clb_conv_build_groups: sel_host int32 [C,8] in host memory -> grp_start [G+1], grp_list (capacity
 * list_cap entries, at most min(C*G, C*8)); returns the number of list entries or a negative status. */
int clb_conv_group_plan(int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int dtype,
                        int *cg, int *nb);
int clb_conv_build_groups(const int32_t *sel_host, int C, int Ci, int cg, int32_t *grp_start, int32_t *grp_list,
                          int list_cap);

/* Gate-weight gradient of the fused block; deterministic two-stage reduction.
 * Replaces convlogic_cuda.full_convlogic_backward_weight (convlogic.cpp:42-43;
 * full_convlogic_kernel.cu:616-701).  gw [C,7,16].  scratch: clb_convtree_bwd_w_scratch_bytes().
 */
size_t clb_convtree_bwd_w_scratch_bytes(int N, int C, int Ho, int Wo, int dtype);
int clb_convtree_bwd_w(const void *gy, const void *x, const void *w, const int32_t *sel, const uint8_t *amax,
                       void *gw, void *scratch, size_t scratch_bytes, int N, int Ci, int H, int W, int C, int sh,
                       int sw, int ph, int pw, int kh, int kw, int wmode, int dtype, void *stream);

/* Gate-weight gradient of the fused block for callers that cannot allocate GPU memory.
 * No counterpart in the reference (every reference entry point allocates through torch).
 * Some hosts of this library own no allocator they may call at this point: a plugin invoked inside a
 * framework's memory-planned region, a real-time loop that pre-allocates everything at start-up, or a
 * thin FFI caller that can pass pointers but has no device-memory API of its own.  For them the
 * partial sums that clb_convtree_bwd_w() keeps in a caller-supplied scratch buffer are kept in a
 * fixed 4 MiB array inside the library (clb_convtree_bwd_w_noalloc_max_bytes(); every GPU that loads
 * the library holds it until the process exits).  Arguments, results and kernels are otherwise those
 * of clb_convtree_bwd_w(); the call itself performs no cudaMalloc/cudaFree or other allocation.
 *   - Shapes whose scratch need (clb_convtree_bwd_w_scratch_bytes()) exceeds the array return
 *     CLB_ERR_TOO_LARGE and launch nothing.
 *   - The first call on each device looks the array's device address up (a one-off runtime query);
 *     make that first call outside any stream capture.
 *   - All calls on a device share the array, and it keeps whatever the previous call left there.
 *     Nothing in it needs to start at zero (every slot is written before it is read), but two calls
 *     whose kernels overlap on the GPU (different streams, no ordering) race on it: serialise them.
 */
size_t clb_convtree_bwd_w_noalloc_max_bytes(void);
int clb_convtree_bwd_w_noalloc(const void *gy, const void *x, const void *w, const int32_t *sel, const uint8_t *amax,
                               void *gw, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh,
                               int kw, int wmode, int dtype, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Stand-alone first gate level (ConvLogicLayer with complete=False).
 * Replace convlogic_cuda.convlogic_forward / convlogic_backward_x / convlogic_backward_weight
 * (convlogic.cpp:31-33; convlogic_kernel.cu:67-107, 322-359, 197-247).
 *   y, gy [N,C,Ho,Wo,4]   w, gw [C,4,16].  Backward-x uses the same group tables as above.
 */
int clb_conv_fwd(const void *x, const void *w, const int32_t *sel, void *y, int N, int Ci, int H, int W, int C,
                 int sh, int sw, int ph, int pw, int kh, int kw, int wmode, int dtype, void *stream);
int clb_conv_bwd_x(const void *gy, const void *x, const void *w, const int32_t *sel, void *gx,
                   const int32_t *grp_start, const int32_t *grp_list, int cg, int nb, int N, int Ci, int H, int W,
                   int C, int sh, int sw, int ph, int pw, int kh, int kw, int wmode, int dtype, void *stream);
size_t clb_conv_bwd_w_scratch_bytes(int N, int C, int Ho, int Wo, int dtype);
int clb_conv_bwd_w(const void *gy, const void *x, const void *w, const int32_t *sel, void *gw, void *scratch,
                   size_t scratch_bytes, int N, int Ci, int H, int W, int C, int sh, int sw, int ph, int pw, int kh,
                   int kw, int wmode, int dtype, void *stream);

/* ------------------------------------------------------------------------------------------------
 * One pairwise gate level on the trailing dimension (TreeLogicLayer).
 * Replace convlogic_cuda.treelogic_forward / treelogic_backward_x / treelogic_backward_weight
 * (convlogic.cpp:35-37; treelogic_kernel.cu:46-86, 252-285, 160-205).
 *   x, gx [N,C,H,W,2X]   y, gy [N,C,H,W,X]   w, gw [C,X,16];  HW = H*W.  Any X >= 1.
 */
int clb_tree_fwd(const void *x, const void *w, void *y, int N, int C, int HW, int X, int wmode, int dtype,
                 void *stream);
int clb_tree_bwd_x(const void *gy, const void *x, const void *w, void *gx, int N, int C, int HW, int X, int wmode,
                   int dtype, void *stream);
size_t clb_tree_bwd_w_scratch_bytes(int N, int C, int HW, int X, int dtype);
int clb_tree_bwd_w(const void *gy, const void *x, const void *w, void *gw, void *scratch, size_t scratch_bytes,
                   int N, int C, int HW, int X, int wmode, int dtype, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Flat LogicLayer on feature-major activations.
 * Replace difflogic_cuda.forward / backward_w / backward_x (src/difflogic/cuda/difflogic.cpp:17-19;
 * difflogic_kernel.cu:89-126, 128-173, 232-269).
 *   x, gx [in,B]   y, gy [out,B]   a, b int64 [out]   w, gw [out,16]
 *   start int64 [in+1], consumers int64 [2*out]: for input feature i the neurons reading it
 *   (the reference's given_x_indices_of_y_start / given_x_indices_of_y).  Any batch size.
 */
int clb_logic_fwd(const void *x, const int64_t *a, const int64_t *b, const void *w, void *y, int64_t in_dim,
                  int64_t out_dim, int64_t B, int wmode, int dtype, void *stream);
int clb_logic_bwd_w(const void *x, const int64_t *a, const int64_t *b, const void *w, const void *gy, void *gw,
                    int64_t in_dim, int64_t out_dim, int64_t B, int wmode, int dtype, void *stream);
int clb_logic_bwd_x(const void *x, const int64_t *a, const int64_t *b, const void *w, const void *gy, void *gx,
                    const int64_t *start, const int64_t *consumers, int64_t in_dim, int64_t out_dim, int64_t B,
                    int wmode, int dtype, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Packed (discretised) inference.  A packed tensor is [rows, words] of `bits`-wide integers
 * (bits in {8,16,32,64}); sample bits*word + i sits in bit i (LSB first), pad bits are zero.
 */
/* Replaces difflogic_cuda.tensor_packbits_cuda (difflogic.cpp:21; difflogic_kernel.cu:335-413).
 * t bool/uint8 [F,B] (non-zero = 1) -> packed [F, ceil(B/bits)]. */
int clb_pack_bits(const uint8_t *t, void *packed, int64_t F, int64_t B, int bits, void *stream);
/* Same, for image batches: t [N, F] sample-major (e.g. a [N,C,H,W] tensor, F = C*H*W) -> packed
 * [F, ceil(N/bits)], i.e. the transpose and the packing in one pass. */
int clb_pack_bits_nmajor(const uint8_t *t, void *packed, int64_t N, int64_t F, int bits, void *stream);
/* Replaces difflogic_cuda.eval (difflogic.cpp:20; difflogic_kernel.cu:272-329).
 * x [in,words], ops uint8 [out] gate ids 0..15 -> y [out,words]. */
int clb_packed_logic(const void *x, const int64_t *a, const int64_t *b, const uint8_t *ops, void *y,
                     int64_t in_dim, int64_t out_dim, int64_t words, int bits, void *stream);
/* Replaces difflogic_cuda.groupbitsum (difflogic.cpp:22-33; difflogic_kernel.cu:418-482).
 * x [F,words] -> counts int32 [B,k], B = words*bits - pad_len; F must be divisible by k
 * (CLB_ERR_SHAPE otherwise, the reference's ValueError). */
int clb_group_popcount(const void *x, int32_t *counts, int64_t F, int64_t words, int bits, int pad_len, int k,
                       void *stream);
/* Packed fused ConvLogic block: bitwise 7-gate tree and OR-pool.  The reference declares such a
 * path (src/convlogic/convlogic_layer.py:357-372, forward_cuda_eval) but never implemented it; it is
 * defined here by the eval-mode float block on {0,1} inputs.
 * x [Ci,H,W,words]  ops uint8 [C,7]  ->  y [C,Ho/2,Wo/2,words]. */
int clb_packed_convtree(const void *x, const uint8_t *ops, const int32_t *sel, void *y, int Ci, int H, int W,
                        int C, int sh, int sw, int ph, int pw, int kh, int kw, int64_t words, int bits,
                        void *stream);

/* Two or three consecutive packed flat layers in one pass (no counterpart in the reference, which runs
 * difflogic_cuda.eval once per layer): neuron j of the LAST layer as a gate tree over 2^levels rows of the FIRST
 * layer's input.  leaf int32 [out][2^levels]: input rows in tree order (first-level gate p reads leaves 2p, 2p+1);
 * ops uint8 [out][2^levels - 1]: gate ids level by level, first level first, root last.  Rows of 8-byte multiples
 * only (CLB_ERR_SHAPE otherwise).  Worth it when every output of a layer is read about once by the next one. */
int clb_packed_tree(const void *x, const int32_t *leaf, const uint8_t *ops, void *y, int64_t in_dim, int64_t out_dim,
                    int levels, int64_t words, int bits, void *stream);

/* Fused input stage of packed inference: thermometer encoding + bit packing.  Replaces the reference's
 * host-side transform `cat([(x > t) for t in thresholds], dim=0)` (src/convlogic/data.py:46-50, thresholds
 * from :52-71) followed by PackBitsTensor (src/difflogic/packbitstensor.py:12-21) on the device, without the
 * [N, levels*channels, H, W] byte tensor in between.
 * pixels [N, channels, HW]: float32 (pixels_u8 == 0) or uint8 (pixels_u8 != 0; compared as v / 255.0f, as
 * torchvision's ToTensor produces them).  thresholds: `levels` floats on the device.
 * packed: feature (i*channels + c, yx) holds pixel[n, c, yx] > thresholds[i], sample n in bit n % 64 of
 * 64-bit word n / 64; bits beyond N are zero.  `words`: 64-bit words per row, ceil(N/64) (0 means that) or one
 * more to make the count even.  to_slab == 0: rows layout [levels*channels*HW, words]; to_slab != 0: slab layout
 * [levels*channels, U, HW] of 16-byte units, U = words / 2 (CLB_ERR_SHAPE when words is odd). */
int clb_thermometer_pack(const void *pixels, int pixels_u8, const float *thresholds, int levels, void *packed,
                         int64_t N, int64_t channels, int64_t HW, int64_t words, int to_slab, void *stream);

/* The same block on the SLAB layout [C][U][H][W] of 16-byte units (U = words / 2 for 64-bit words; one unit
 * = 128 samples), in which the image of one (channel, sample slab) is contiguous and can be staged in shared
 * memory.  Stride 1, at most 256 pooled outputs per image (CLB_ERR_SHAPE otherwise: use the rows layout).
 * x [Ci,U,H,W] units -> y [C,U,Ho/2,Wo/2] units.  clb_packed_layout converts between rows [C*HW, 2U words]
 * and slab [C,U,HW] (to_slab != 0: src is rows; else src is slab).  `scratch`: device memory of
 * clb_packed_convtree_slab_scratch_bytes(C) bytes, 16-byte aligned, holding the per-channel tap records the
 * call derives from `sel` and `ops`.  No counterpart in the reference. */
int clb_packed_layout(const void *src, void *dst, int64_t C, int64_t HW, int64_t U, int to_slab, void *stream);
int64_t clb_packed_convtree_slab_scratch_bytes(int C);
int clb_packed_convtree_slab(const void *x, const uint8_t *ops, const int32_t *sel, void *y, void *scratch, int Ci,
                             int H, int W, int C, int sh, int sw, int ph, int pw, int kh, int kw, int64_t U,
                             void *stream);

/* Three consecutive flat layers as one differentiable gate tree per neuron of the last layer (no counterpart in
 * the reference, which calls difflogic_cuda.forward / backward_w / backward_x once per layer).  Valid when every
 * output of a layer is read at most once by the next one (layer widths halving with `randperm(2*out) % in`
 * connections).  leaf int32 [T][8]: rows of the first layer's feature-major input x [in, B] in tree order; node
 * int32 [T][7]: the neuron at each tree position (4 of the first layer, 2 of the second, 1 of the third); w0/w1/w2:
 * the three layers' gate tensors [out_l][16] (wmode as elsewhere).  y [T][B].
 * Backward: tapgrad is scratch of T*8*B floats; gw0/gw1/gw2 [out_l][16] must be zero on entry (neurons no tree
 * uses keep zero); gx [in][B] may be NULL; start int64 [in+1], list int32 [T*8]: leaf slots t*8+k grouped by the
 * feature they read, in increasing slot order.  Fixed summation order. */
int clb_logic_tree_fwd(const float *x, const int32_t *leaf, const int32_t *node, const float *w0, const float *w1,
                       const float *w2, float *y, int64_t T, int64_t B, int wmode, void *stream);
int clb_logic_tree_bwd(const float *x, const int32_t *leaf, const int32_t *node, const float *w0, const float *w1,
                       const float *w2, const float *gy, float *tapgrad, float *gw0, float *gw1, float *gw2,
                       float *gx, const int64_t *start, const int32_t *list, int64_t in_dim, int64_t T, int64_t B,
                       int wmode, void *stream);
/* The forward of a training step whose trees feed GroupSum(k, tau) + mean cross-entropy (src/convlogic/model.py:137-152 on
 * top of src/difflogic/difflogic.py:203-208): the trees' outputs are added into their class sums as they are produced -- the
 * activation y [T][B] is not written -- and the head finishes as in clb_group_sum_ce: loss (one float), dscore [B][k].
 * labels int64 [B].  CLB_ERR_SHAPE for shapes it does not take (B > 512 or not a multiple of 4, k > 32, T % k != 0): run
 * clb_logic_tree_fwd + clb_group_sum_ce there.  scratch: clb_logic_tree_fwd_ce_scratch_bytes(T, B, k). */
size_t clb_logic_tree_fwd_ce_scratch_bytes(int64_t T, int64_t B, int k);
int clb_logic_tree_fwd_ce(const float *x, const int32_t *leaf, const int32_t *node, const float *w0, const float *w1,
                          const float *w2, const int64_t *labels, float *dscore, float *loss, void *scratch, size_t scratch_bytes,
                          int64_t T, int64_t B, int k, double tau, int wmode, void *stream);
/* The same backward when the trees feed GroupSum + cross-entropy (clb_group_sum_ce): instead of the gradient tensor
 * gy [T][B] it takes that head's dscore [B][k], the scalar gradient that reaches the loss (`scale`, one float on the
 * device) and tau; tree t belongs to class t / (T / k) and gy[t][b] = dscore[b][class] / (tau / scale), the values
 * clb_group_sum_bwd_scaled would write -- bit for bit -- without the tensor being written or read. */
int clb_logic_tree_bwd_scores(const float *x, const int32_t *leaf, const int32_t *node, const float *w0, const float *w1,
                              const float *w2, const float *dscore, const float *scale, int k, double tau, float *tapgrad,
                              float *gw0, float *gw1, float *gw2, float *gx, const int64_t *start, const int32_t *list,
                              int64_t in_dim, int64_t T, int64_t B, int wmode, void *stream);

/* GroupSum on float activations (src/difflogic/difflogic.py:203-208: `x.reshape(..., k, F/k).sum(-1) / tau`), taken
 * directly from the feature-major [F, B] output of clb_logic_fwd: out [B, k] = sum over the class's F/k rows / tau.
 * scratch: clb_group_sum_scratch_bytes(F, B, k, dtype) bytes.  Fixed summation order.  clb_group_sum_bwd is its
 * gradient: gy [F, B] = gout [B, k][class of f] / tau.  CLB_ERR_SHAPE when F % k != 0 (the reference asserts). */
size_t clb_group_sum_scratch_bytes(int64_t F, int64_t B, int k, int dtype);
int clb_group_sum_fwd(const void *y, void *out, void *scratch, size_t scratch_bytes, int64_t F, int64_t B, int k,
                      double tau, int dtype, void *stream);
int clb_group_sum_bwd(const void *gout, void *gy, int64_t F, int64_t B, int k, double tau, int dtype, void *stream);
/* The same with every value multiplied by *scale, a one-element device array of the gradient's dtype (the upstream
 * gradient of a scalar loss); scale may be NULL. */
int clb_group_sum_bwd_scaled(const void *gout, const void *scale, void *gy, int64_t F, int64_t B, int k, double tau, int dtype,
                             void *stream);

/* GroupSum followed by the mean cross-entropy loss, forward and the gradient w.r.t. the scores in one pass; stands in for
 * GroupSum.forward (src/difflogic/difflogic.py:203-208) + torch.nn.CrossEntropyLoss as the training step applies them
 * (src/convlogic/model.py:137-152).  y feature-major [F, B] fp32, labels int64 [B];
 * scores [B, k] (may be NULL) = class sums / tau, dscore [B, k] = (softmax(scores) - one_hot(labels)) / B, loss [1].
 * scratch as for clb_group_sum_fwd.  k <= 32.  Feed dscore (times the upstream scalar) to clb_group_sum_bwd. */
int clb_group_sum_ce(const float *y, const int64_t *labels, float *scores, float *dscore, float *loss, void *scratch,
                     size_t scratch_bytes, int64_t F, int64_t B, int k, double tau, void *stream);

/* out [cols][rows] = transpose of in [rows][cols], fp32, out != in.  The copy between the [batch][features] tensors of
 * the conv blocks / the caller and the feature-major [features][batch] activations of the flat layers (the reference
 * keeps [batch][features] and transposes inside its kernels' indexing, difflogic_kernel.cu:60-93).  rows <= 2 097 120. */
int clb_transpose_f32(const float *in, float *out, int64_t rows, int64_t cols, void *stream);

/* One Adam / AdamW step over a flat fp32 parameter buffer (all gate logits of a model in one array, their gradients in
 * another); stands in for torch.optim.AdamW as configured at src/convlogic/model.py:179-180.  step counts from 1;
 * decoupled != 0: AdamW (p *= 1 - lr * weight_decay), else the weight decay is added to the gradient.  All four arrays
 * 16-byte aligned.  m and v are the running moments (zero before the first step). */
int clb_adam_step(float *p, const float *g, float *m, float *v, int64_t n, double lr, double beta1, double beta2, double eps,
                  double weight_decay, int64_t step, int decoupled, void *stream);

/* ---- Compiled network -----------------------------------------------------------------------------------
 * A discretised stack (fused ConvLogic blocks, then flat LogicLayers, then GroupSum) serialised into one blob
 * and run with one call that enqueues the packed kernels above back to back.  It takes the place of the
 * reference's CompiledLogicNet (src/difflogic/compiled_model.py:41-361: C source generated per network,
 * compiled with gcc, run on the CPU, flat layers only): the artefact is the blob (written by
 * convlogic_b200.CompiledLogicNet.save, layout in csrc/net.cu), the code is this library, and fused conv
 * blocks are included.
 *   clb_net_device_bytes   validates a blob and returns the device memory the parameters need.
 *   clb_net_create         copies the parameters into caller-provided device memory (16-byte aligned, one
 *                          asynchronous copy on `stream`; `blob` must stay valid until it has run) and returns
 *                          a host-side handle; clb_net_destroy frees the handle (never the device memory).
 *   clb_net_workspace_bytes  device workspace for a batch (two activation buffers of the widest layer with the
 *                          batch padded to 128 samples, plus kernel scratch); 256-byte aligned.
 *   clb_net_forward        input_kind 0: bool / uint8 bits [batch][in_features] (what the reference's
 *                          `apply_logic_gate_net(bool const *inp, int *out, size_t len)` takes, compiled_model.py:
 *                          243-330); 1 / 2: float32 / uint8 pixels [batch][in_channels/levels][H*W] with
 *                          `levels` device thresholds (clb_thermometer_pack); 3: packed rows [in_features]
 *                          [2*ceil(batch/128)] of 64-bit words.  counts: int32 [batch][num_classes], as
 *                          clb_group_popcount.  Nothing is allocated and nothing synchronises. */
typedef struct clb_net clb_net;
int clb_net_device_bytes(const void *blob, size_t bytes, size_t *device_bytes);
int clb_net_create(const void *blob, size_t bytes, void *device_mem, void *stream, clb_net **net);
void clb_net_destroy(clb_net *net);
int clb_net_info(const clb_net *net, int64_t *in_features, int *num_classes, int *n_layers);
size_t clb_net_workspace_bytes(const clb_net *net, int64_t batch);
int clb_net_forward(const clb_net *net, int input_kind, const void *input, const float *thresholds, int levels,
                    int64_t batch, int32_t *counts, void *workspace, size_t workspace_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* CONVLOGIC_B200_H */
