/*
 * fovi_b200 — C ABI of the B200 (sm_100a) foveated hot path: the sensor's grid sample and
 * the KNNConv layers that consume it.
 *
 * The reference (nblauch/fovi) is pure Python and has no FFI; its extension points for this
 * path are the Python classes cited at each entry point below.  Every function here is what a
 * binding for that class calls.  Conventions:
 *   - all image/activation/weight/output buffers are caller-owned DEVICE pointers;
 *     tables given to *_plan_create are HOST pointers and are copied;
 *   - work is enqueued on the caller's stream (a cudaStream_t passed as void*); nothing
 *     synchronises the device except the *_plan_create functions;
 *   - every function returns a status (0 = FOVI_OK); nothing throws, traps or aborts;
 *   - a plan may be used from several host threads on distinct streams
 *     (fovi_knnconv_forward keeps a small per-plan status word that concurrent calls share).
 */
#ifndef FOVI_B200_H
#define FOVI_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  FOVI_OK = 0,
  FOVI_ERR_INVALID_ARGUMENT = 1, /* null pointer, bad enum, negative size                      */
  FOVI_ERR_UNSUPPORTED = 2,      /* shape/dtype/layout combination the kernels do not cover    */
  FOVI_ERR_TABLE_RANGE = 3,      /* neighbour index outside [0, n_in] or tap outside [0, V)    */
  FOVI_ERR_CUDA = 4,             /* a CUDA runtime/driver call failed (fovi_last_cuda_error)   */
  FOVI_ERR_ALIGNMENT = 5,        /* pointer or stride not aligned as documented                */
  FOVI_ERR_DEVICE_TIMEOUT = 6,   /* a bounded in-kernel wait gave up (reported by *_check)     */
  FOVI_ERR_NO_DEVICE = 7         /* no sm_100 device is current                                */
} fovi_status;

typedef enum { FOVI_F32 = 0, FOVI_BF16 = 1, FOVI_U8 = 2 /* sampler images only */ } fovi_dtype;
typedef enum { FOVI_NEAREST = 0, FOVI_BILINEAR = 1 } fovi_sample_mode;
typedef enum { FOVI_PAD_ZEROS = 0, FOVI_PAD_BORDER = 1 } fovi_pad_mode;

/* Output layouts of the sampler.  B images, F fixations, C channels, N sensor points.       */
typedef enum {
  FOVI_OUT_BFCN = 0, /* [B,F,C,N]  what policies.py:277 stacks                                */
  FOVI_OUT_FBCN = 1, /* [F,B,C,N]  the '(f b) c n' flattening of fovinet.py:281               */
  FOVI_OUT_BFNC = 2, /* [B,F,N,Cp] points-major, channels last, Cp = out_channel_stride >= C,
                        channels C..Cp-1 written as 0: the KNNConv kernels' input layout      */
  FOVI_OUT_FBNC = 3, /* [F,B,N,Cp]                                                            */
  FOVI_OUT_FB_PAIRS = 4, /* [ceil(F*B/128), ceil(N/2), 128, 2, 4]: tiles of 128 image x fixation rows
                            (row = f*B + b) outermost, then point pairs, then the rows of the tile,
                            then the two points of the pair with 4 channels each (channels C..3 and
                            an odd last point are written as 0; rows past F*B are not written);
                            bf16, C <= 4.  The input layout of a KNNConv plan with c_in <= 4
                            (FOVI_X_PAIRS).                                                     */
  FOVI_OUT_BF_PAIRS = 5  /* same with row = b*F + f                                            */
} fovi_sample_layout;

/* Input layout the tensor-core path of a KNNConv plan expects (fovi_knnconv_x_layout). */
typedef enum {
  FOVI_X_BNC = 0,  /* [B, n_in, cin_packed] bf16, channels last                                */
  FOVI_X_PAIRS = 1 /* [ceil(B/128), ceil(n_in/2), 128, 2, 4] bf16 (see FOVI_OUT_FB_PAIRS); chosen when
                      c_in <= 4: a run of consecutive point pairs of one 128-row batch tile is one
                      contiguous block of 2 KB per pair; values must be finite                  */
} fovi_x_layout;

/* Activation layouts of KNNConv. */
typedef enum {
  FOVI_ACT_BCN = 0, /* [B,C,N] points last — the reference's layout (knn.py:538-557)          */
  FOVI_ACT_BNC = 1  /* [B,N,C] channels last                                                   */
} fovi_act_layout;

const char* fovi_status_string(int status);
/* Text of the last CUDA error seen by this library on the calling thread ("" if none). */
const char* fovi_last_cuda_error(void);
/* Library version, "major.minor". */
const char* fovi_version(void);

/* ------------------------------------------------------------------------------------------
 * Sensor sampler.
 * Replaces GridSampler (fovi/sensing/samplers.py:51-130): its constructor's
 * `sampling_grid` (samplers.py:87) is what the plan is built from, and its forward
 * (samplers.py:91-112: transform_sampling_grid, coords.py:590-642, then F.grid_sample with
 * align_corners=False) is fovi_sample_forward — for all F fixations of every image in one
 * launch instead of the per-fixation Python loop of policies.py:266-277.
 * ------------------------------------------------------------------------------------------ */
typedef struct fovi_sampler_plan fovi_sampler_plan;

/* grid_xy: HOST [N,2] float32, the rows of GridSampler.sampling_grid[0,0] — (x, -y) of the
 * sensor's cartesian coordinates in [-1,1].  The plan keeps sorted copies on the current
 * device (points are visited in image order; results are written at their original index).
 * Synchronises the device. */
int fovi_sampler_plan_create(const float* grid_xy, int n_points, fovi_sampler_plan** out);
void fovi_sampler_plan_destroy(fovi_sampler_plan* plan);
int fovi_sampler_plan_num_points(const fovi_sampler_plan* plan);

/* img        : [B,C,H,W] elements of `dtype`, element strides img_strides[4] (any NCHW or
 *              NHWC-strided view; no overlap).  FOVI_U8 images (what a data loader hands over before
 *              its float conversion) are sampled as the float32 values 0..255 they hold, i.e. the
 *              result is the reference's on img.float(); a quarter of the float32 bytes cross PCIe.
 * fix_rc     : DEVICE [B,F,2] float32, normalised fixation centre (row, col)
 *              — RetinalTransform._check_fix_loc, retina.py:211-237.
 * fix_hw     : DEVICE [B,F,2] float32, fixation size in pixels (height, width)
 *              — RetinalTransform._check_fixation_size, retina.py:176-209.
 * out        : `out_dtype` elements in `layout`; out_channel_stride is Cp for the *NC layouts
 *              (ignored otherwise).
 * Arithmetic is float32 in the reference's operation order; with float32 in and out the result
 * equals the reference's CPU result bit for bit. */
int fovi_sample_forward(const fovi_sampler_plan* plan, const void* img, int dtype, int B, int C, int H, int W,
                        const int64_t* img_strides, const float* fix_rc, const float* fix_hw, int F, int mode,
                        int pad, void* out, int out_dtype, int layout, int out_channel_stride, void* stream);

/* Gradient of fovi_sample_forward with respect to the image: what autograd through F.grid_sample gives
 * the reference (samplers.py:108) when the images require grad.  grad_out: [B,F,C,N] (FOVI_OUT_BFCN) or
 * [F,B,C,N] (FOVI_OUT_FBCN) of go_dtype; grad_img: float32 contiguous [B,C,H,W], ACCUMULATED into with
 * atomic adds (zero it first for a plain gradient; the order of the additions is not fixed, so results
 * agree with the reference to float32 rounding, not bit for bit).  Fixations carry no gradient. */
int fovi_sample_backward(const fovi_sampler_plan* plan, const void* grad_out, int go_dtype, int layout, int B, int C, int H, int W,
                         const float* fix_rc, const float* fix_hw, int F, int mode, int pad, float* grad_img, void* stream);

/* Synchronises `stream` and returns FOVI_ERR_DEVICE_TIMEOUT if a sampler launch on this plan since the
 * last check gave up on the (bounded) wait for its asynchronous image copies; clears the word.  Such a
 * launch leaves its part of the output unwritten; nothing faults or hangs.  The reference has no
 * counterpart (F.grid_sample has no device-side waits). */
int fovi_sampler_check(fovi_sampler_plan* plan, void* stream);

/* ------------------------------------------------------------------------------------------
 * KNNConv.
 * Replaces KNNConvLayer.forward (fovi/arch/knn.py:538-557): zero-pad + gather of the K
 * neighbours (knn.py:484-503), the one-hot tap reassignment local_rf (knn.py:505-526) and the
 * shared linear map over Cin*V (knn.py:555), evaluated as
 *   out[b,n,o] = bias[o] + sum_k sum_c X[b, idx[k,n], c] * W[o, c*V + tap[n,k]]
 * with pad neighbours (idx == n_in) skipped.
 * Non-finite inputs: on the channels-last layout (FOVI_X_BNC) an Inf / NaN at an input point reaches exactly the outputs
 * whose neighbourhoods contain the point, as in the reference.  On the pair layout (FOVI_X_PAIRS, c_in <= 4) the two points
 * of a pair (2p, 2p+1) are multiplied together, the one that is not a neighbour by zero weights, so a non-finite value also
 * reaches the outputs whose neighbourhoods contain only the point's pair partner, and with a grouped plan the other output
 * points of the group (0 * Inf = NaN): pair-layout inputs (images) must be finite.
 * ------------------------------------------------------------------------------------------ */
typedef struct fovi_knnconv_plan fovi_knnconv_plan;

/* knn_idx_pad : HOST [K,n_out] int32 — KNNConvLayer.knn_indices_pad_token (knn.py:451-453),
 *               values in [0,n_in], n_in marks a pad neighbour.
 * tap         : HOST [n_out,K] uint16 — argmax over the last axis of the one-hot
 *               KNNConvLayer.local_rf [n_out,K,V] (knn.py:599-647).
 * Validates the ranges (FOVI_ERR_TABLE_RANGE), compacts pad entries away and uploads the
 * tables to the current device.  Synchronises the device. */
int fovi_knnconv_plan_create(const int32_t* knn_idx_pad, const uint16_t* tap, int n_in, int n_out, int K, int V,
                             int c_in, int c_out, fovi_knnconv_plan** out);
void fovi_knnconv_plan_destroy(fovi_knnconv_plan* plan);

/* Channel count of the packed bf16 operands: c_in rounded up to a multiple of 8 (kept when it
 * is a multiple of 64).  With FOVI_X_BNC, activations handed to the tensor-core path are
 * [B,n_in,cin_packed] bf16 with channels c_in..cin_packed-1 equal to 0. */
int fovi_knnconv_cin_packed(const fovi_knnconv_plan* plan);
/* FOVI_X_BNC or FOVI_X_PAIRS (c_in <= 4). */
int fovi_knnconv_x_layout(const fovi_knnconv_plan* plan);
/* 1 if fovi_knnconv_forward (tensor cores) covers this plan's shape: c_out a multiple of 16 and neighbour lists of
 * at most 256 entries; 0 otherwise (fovi_knnconv_forward_f32 covers every shape). */
int fovi_knnconv_tc_supported(const fovi_knnconv_plan* plan);
/* Number of non-pad (n,k) entries: algorithmic FLOPs per image = 2*c_in*c_out*nnz. */
int64_t fovi_knnconv_nnz(const fovi_knnconv_plan* plan);

/* Repack KNNConvLayer.weight ([c_out, c_in*V], c-major/v-minor, knn.py:462) for the kernels.
 * dst_dtype f32 (exact path) or bf16 with FOVI_X_BNC: V slabs [V, c_out, cin_packed], padded
 * channels zero.  dst_dtype bf16 with FOVI_X_PAIRS: per output point the slabs of its own
 * neighbour pairs, [n_out, pair_slots, c_out, 8] (the reference's local_rf applied to the weights,
 * knn.py:528-536, in bf16); slots or pair halves without a neighbour are zero.
 * W, dst: device pointers; size from fovi_knnconv_packed_weight_bytes. */
int fovi_knnconv_pack_weights(const fovi_knnconv_plan* plan, const void* W, int w_dtype, void* dst, int dst_dtype,
                              void* stream);
/* Bytes of the packed weight buffer for `dst_dtype`. */
int64_t fovi_knnconv_packed_weight_bytes(const fovi_knnconv_plan* plan, int dst_dtype);

/* Grouped first layer.  With c_in <= 4 the MMA's N axis holds only c_out (64-96) columns; G consecutive output points can
 * share one accumulator instead: create the plan for n_out/G "points" with G*c_out "channels", the neighbour list of
 * group g being the union of its members' lists (knn_idx_pad[k][g]) and tap[g][k] = k.  This call packs the weights for
 * such a plan: W is the layer's [c_out, c_in*V] weight, member_tap DEVICE uint16 [n_out/G, K, G] gives for union entry k
 * of group g the tap member j uses for it (0xFFFF: none).  The forward call is unchanged and its output
 * [B, n_out/G, G*c_out] is the layer's [B, n_out, c_out] as it stands.  No counterpart in the reference (its forward,
 * fovi/arch/knn.py:538-557, has no such tiling concern). */
int fovi_knnconv_pack_weights_grouped(const fovi_knnconv_plan* plan, const void* W, int w_dtype, const uint16_t* member_tap, int G,
                                      int V, void* dst, void* stream);

/* Convert activations [B,C,N] (x_dtype, contiguous) to a tensor-core input layout:
 * x_layout FOVI_X_BNC: [B,N,cp] bf16 with zero-filled pad channels (cp >= C, multiple of 8);
 * x_layout FOVI_X_PAIRS: [ceil(B/128),ceil(N/2),128,2,4] bf16 (C <= 4; cp ignored). */
int fovi_pack_points(const void* x, int x_dtype, int B, int C, int N, void* dst, int cp, int x_layout, void* stream);

/* Tensor-core path (tcgen05 MMA, bf16 operands, fp32 accumulation in tensor memory).
 * X    : bf16 in the plan's input layout (fovi_knnconv_x_layout), 16-byte aligned.
 * Wt   : packed bf16 weights from fovi_knnconv_pack_weights.
 * bias : [c_out] float32 or NULL.
 * Y    : [B,n_out,c_out] of y_dtype (bf16 or f32), 16-byte aligned; c_out % 8 == 0.
 * relu : apply max(.,0) after the bias.
 * Requires c_out % 16 == 0.  A bounded in-kernel wait that gives up makes the kernel store a
 * code readable with fovi_knnconv_check; the launch itself still returns FOVI_OK. */
int fovi_knnconv_forward(fovi_knnconv_plan* plan, const void* X, const void* Wt, const float* bias, void* Y,
                         int y_dtype, int B, int relu, void* stream);

/* Allocation-free variant of the tensor-core path for inputs in the reference's [B,c_in,n_in]
 * layout.  It has no counterpart in the reference (which leaves all memory to PyTorch's caching
 * allocator); it exists for callers that must not allocate device memory where they run the
 * layer — a real-time or serving loop with a budget fixed at start-up, a plug-in callback under a
 * host that owns the allocator — and for whom cudaMalloc's device-wide synchronisation is not
 * acceptable either.  The repacked activations are kept in a fixed array inside the library
 * (fovi_static_scratch_bytes(), 32 MiB, resident on every GPU that loads the library until exit)
 * instead of a buffer the caller would have to provide.  Larger batches are rejected with
 * FOVI_ERR_UNSUPPORTED and a message in fovi_last_cuda_error().  No cudaMalloc/cudaFree or other
 * allocating call is made.  The first call on a device resolves the array's device address
 * (cudaGetSymbolAddress); make that first call before any stream capture.  All calls on a device
 * share the array and it keeps the previous call's contents (the parts that must be zero are
 * cleared on every call): calls that overlap on the GPU race, so issue them on one stream.
 * X: [B,c_in,n_in] of x_dtype (f32 or bf16), contiguous; the other arguments as for
 * fovi_knnconv_forward. */
int64_t fovi_static_scratch_bytes(void);
int fovi_knnconv_forward_bcn_static(fovi_knnconv_plan* plan, const void* X, int x_dtype, const void* Wt,
                                    const float* bias, void* Y, int y_dtype, int B, int relu, void* stream);

/* Exact float32 path (CUDA cores, float32 multiply-adds): the fp32 parity case.
 * X : [B,c_in,n_in] (FOVI_ACT_BCN) or [B,n_in,c_in] (FOVI_ACT_BNC) of x_dtype; Wt: packed
 * f32 slabs [V,c_out,cin_packed]; Y: float32 in y_layout. */
int fovi_knnconv_forward_f32(const fovi_knnconv_plan* plan, const void* X, int x_dtype, int x_layout,
                             const float* Wt, const float* bias, float* Y, int y_layout, int B, int relu,
                             void* stream);

/* Tensor-core forward whose results are ADDED into rows of a float32 Y instead of stored: output point n of the plan adds
 * its [B, c_out] block into Y[:, out_map[n], :] (Y: [B, n_out_y, c_out] float32, initialised by the caller; out_map: device
 * int32 [n_out] with values in [0, n_out_y); no bias, no ReLU).  The additions are float32 reductions in L2, so their order --
 * and with it the last bits of Y -- may differ between runs.  This is the weight-gradient contraction of KNNConv
 * (fovi/arch/knn.py:538-557 under autograd): one "output point" per part of a filter tap's (output point, neighbour) list,
 * every part reduced into its tap (fovi_b200/grad.py), where the reference's autograd uses index_add-style scatter kernels. */
int fovi_knnconv_forward_scatter_add(fovi_knnconv_plan* plan, const void* X, const void* Wt, float* Y, int B, const int* out_map,
                                     int n_out_y, void* stream);

/* Diagnostic for the failure path: launches the plan's tensor-core kernel with every operand load withheld and a short
 * wait limit, so the kernel's first consumer waits run out.  Nothing faults or hangs: the kernel records the wait site,
 * all its roles leave, tensor memory is freed.  A following fovi_knnconv_check must return FOVI_ERR_DEVICE_TIMEOUT, and
 * the context must remain usable (the next fovi_knnconv_forward gives correct results).  Y's contents are unspecified.
 * The reference has no counterpart (it has no device-side waits). */
int fovi_knnconv_selftest_wait_timeout(fovi_knnconv_plan* plan, const void* X, const void* Wt, void* Y, int y_dtype, int B,
                                       void* stream);

/* Synchronises `stream` and returns FOVI_ERR_DEVICE_TIMEOUT if any tensor-core launch on this
 * plan since the last check gave up on a wait; clears the word. */
int fovi_knnconv_check(fovi_knnconv_plan* plan, void* stream);

/* Sensor -> first KNNConv in one call (the multi-fixation loop of policies.py:266-277 followed by the
 * first KNNConvLayer.forward of the backbone, knnalexnet.py:118-119): samples all F fixations straight
 * into the layout `conv` consumes, in `intermediate` (caller-owned device scratch of
 * fovi_fused_intermediate_bytes(conv, B*F) bytes), then runs the tensor-core layer.  For the two launches
 * the intermediate is held in L2 through the stream's access-policy window (persisting for the sampler's
 * writes, released by the convolution's reads), so the sensor output makes no round trip through HBM; the
 * window is cleared before the call returns.  row_order 0: output rows '(f b)' (fovi/fovinet.py:281),
 * 1: '(b f)'.  Requires the sampler's point count == conv's n_in and C == conv's c_in.  Other arguments as
 * for fovi_sample_forward / fovi_knnconv_forward. */
int64_t fovi_fused_intermediate_bytes(const fovi_knnconv_plan* conv, int rows);
int fovi_sample_knnconv_fused(const fovi_sampler_plan* sampler, fovi_knnconv_plan* conv, const void* img, int dtype, int B,
                              int C, int H, int W, const int64_t* img_strides, const float* fix_rc, const float* fix_hw,
                              int F, int mode, int pad, void* intermediate, const void* Wt, const float* bias, void* Y,
                              int y_dtype, int relu, int row_order, void* stream);

/* ------------------------------------------------------------------------------------------
 * Depthwise KNN convolution: out[b, c*g + j, n] = bias[c*g + j] + sum_k Xpad[b, c, idx[k,n]] * W[c, tap[n,k], j],
 * g = c_out / c_in.  Replaces KNNDepthwiseConvLayer.forward (fovi/arch/knn.py:847-872) and the depthwise half of
 * KNNDepthwiseSeparableConvLayer.forward (fovi/arch/knn.py:776-800).  `plan` is a fovi_knnconv_plan created with this
 * layer's tables and channel counts (c_out a multiple of c_in).  Wp: DEVICE float32 [V, c_out], Wp[v][c*g + j] = W[c][v][j].
 * X: [B,c_in,n_in] (FOVI_ACT_BCN) or [B,n_in,c_in] (FOVI_ACT_BNC); Y likewise with c_out, n_out.
 * ------------------------------------------------------------------------------------------ */
int fovi_knn_depthwise_forward(const fovi_knnconv_plan* plan, const void* X, int x_dtype, int x_layout, const float* Wp,
                               const float* bias, void* Y, int y_dtype, int y_layout, int B, int relu, void* stream);

/* Gradients of fovi_knn_depthwise_forward (autograd through fovi/arch/knn.py:847-872).  gY: the output gradient in
 * `y_layout` of g_dtype.  gX (may be NULL): float32 in X's layout, ACCUMULATED into (zero it first); needs Wp.
 * gWp (may be NULL): float32 [V, c_out] in Wp's layout, ACCUMULATED into; needs X.  float32 atomics: sums agree with
 * the reference to rounding.  The bias gradient is the plain sum of gY over rows and points. */
int fovi_knn_depthwise_backward(const fovi_knnconv_plan* plan, const void* X, int x_dtype, int x_layout, const float* Wp, const void* gY,
                                int g_dtype, int y_layout, int B, float* gX, float* gWp, void* stream);

/* ------------------------------------------------------------------------------------------
 * Backward pass of KNNConv.  The reference gets its gradients from autograd through gather, one-hot matmul and linear
 * (fovi/arch/knn.py:538-557).  Here both gradient contractions are run by fovi_knnconv_forward on derived plans (the
 * transposed layer for the input gradient; for the weight gradient the batch takes the place of the channels, see
 * fovi_b200/grad.py).  The one extra device routine is the layout change that puts the batch index innermost.
 *
 * src: logical [B, I, J] of `dtype`, element (b,i,j) at b*sb + i*si + j*sj (element strides; si == 1 or sj == 1).
 * dst: [I, Jp, Bp] bf16, fully written: zeros where j >= J or b >= B.
 * ------------------------------------------------------------------------------------------ */
int fovi_batch_to_inner(const void* src, int dtype, int B, int I, int J, long long sb, long long si, long long sj, void* dst, int Jp,
                        int Bp, void* stream);

/* fovi_batch_to_inner fused with the first steps of a layer's backward pass (fovi_b200/grad.py): `grad` is the upstream
 * gradient and `act` (may be NULL: no ReLU) the layer's output in the same layout and dtype; the gradient is zeroed where the
 * output is not positive (ReLU backward), written back in the source layout to `masked` (may be NULL), transposed to `dst`
 * like fovi_batch_to_inner, and summed over everything but the contiguous source index into colsum (float32, one entry per
 * value of that index: the bias gradient when the channels are contiguous; may be NULL; zeroed here).  Needs even extents and
 * strides (FOVI_ERR_UNSUPPORTED otherwise: use the separate calls). */
int fovi_relu_backward_to_inner(const void* grad, const void* act, int dtype, int B, int I, int J, long long sb, long long si,
                                long long sj, void* masked, void* dst, int Jp, int Bp, float* colsum, void* stream);

/* Bias gradient: dst[c] = sum over the R rows of the row-major [R, C] matrix src (bf16 or float32, C even), float32
 * accumulation; dst is overwritten.  (The reference: autograd of the bias add in F.linear, fovi/arch/knn.py:555.) */
int fovi_column_sum(const void* src, int dtype, long long R, int C, float* dst, void* stream);

/* Segment sums of the weight gradient of a layer with at most 4 input channels (fovi_b200/grad.py): prod is float32
 * [R][S][4] (row = output channel, slot = (output point, neighbour) pair, 4 channel products); the slots of filter tap v are
 * seg_slot[seg_start[v] .. seg_start[v+1]) (device int32 arrays, seg_start has V+1 entries).
 * dst[o*dst_pitch + 4*v + c] += sum of prod[o][slot][c] over the tap's slots.  No atomics: results are deterministic. */
int fovi_tap_segment_sum(const float* prod, int R, long long S, const int* seg_start, const int* seg_slot, int V, float* dst,
                         int dst_pitch, void* stream);


/* ------------------------------------------------------------------------------------------
 * Table construction on the host, with a reproducible rule for ties.
 * Replaces the neighbour search _compute_euclidean_distances_batched + topk (fovi/arch/knn.py:101-152) and
 * compute_local_rf (fovi/arch/knn.py:599-647).  The reference's float32 library calls rank the (frequent) exact and
 * near ties of a ring-symmetric sensor differently from machine to machine; here distances are evaluated in double
 * precision from the float32 coordinates with correctly rounded operations in a fixed order and ties go to the lower
 * index, so the tables are a function of the coordinates alone.  All pointers are HOST memory; no device is needed.
 * ------------------------------------------------------------------------------------------ */

/* ---- Sensor geometry on the host (no device needed): fovi/sensing/coords.py:204-370 (ring radii evenly spaced in
 * log(r + a), angles per ring for isotropic spacing), :68-87 (pad rings outside the field of view) and
 * fovi/sensing/manifold.py:32-48, 139-170 (cortical manifold: rho = M(r) sin(r) 180/pi, z = integral of sqrt(M^2 - rho'^2)).
 * Same formulas and rounding points as the reference (float32 ring radii, double elsewhere) on the C library's functions:
 * identical point counts, coordinates within a few units in the last float32 place of the reference's (3e-7 for the
 * normalised cartesian coordinates, 4e-6 for the cortical ones on the recorded sensors). */
/* Normalised ring radii (float32 [res], fov/2 -> 1) and angles per ring (int [res]); either may be NULL.
 * Returns the total number of sample points, or minus a FOVI_ERR_* code. */
long long fovi_sensor_ring_layout(double fov, double cmf_a, int res, float* radius, int* counts);
/* The n_points (= fovi_sensor_ring_layout's result) sample points, ring by ring: cartesian [n,2] (x, y in [-max_val, max_val]),
 * polar [n,2] (radius, angle), cortical [n,3], all double. */
int fovi_sensor_points(double fov, double cmf_a, int res, double max_val, long long n_points, double* cartesian, double* polar,
                       double* cortical);
/* Pad rings continuing outward at the last ring spacing for `padding_distance` (0.5 in the reference), sampled at the same
 * spacing in angle: cartesian [n,2] and cortical [n,3], float32, `capacity` points of room.  Returns the number of pad points
 * (with both outputs NULL: only that), or minus a FOVI_ERR_* code. */
long long fovi_sensor_pad_points(double fov, double cmf_a, int res, double max_val, double padding_distance, long long capacity,
                                 float* cartesian_pad, float* cortical_pad);

/* pts [n_pts,dim]: the layer's input points followed by its pad ring (cortical or visual-field coordinates);
 * targets [n_out,dim]: the output points.  idx_out [K,n_out]: the K nearest points of each target, nearest first
 * (order: distance, then index); dist_out [K,n_out] (may be NULL): their distances. */
int fovi_knn_table_build(const float* pts, int n_pts, int dim, const float* targets, int n_out, int K, int32_t* idx_out,
                         float* dist_out);

/* knn_idx [K,n_out] indexes pts (pad ring included).  sample_cortex != 0: each neighbour is placed at (distance to the
 * output point in `pts`/`out_pts` coordinates, direction in the visual field `pts_cart`/`out_cart` [.,2]); == 0: at its
 * own coordinates (dim == 2).  The neighbourhood is min-max normalised to [-1,1]^2 and each neighbour takes the nearest
 * node of the side x side reference frame (node order x-major, ties to the lower node).
 * tap_out [n_out,K]; nb_out [K,n_out,2] (may be NULL): the normalised neighbour coordinates. */
int fovi_tap_table_build(const int32_t* knn_idx, int K, int n_out, const float* pts, int n_pts, int dim, const float* pts_cart,
                         const float* out_pts, const float* out_cart, int side, int sample_cortex, uint16_t* tap_out, float* nb_out);

/* ------------------------------------------------------------------------------------------
 * KNN pooling.
 * Replaces KNNPoolingLayer.forward (fovi/arch/knn.py:345-394) for the modes 'max', 'avg', 'sum' and
 * 'gaussian': reduction over the K neighbours of each output point, pad neighbours (and NaN inputs)
 * ignored.
 * ------------------------------------------------------------------------------------------ */
typedef struct fovi_knnpool_plan fovi_knnpool_plan;
typedef enum { FOVI_POOL_MAX = 0, FOVI_POOL_AVG = 1, FOVI_POOL_SUM = 2, FOVI_POOL_WEIGHTED = 3 } fovi_pool_mode;

/* knn_idx_pad: HOST [K,n_out] int32 — KNNPoolingLayer.knn_indices_pad_token (knn.py:316-319). */
int fovi_knnpool_plan_create(const int32_t* knn_idx_pad, int n_in, int n_out, int K, fovi_knnpool_plan** out);
void fovi_knnpool_plan_destroy(fovi_knnpool_plan* plan);
/* Neighbour weights of FOVI_POOL_WEIGHTED: w_kn HOST [K,n_out] float32 — KNNPoolingLayer.gaussian_weights
 * (knn.py:325-343).  The forward drops the weights of pad / NaN neighbours and renormalises the rest:
 * y = sum_k x_k w_k / (sum of valid w_k + 1e-8), knn.py:372-390.  Synchronises the device. */
int fovi_knnpool_set_weights(fovi_knnpool_plan* plan, const float* w_kn);
/* X: [B,C,n_in] (FOVI_ACT_BCN) or [B,n_in,C] (FOVI_ACT_BNC) of `dtype`; Y: same layout and dtype with n_out
 * points.  An output point without any valid neighbour gives -inf (max), NaN (avg), 0 (sum), as the reference. */
int fovi_knnpool_forward(const fovi_knnpool_plan* plan, const void* X, int dtype, int layout, int B, int C, int mode,
                         void* Y, void* stream);

/* Gradient of fovi_knnpool_forward with respect to X (autograd through the reference's gather and nan-aware reductions,
 * fovi/arch/knn.py:345-394): dX (float32, X's layout and shape, overwritten) receives from every output element its
 * upstream gradient gY, shared out to the neighbours it read -- sum: 1 each; avg: 1/count; gaussian: the renormalised
 * weight; max: all to the first neighbour in list order holding the maximum.  Float32 atomic adds: the last bits may vary. */
int fovi_knnpool_backward(const fovi_knnpool_plan* plan, const void* X, int x_dtype, const void* gY, int g_dtype, int layout, int B,
                          int C, int mode, float* dX, void* stream);

/* Number of kernels this library has launched from the calling process (all entry points). */
int64_t fovi_launch_count(void);

/* ------------------------------------------------------------------------------------------
 * Per-sample normalisation of KNN activations.
 * Replaces KNNChannelNorm / KNNCoordNorm / KNNLayerNorm / KNNGroupNorm .forward
 * (fovi/arch/norm.py:14-101: torch LayerNorm over [C], [N] or [C,N], GroupNorm over channel groups,
 * applied to [B,C,N]):  y = (x - mean) / sqrt(var + eps) * weight + bias  with the biased variance of
 *   FOVI_NORM_CHANNEL : the C channels of every (sample, point);        weight, bias [C]
 *   FOVI_NORM_COORD   : the N points of every (sample, channel);        weight, bias [N]
 *   FOVI_NORM_LAYER   : all C*N values of a sample;                     weight, bias [C,N]
 *   FOVI_NORM_GROUP   : N points x C/groups channels of every group;    weight, bias [C]
 * x, y: [B,C,N] (FOVI_ACT_BCN) or [B,N,C] (FOVI_ACT_BNC), same layout; weight / bias: DEVICE float32
 * or NULL; stats: DEVICE scratch of 2 * fovi_knn_norm_stat_groups(...) float32 (receives mean and
 * 1/std of every statistics group); relu: apply max(.,0) last.
 * ------------------------------------------------------------------------------------------ */
typedef enum { FOVI_NORM_CHANNEL = 0, FOVI_NORM_COORD = 1, FOVI_NORM_LAYER = 2, FOVI_NORM_GROUP = 3 } fovi_norm_mode;
int64_t fovi_knn_norm_stat_groups(int mode, int B, int C, int N, int groups);
int fovi_knn_norm_forward(const void* x, int x_dtype, int layout, int B, int C, int N, int mode, int groups, const float* weight,
                          const float* bias, float eps, int relu, float* stats, void* y, int y_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FOVI_B200_H */
