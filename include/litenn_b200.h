/*
 * litenn_b200 -- C ABI of the sm_100a device backend for the LiteNN op layer.
 *
 * Every entry point is plain C: device pointers cross the boundary as uint64_t,
 * sizes as int64_t/int, all tensors are contiguous row-major fp32 (images NCHW).
 * Every call returns 0 on success or a negative LNN_E_* code; the text of the
 * last failure on the calling thread is returned by lnn_last_error().
 * All op entry points only enqueue work on the device's single in-order stream
 * (the counterpart of LiteNN's in-order command queue, litenn/core/minicl/
 * api/OpenCL/OpenCL.py:349-351); lnn_d2h and lnn_sync are the blocking points.
 * The library is not re-entrant per device: one host thread drives a device.
 *
 * Citations "ref:" name the file:line of iperov/litenn that an entry replaces.
 */
#ifndef LITENN_B200_H
#define LITENN_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LNN_OK              0
#define LNN_E_INVALID      -1   /* bad argument (shape, null pointer, unknown op id)   */
#define LNN_E_CUDA         -2   /* a CUDA runtime/driver call failed                    */
#define LNN_E_NOMEM        -3   /* device allocation failed even after pool eviction    */
#define LNN_E_NOTINIT      -4   /* device not initialised with lnn_init                 */
#define LNN_E_UNSUPPORTED  -5   /* configuration outside what the kernels implement     */
#define LNN_E_NCCL         -6   /* NCCL missing or a collective failed                  */
#define LNN_E_TIMEOUT      -7   /* a bounded device-side wait expired (status word set) */

#define LNN_MAX_DEVICES 16
#define LNN_MAX_DIMS 6

/* ---- runtime: replaces litenn/core/minicl/{devices,CLDevice,CLBuffer}.py ------------ */

int lnn_version(void);
const char* lnn_last_error(void);

/* ref: minicl/devices.py:88-105 (get_all) */
int lnn_device_count(int* count);
/* ref: minicl/devices.py:107-143 (device name / global_mem_size) */
int lnn_device_info(int dev, char* name, int name_len, uint64_t* total_mem,
                    int* sm_count, int* cc_major, int* cc_minor);
/* ref: minicl/CLDevice.py:180-190 (context + in-order queue created on demand) */
int lnn_init(int dev);
/* ref: minicl/CLDevice.py:105-118 (_cleanup) */
int lnn_shutdown(int dev);
/* ref: minicl/CLDevice.py:120-165 (_mem_alloc: size-keyed pool, evict largest pooled and retry) */
int lnn_alloc(int dev, uint64_t bytes, uint64_t* ptr);
/* ref: minicl/CLDevice.py:167-178 (_mem_free: return buffer to the pool) */
int lnn_free(int dev, uint64_t ptr, uint64_t bytes);
/* ref: minicl/CLDevice.py:39-49 (memory counters) */
int lnn_mem_stats(int dev, uint64_t* allocated_bytes, uint64_t* pooled_bytes);
/* release every pooled (unused) buffer back to the driver */
int lnn_pool_trim(int dev);
/* ref: minicl/CLBuffer.py:78-80 (blocking write from host memory) */
int lnn_h2d(int dev, uint64_t dst, const void* src, uint64_t bytes);
/* ref: minicl/CLBuffer.py:99-115 (blocking read into host memory) */
int lnn_d2h(int dev, void* dst, uint64_t src, uint64_t bytes);
/* ref: minicl/CLBuffer.py:66-67 (same-device copy) */
int lnn_d2d(int dev, uint64_t dst, uint64_t src, uint64_t bytes);
/* ref: minicl/CLBuffer.py:83-96 (fill), initializer/Scalar.py */
int lnn_fill_f32(int dev, uint64_t dst, int64_t count, float value);
/* dst[i] = hash(i + seed) * (high - low) + low with the reference's counter-based PCG hash: the
 * same bits as its device-side initializer.  ref: initializer/RandomUniform.py:12-28,
 * CLKernelHelper.py:210-216 */
int lnn_init_uniform(int dev, uint64_t dst, int64_t count, uint32_t seed, float low, float high);
/* dst[i] = mean + sqrt(-2 log(rx)) * cos(2 PI ry) * stddev, (rx, ry) the 2-D PCG hash of
 * (i + seed, 1).  ref: initializer/RandomNormal.py:10-30, CLKernelHelper.py:218-233,250-253 */
int lnn_init_normal(int dev, uint64_t dst, int64_t count, uint32_t seed, float mean, float stddev);
/* ref: minicl/CLDevice.py:51-55 (wait = clFinish) */
int lnn_sync(int dev);
/* asynchronous copies on the device stream; host memory should come from lnn_host_alloc */
int lnn_h2d_async(int dev, uint64_t dst, const void* src, uint64_t bytes);
int lnn_d2h_async(int dev, void* dst, uint64_t src, uint64_t bytes);
/* Host->device copy on a second stream, so that the next batch uploads while the current one
 * computes.  The copy starts after `after_event` (an lnn_event recorded on the compute stream
 * after the last kernel that read `dst`; 0 = no dependency).  lnn_wait_prefetch makes the
 * compute stream wait for every prefetch issued so far.  The reference uploads with a
 * blocking write (minicl/CLBuffer.py:78-80). */
int lnn_h2d_prefetch(int dev, uint64_t dst, const void* src, uint64_t bytes, uint64_t after_event);
int lnn_wait_prefetch(int dev);
/* The mirror image for results: a device->host copy ordered after the work enqueued so far but
 * on its own stream, so that the next batch's kernels do not wait for it; the source buffer must
 * stay allocated until lnn_wait_readback (which blocks the host) returns.  `dst` should be
 * pinned (lnn_host_alloc).  ref: minicl/CLBuffer.py:99-115 is the blocking form */
int lnn_d2h_readback(int dev, void* dst, uint64_t src, uint64_t bytes);
int lnn_wait_readback(int dev);
int lnn_host_alloc(uint64_t bytes, void** ptr);   /* pinned host memory */
int lnn_host_free(void* ptr);
/* number of kernels this library has launched on the device since lnn_init */
int lnn_launch_count(int dev, uint64_t* count);
/* Read-and-clear the device status word that bounded waits in the tile kernels set when they
 * give up ({LNN_E_TIMEOUT, role, tile, step}).  While the word is set, later tile kernels return
 * at once, so their outputs are not results; lnn_sync and lnn_d2h read the word with the
 * synchronisation they perform anyway and return LNN_E_TIMEOUT (clearing it) when it is set.
 * The reference has no counterpart: an OpenCL kernel that waits forever hangs the queue. */
int lnn_device_status(int dev, int* status);
/* Test hook: writes the status word from the host, as if a wait had expired (no kernel runs). */
int lnn_debug_set_status(int dev, int code, int role, int tile, int step);
/* CUDA events on the device stream (for timing on the stream the kernels run on) */
int lnn_event_create(int dev, uint64_t* ev);
int lnn_event_record(int dev, uint64_t ev);
int lnn_event_elapsed_ms(int dev, uint64_t ev_start, uint64_t ev_stop, float* ms);
int lnn_event_destroy(int dev, uint64_t ev);
/* Optional per-kernel timing: while enabled, launches of the slots below are bracketed by
 * CUDA events on the device stream; lnn_profile_read synchronises, then returns how many
 * launches a slot saw and their summed device time, and clears the slot. */
enum { LNN_PROF_TC_GEMM = 0, LNN_PROF_TC_CONV = 1, LNN_PROF_TC_DW = 2, LNN_PROF_PREP = 3, LNN_PROF_FEWCH = 4,
       LNN_PROF_SLOTS = 5 };
int lnn_profile_enable(int dev, int on);
int lnn_profile_read(int dev, int slot, uint64_t* launches, float* total_ms);

/* ---- element-wise: replaces litenn/core/op/element_wise_op.py ------------------------ */

enum {
  LNN_EW_ABS = 0, LNN_EW_ADD_CONST, LNN_EW_CLIP, LNN_EW_COS, LNN_EW_EXP, LNN_EW_LEAKY_RELU,
  LNN_EW_LOG, LNN_EW_MUL_CONST, LNN_EW_RDIV_CONST, LNN_EW_RSUB_CONST, LNN_EW_RELU,
  LNN_EW_SIGMOID, LNN_EW_SIN, LNN_EW_SQRT, LNN_EW_SQUARE, LNN_EW_TANH, LNN_EW_COUNT
};
/* O (+)= f(I).  p0,p1: op constants (value / min,max / alpha); flag: clip preserve_gradient.
 * ref: op/element_wise_op.py:83-96 (forward template), :112-364 (bodies) */
int lnn_eltwise_fwd(int dev, int op, uint64_t O, uint64_t I, int64_t n,
                    float p0, float p1, int flag, int accumulate);
/* dI += g(I, O, dO).  ref: op/element_wise_op.py:98-110 */
int lnn_eltwise_bwd(int dev, int op, uint64_t dI, uint64_t I, uint64_t O, uint64_t dO,
                    int64_t n, float p0, float p1, int flag);

/* ---- broadcast binary: replaces litenn/core/op/dual_wise_op.py ----------------------- */

enum {
  LNN_BIN_ADD = 0, LNN_BIN_SUB, LNN_BIN_MUL, LNN_BIN_DIV, LNN_BIN_MAX, LNN_BIN_MIN,
  LNN_BIN_BCE, LNN_BIN_COUNT
};
/* O (+)= f(A,B) with numpy broadcasting.  rank <= LNN_MAX_DIMS; a_shape/b_shape are the
 * operands' shapes left-padded with 1 to `rank`; o_shape the broadcast result.
 * ref: op/dual_wise_op.py:132-151, info/InfoBroadcast.py:40-86 */
int lnn_binary_fwd(int dev, int op, uint64_t O, uint64_t A, uint64_t B, int rank,
                   const int64_t* o_shape, const int64_t* a_shape, const int64_t* b_shape,
                   int accumulate);
/* which = 0: dX += dA(A,B,O,dO) ; which = 1: dX += dB(A,B,O,dO).  dX has the OUTPUT shape
 * (the caller reduces it over the broadcast axes).  ref: op/dual_wise_op.py:153-191 */
int lnn_binary_bwd(int dev, int op, int which, uint64_t dX, uint64_t A, uint64_t B,
                   uint64_t O, uint64_t dO, int rank, const int64_t* o_shape,
                   const int64_t* a_shape, const int64_t* b_shape);
/* Softmax over the rows of X[rows, cols] and its gradient, one launch each: P = exp(X) / sum(exp(X))
 * with no max-subtraction and the row sum in the reference's halving-tree order (the values of its
 * exp, reduce_sum, div composition); dX += gradient of that composition.  cols <= 8192.
 * ref: op/element_wise_op.py:309-314, op/reduce.py:279-301, op/dual_wise_op.py:268-281 */
int lnn_softmax_fwd(int dev, uint64_t P, uint64_t X, int64_t rows, int64_t cols);
int lnn_softmax_bwd(int dev, uint64_t dX, uint64_t X, uint64_t dP, int64_t rows, int64_t cols);
/* Categorical cross-entropy of probabilities P[rows, cols] against targets T (one row per sample, or
 * a single row with t_row_stride = 0): L[r] = sum_j -T[r][j] * log(clip(P[r][j], 1e-7, 1 - 1e-7)),
 * and dP += its gradient for an upstream dL[rows].  One launch each.
 * ref: op/dual_wise_op.py:228-250, op/element_wise_op.py:133-176 (clip), :225-232 (log) */
int lnn_cce_fwd(int dev, uint64_t L, uint64_t P, uint64_t T, int64_t rows, int64_t cols, int64_t t_row_stride);
int lnn_cce_bwd(int dev, uint64_t dP, uint64_t P, uint64_t T, uint64_t dL, int64_t rows, int64_t cols,
                int64_t t_row_stride);
/* y (+)= leaky_relu(x*g + b, alpha) for x[N,C,HW], g,b[C]: the three reference kernels
 * mul, add, leaky_relu (separately rounded) in one pass.
 * ref: op/dual_wise_op.py:194-204,283-295 + op/element_wise_op.py:207-221 */
int lnn_scale_bias_lrelu(int dev, uint64_t y, uint64_t x, uint64_t g, uint64_t b,
                         int64_t n, int64_t c, int64_t hw, float alpha, int accumulate);

/* ---- pooling: replaces litenn/core/op/pool2D.py -------------------------------------- */

enum { LNN_POOL_AVG = 0, LNN_POOL_MAX = 1, LNN_POOL_MIN = 2 };
/* ref: op/pool2D.py:111-146 */
int lnn_pool2d_fwd(int dev, int mode, uint64_t O, uint64_t I, int64_t n, int64_t c,
                   int ih, int iw, int oh, int ow, int pool, int stride, int padl, int padt);
/* dZ = gradient of leaky_relu (act = 1) after the gradient of max_pool2D(2, 2) in one pass, written
 * (not added): Y = leaky_relu(Z) [n,c,ih,iw] is the pooling input, P [n,c,ih/2,iw/2] its output,
 * dP the gradient of P.  Same roundings as lnn_pool2d_bwd into a zero-filled tensor followed by
 * lnn_eltwise_bwd(leaky_relu) into another.  Needs even ih, iw % 4 == 0, 16-byte aligned Y / dZ;
 * LNN_E_UNSUPPORTED otherwise.  ref: op/pool2D.py:147-230 + op/element_wise_op.py:207-221 */
int lnn_pool2x2_lrelu_bwd(int dev, uint64_t dZ, uint64_t Y, uint64_t P, uint64_t dP, int64_t n,
                          int64_t c, int ih, int iw, float alpha, int act);
/* The same gradient without the full-resolution activation: IDX [n,c,ih/2,iw/2] bytes is the map
 * of winning window positions (0..3 row-major, 4 = none) that lnn_conv2d_fwd_packed writes beside
 * a pooled NCHW result.  T (optional, pooled size) receives the winner's gradient: its sum over
 * (n, h, w) is the bias gradient of the block, so no pass over a full-resolution tensor is needed
 * for it.  dZ bit-identical to lnn_pool2x2_lrelu_bwd.  Same shape / alignment rules.
 * ref: op/pool2D.py:147-230 + op/element_wise_op.py:207-221 */
int lnn_pool2x2_idx_lrelu_bwd(int dev, uint64_t dZ, uint64_t T, uint64_t IDX, uint64_t P, uint64_t dP,
                              int64_t n, int64_t c, int ih, int iw, float alpha, int act);
/* The same gradient written straight into the packed split-FP16 operand format (HI / LO as sized
 * by lnn_packed_bytes(n, c, ih, iw, 2)) that lnn_conv2d_dx_packed / _dw_packed read: no
 * full-resolution fp32 gradient, no largest-magnitude pass and no split pass over it.  T (pooled
 * size, required) receives the winners' gradients.  The copies equal lnn_nhwc_split of the dZ that
 * lnn_pool2x2_idx_lrelu_bwd writes, bit for bit.  Precision 2 only.
 * ref: op/pool2D.py:147-230 + op/element_wise_op.py:207-221 */
int lnn_pool2x2_idx_lrelu_bwd_packed(int dev, uint64_t HI, uint64_t LO, uint64_t T, uint64_t IDX,
                                     uint64_t P, uint64_t dP, int64_t n, int64_t c, int ih, int iw,
                                     float alpha, int act);
/* T [n,c,oh,ow] = the gradient that reaches the winner of each pooling window (the non-zero
 * elements of the dZ above, in pooled layout), from the pooled values P, their gradient dP and the
 * map IDX.  ref: op/pool2D.py:147-230 + op/element_wise_op.py:207-221 */
int lnn_pool2x2_winner_grad(int dev, uint64_t T, uint64_t IDX, uint64_t P, uint64_t dP, int64_t n,
                            int64_t c, int oh, int ow, float alpha, int act);
/* dI += ... ; ref: op/pool2D.py:147-230 (I and O are only read for max/min) */
int lnn_pool2d_bwd(int dev, int mode, uint64_t dI, uint64_t I, uint64_t dO, uint64_t O,
                   int64_t n, int64_t c, int ih, int iw, int oh, int ow,
                   int pool, int stride, int padl, int padt);

/* ---- reductions: replaces litenn/core/op/reduce.py ----------------------------------- */

enum { LNN_RED_SUM = 0, LNN_RED_MEAN = 1, LNN_RED_MAX = 2, LNN_RED_MIN = 3 };
/* Input viewed as [outer][r0][mid][r1][inner]; axes r0 and r1 are reduced (COLS = r0*r1,
 * column index r0_i*r1 + r1_i), output [outer][mid][inner].  The summation tree is the
 * reference's ceil-halving tree (column c pairs with c + ceil(n/2)), so results are
 * bit-identical to it.  O (+)= result.  Uses pooled scratch when one row is split.
 * ref: op/reduce.py:166-205,279-301, info/InfoReduction.py:25-50 */
int lnn_reduce(int dev, int op, uint64_t O, uint64_t I, int64_t outer, int64_t r0,
               int64_t mid, int64_t r1, int64_t inner, int accumulate);
/* No counterpart in the reference.  lnn_reduce for callers that must not allocate device
 * memory (a serving loop that cannot afford a cudaMalloc stall, a host application that owns
 * the whole GPU heap, a process that is already out of memory): same arguments, bit-identical
 * result, but the partial sums of split rows live in a fixed 1 MiB device array inside the
 * library (one copy per device, kept until exit).  Refuses with LNN_E_UNSUPPORTED when the
 * partials need more than 2^18 floats.  The first call on a device looks up the array's
 * address and should come before any stream capture; calls share the array, so calls made
 * to overlap on one GPU race. */
int lnn_reduce_noalloc(int dev, int op, uint64_t O, uint64_t I, int64_t outer, int64_t r0,
                       int64_t mid, int64_t r1, int64_t inner, int accumulate);
/* dI += broadcast(dO) [/COLS] (sum, mean) or dO at the first column equal to O (max, min).
 * ref: op/reduce.py:207-216,250-276 (ties: lowest column index wins) */
int lnn_reduce_bwd(int dev, int op, uint64_t dI, uint64_t I, uint64_t dO, uint64_t O,
                   int64_t outer, int64_t r0, int64_t mid, int64_t r1, int64_t inner);

/* ---- data movement: replaces op/transpose.py, op/slice.py ---------------------------- */

/* O[perm(i)] (+)= I[i]; in_shape has `rank` extents, axes the permutation (out axis k =
 * in axis axes[k]).  ref: op/transpose.py:60-103 */
int lnn_transpose(int dev, uint64_t O, uint64_t I, int rank, const int64_t* in_shape,
                  const int* axes, int accumulate);
/* O[o] (+)= I[begin + o*step] per axis (fwd) ; ref: op/slice.py:168-178 */
int lnn_slice_fwd(int dev, uint64_t O, uint64_t I, int rank, const int64_t* in_shape,
                  const int64_t* out_shape, const int64_t* begin, const int64_t* step,
                  int accumulate);
/* dI[begin + o*step] += dO[o] ; ref: op/slice.py:180-190 */
int lnn_slice_bwd(int dev, uint64_t dI, uint64_t dO, int rank, const int64_t* in_shape,
                  const int64_t* out_shape, const int64_t* begin, const int64_t* step);

/* ---- contractions (tcgen05 tile engine) ----------------------------------------------- */

/* `precision` of the contraction entries: every fp32 operand is split into two parts of 11
 * significant bits each and hi*hi + hi*lo + lo*hi is accumulated in fp32 on the tensor cores.
 *   2 = split FP16 (default of the host layer): x / s = hi + lo in fp16 with s an exact power of
 *       two taken from the operand's largest magnitude; fp32-level accuracy, tcgen05 kind::f16
 *   3 = split TF32: x = hi + lo in tf32; same accuracy at any magnitude, tcgen05 kind::tf32,
 *       twice the instructions and operand bytes of 2
 *   1 = plain TF32 (hi only), about 1e-3 relative */

/* C[b] (+)= op(A[b]) * op(B[b]) (+ bias[n]) for b < batch, row-major fp32.
 * trans_a = 0: A is [M,K]; 1: A is stored [K,M].  trans_b = 0: B is [K,N]; 1: stored [N,K].
 * bias may be 0.
 * ref: op/matmul.py:8-164 (forward), :64-72 (gradients = the transposed variants),
 *      module/Dense.py:44-48 (bias) */
int lnn_gemm_f32(int dev, uint64_t C, uint64_t A, uint64_t B, uint64_t bias,
                 int64_t batch, int64_t m, int64_t n, int64_t k,
                 int trans_a, int trans_b, int accumulate, int precision);

/* geometry shared by the three convolution entry points (NCHW / OIHW) */
typedef struct lnn_conv_geom {
  int n, ic, ih, iw;        /* input  [n, ic, ih, iw]   */
  int oc, kh, kw;           /* kernel [oc, ic, kh, kw]  */
  int oh, ow;               /* output [n, oc, oh, ow]   */
  int stride, dilation;
  int padl, padt;           /* left / top zero padding (right / bottom follow from oh, ow) */
} lnn_conv_geom;

/* act: 0 none, 1 leaky_relu(alpha) applied after the optional bias[oc].
 * Y (+)= conv2D(X, W) (+ bias).  ref: op/conv2D.py:9-44, op/unfold2D.py:84-111,
 * module/Conv2D.py:58-62 */
int lnn_conv2d_fwd(int dev, const lnn_conv_geom* g, uint64_t Y, uint64_t X, uint64_t W,
                   uint64_t bias, int act, float alpha, int accumulate, int precision);
/* Inference fusion: Y = max_pool2D(act(conv2D(X, W) + bias), 2, 2, 'same'), Y is
 * [n, oc, ceil(oh/2), ceil(ow/2)].  Same values as the three separate entries.
 * ref: op/conv2D.py:9-44 + op/element_wise_op.py:207-221 + op/pool2D.py:47-146 */
int lnn_conv2d_pool_fwd(int dev, const lnn_conv_geom* g, uint64_t Y, uint64_t X, uint64_t W,
                        uint64_t bias, int act, float alpha, int precision);
/* Operand format of the tensor-core convolution: channel-innermost copies hi and lo of an NCHW
 * activation, each [n][h][w][cp] with cp = c rounded up to 8 (pad channels zero).  precision 3 / 1:
 * fp32 elements, hi = tf32(x), lo = tf32(x - hi) (lo may be 0 for precision 1).  precision 2: fp16
 * elements of x / s, and the hi buffer ends with a 16-byte trailer that holds the fp32 bit pattern
 * of the tensor's largest magnitude, from which every consumer derives s.  lnn_packed_bytes gives
 * the two buffer sizes.  The reference has no such format: its conv2D materialises an im2col
 * buffer per call (op/conv2D.py:39-41, op/unfold2D.py:84-110); lnn_nhwc_split is the explicit
 * form of the pre-pass lnn_conv2d_fwd runs. */
int lnn_packed_bytes(int64_t n, int64_t c, int64_t h, int64_t w, int precision, uint64_t* hi_bytes,
                     uint64_t* lo_bytes);
int lnn_nhwc_split(int dev, uint64_t hi, uint64_t lo, uint64_t X, int n, int c, int h, int w,
                   int precision);
/* conv2D forward (+ bias, leaky_relu, optional max_pool2D(2,2,'same')) whose input and / or output
 * stay in that format, so that a chain of convolutions never writes or re-reads the NCHW
 * activations between layers.  in_packed: X / X_lo are the packed copies of the input
 * [n][ih][iw][pad8(ic)].  out_packed: Y / Y_lo receive the packed copies of the (pooled) result
 * [n][oh'][ow'][pad8(oc)]; otherwise Y is the NCHW result.  With pool = 1 and out_packed = 0 a
 * non-zero Y_lo receives one byte per pooled element [n][oc][oh'][ow']: the window position
 * (0..3 in row-major order, 4 = none) of the first element equal to the pooled value, which is
 * all that lnn_pool2x2_idx_lrelu_bwd needs of the full-resolution activation (a training step
 * then never writes it); in every other combination Y_lo is ignored when out_packed = 0.  The
 * values are those of the un-fused entries (the packed result equals lnn_nhwc_split of their
 * output for precisions 1 and 3; for precision 2 its scale comes from a bound of the result).
 * ref: op/conv2D.py:9-44, module/Conv2D.py:58-62, op/element_wise_op.py:207-221,
 * op/pool2D.py:47-146 */
int lnn_conv2d_fwd_packed(int dev, const lnn_conv_geom* g, uint64_t Y, uint64_t Y_lo, uint64_t X,
                          uint64_t X_lo, uint64_t W, uint64_t bias, int act, float alpha, int pool,
                          int in_packed, int out_packed, int precision);
/* dX += conv2D_transpose-like gradient.  ref: op/conv2D.py:46-50, op/unfold2D.py:112-138 */
int lnn_conv2d_dx(int dev, const lnn_conv_geom* g, uint64_t dX, uint64_t dY, uint64_t W,
                  int precision);
/* dW += gradient of the kernel.  ref: op/conv2D.py:52-54 */
int lnn_conv2d_dw(int dev, const lnn_conv_geom* g, uint64_t dW, uint64_t dY, uint64_t X,
                  int precision);
/* dW += the kernel gradient of a pooled block (conv -> [bias, leaky_relu] -> max_pool2D(2,2)) computed
 * from the winners of its pooling windows: T and IDX as written by lnn_pool2x2_winner_grad and
 * lnn_conv2d_fwd_packed (pooled size), X the NCHW input.  The same sums as lnn_conv2d_dw over the
 * full-resolution gradient, whose other elements are zero, in another (fixed) order.  At most 4 input
 * channels, 3x3, unit stride, 'same' padding, even height, width % 64 == 0; LNN_E_UNSUPPORTED
 * otherwise.  ref: op/conv2D.py:46-54 (dK) after op/pool2D.py:147-230 */
int lnn_conv2d_dw_winners(int dev, const lnn_conv_geom* g, uint64_t dW, uint64_t T, uint64_t IDX, uint64_t X);
/* The same two gradients from operands that are already in the packed format of lnn_nhwc_split
 * (dY [n][oh][ow][pad8(oc)], X [n][ih][iw][pad8(ic)], hi and lo each), so that a training step
 * repacks dY once for both gradients and reuses the copy of X its forward pass made.
 * ref: op/conv2D.py:46-54 */
int lnn_conv2d_dx_packed(int dev, const lnn_conv_geom* g, uint64_t dX, uint64_t dY_hi, uint64_t dY_lo,
                         uint64_t W, int precision);
int lnn_conv2d_dw_packed(int dev, const lnn_conv_geom* g, uint64_t dW, uint64_t dY_hi, uint64_t dY_lo,
                         uint64_t X_hi, uint64_t X_lo, int precision);

/* Transposed convolution Y[n, OC, OH, OW] (+)= conv2DTranspose(X[n, IC, IH, IW], K[OC, IC, KH, KW]) and its two
 * gradients, on the same tile engine: they are the three GEMMs of a convolution with the roles
 * swapped.  `g` is the geometry of the convolution whose input gradient the forward pass is:
 * g->ic = OC, g->ih / g->iw = OH / OW, g->oc = IC, g->oh / g->ow = IH / IW, stride, dilation, padl, padt.
 * ref: op/conv2DTranspose.py:8-46,68-70, op/unfold2D.py:112-138 */
int lnn_conv2d_transpose_fwd(int dev, const lnn_conv_geom* g, uint64_t Y, uint64_t X, uint64_t K, int accumulate,
                             int precision);
int lnn_conv2d_transpose_dx(int dev, const lnn_conv_geom* g, uint64_t dX, uint64_t dY, uint64_t K, int precision);
int lnn_conv2d_transpose_dk(int dev, const lnn_conv_geom* g, uint64_t dK, uint64_t dY, uint64_t X, int precision);

/* Depthwise convolution (one KH x KW filter per channel; g->oc == g->ic, K is [C, KH, KW]) and its
 * gradients; HBM-bound kernels, forward and dX bit-identical to the reference's, dK by its two
 * steps (products, then tree-ordered row sums).  ref: op/depthwise_conv2D.py:9-123 */
int lnn_depthwise_conv2d_fwd(int dev, const lnn_conv_geom* g, uint64_t Y, uint64_t X, uint64_t K, int accumulate);
int lnn_depthwise_conv2d_dx(int dev, const lnn_conv_geom* g, uint64_t dX, uint64_t dY, uint64_t K);
int lnn_depthwise_conv2d_dk(int dev, const lnn_conv_geom* g, uint64_t dK, uint64_t dY, uint64_t X);

/* ---- optimiser + data-parallel sync --------------------------------------------------- */

/* V += -lr * (G * gscale)   (momentum 0 form of the reference's two kernels, with the
 * 1/ndev of gradient averaging folded into gscale).  ref: optimizer/SGD.py:42-83 */
int lnn_sgd_step(int dev, uint64_t V, uint64_t G, int64_t n, float lr, float gscale);

/* One update of a parameter tensor V from its gradient G with the optimizer's state tensors:
 * SGD with momentum (S1 = accumulator; nesterov optional), RMSprop (S1 = mean square, beta1 = rho),
 * Adam (S1 = first, S2 = second moment).  The learning rate is decayed by 1/(1 + lr_decay*iteration)
 * and dropped per element where hash(index + seed) <= lr_dropout, as the reference's kernels do
 * (SGD evaluates that in both of its kernels: seed_a for the accumulator, seed_b for the update).
 * ref: optimizer/SGD.py:42-83, optimizer/RMSprop.py:37-69, optimizer/Adam.py:43-84,
 *      optimizer/Optimizer.py:160-203 */
enum { LNN_OPT_SGD = 0, LNN_OPT_RMSPROP = 1, LNN_OPT_ADAM = 2 };
typedef struct lnn_opt_params {
  float lr, lr_decay, lr_dropout, gscale;
  float beta1, beta2;          /* SGD: momentum in beta1; RMSprop: rho in beta1 */
  uint32_t iteration, seed_a, seed_b;
  int nesterov;
} lnn_opt_params;
int lnn_optimizer_step(int dev, int kind, uint64_t V, uint64_t G, uint64_t S1, uint64_t S2, int64_t n,
                       const lnn_opt_params* p);

/* NCCL (loaded with dlopen on first use).  One communicator per device slot.
 * ref: optimizer/Optimizer.py:149-153 (host-staged replica averaging, replaced by a
 * gradient all-reduce) */
int lnn_nccl_unique_id(void* id128);                       /* writes 128 bytes */
int lnn_nccl_init_rank(int dev, int nranks, int rank, const void* id128);
int lnn_nccl_init_all(const int* devs, int ndev);          /* single-process, all devices */
int lnn_nccl_allreduce_sum(int dev, uint64_t buf, int64_t count);
int lnn_nccl_group_start(void);
int lnn_nccl_group_end(void);
int lnn_nccl_destroy(int dev);

#ifdef __cplusplus
}
#endif
#endif /* LITENN_B200_H */
