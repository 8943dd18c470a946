/*
 * C ABI of the B200 optimisation layers.  Plain pointers and sizes only; every pointer is a DEVICE pointer on the
 * current CUDA device unless its name ends in _host.  All calls enqueue work on `stream` (a cudaStream_t passed
 * as void*) and return without synchronising the host unless stated otherwise.
 *
 * Return value: 0 on success, one of the CNL_ERR_* codes otherwise; cnl_last_error() gives a message for the
 * calling thread's last failure.
 *
 * Tensor layouts (row-major, fp32):
 *   b, init, out, grad_out, g_b, g_init : [n][ch][h][w]
 *   wx, wy, c, g_wx, g_wy, g_c          : [n][1][h][w]
 *   wx[h][w] couples pixel (h,w) with (h,w+1); wy[h][w] couples (h,w) with (h+1,w).
 */
#ifndef CNL_B200_H
#define CNL_B200_H

#ifdef __cplusplus
extern "C" {
#endif

#define CNL_OK 0
#define CNL_ERR_BAD_ID 1      /* id outside 0..9: same code the reference returns (cudaTV/cudaCode/TVInpaintFista.cu:1468-1472) */
#define CNL_ERR_BAD_SHAPE 2   /* n, ch, h or w < 1, or sizes beyond the supported range */
#define CNL_ERR_BAD_ITS 3     /* fewer than 2 iterations */
#define CNL_ERR_NO_FORWARD 4  /* backward(id) without a matching forward(id) (same n, ch, h, w, its) */
#define CNL_ERR_ALLOC 5       /* device allocation failed or the history would exceed the configured budget */
#define CNL_ERR_CUDA 6        /* a CUDA runtime call or kernel launch reported an error */
#define CNL_ERR_NULL 7        /* a required pointer is null */
#define CNL_ERR_BAD_OPTION 8

#define CNL_NUM_IDS 10        /* __uniqueIds__, cudaTV/cudaCode/TVInpaintFista.h:5 */

/* options for cnl_tv_set_option */
#define CNL_OPT_CONDITIONER 1   /* 1 (default): stateful spike kill / rescale of returned gradients after 10 runs
                                   (cudaTV/cudaCode/TVInpaintFista.cu:128-155, :1760-1792); 0: off */
#define CNL_OPT_FUSE 2          /* iterations fused per launch: 0 = automatic (default), 1 = one launch per iteration,
                                   2..4 = fixed temporal-blocking factor.  Rows that are not a multiple of four floats
                                   and tensors that are not 16-byte aligned are staged into zero-padded copies (any
                                   value but 1); keep the value between a forward call and its backward call */

#define CNL_OPT_TIMING 3        /* 1: bracket the forward and the reverse iteration loop of every call with CUDA events on
                                   the caller's stream (up to 64 calls are kept); setting the option clears the records */
#define CNL_OPT_RECOMPUTE 4     /* 0 (default): every pre-prox iterate is kept on the device (2*floor(its/2) volumes) unless
                                   that exceeds the CNL_MAX_ARENA_GB budget; 1: always keep only the floor(sqrt(its))
                                   checkpoints (y and x) and let the backward pass rebuild the history one checkpoint
                                   segment at a time, as the reference does (cudaTV/cudaCode/TVInpaintFista.cu:1690-1760).
                                   Costs one extra forward sweep per backward pass; not available with
                                   CNL_OPT_FUSE = 1 */
#define CNL_OPT_FLOW 5          /* 1 (default): a sweep of 4-iteration time blocks runs as ONE cooperative launch whose tiles are
                                   ordered by per-tile progress counters in device memory (no launch boundary, no idle tail
                                   between time blocks); 0: one launch per time block.  Both give the same bits.  Applies with
                                   CNL_OPT_FUSE = 0 or 4, every iterate resident and at most 512 iterations; environment
                                   variable CNL_TV_NO_FLOW=1 switches it off for the whole process.  A wait on a neighbouring
                                   tile that does not end within about a second makes the sweep stop; the next call on the
                                   device then returns CNL_ERR_CUDA with that reason.  Value 2 is a self-test of exactly that: the next
                                   forward sweep starts from counters no tile can satisfy, so its waits run out */

/*
 * Forward pass of the unrolled FISTA TV-inpainting layer: 2*floor(its/2) iterations starting from x = y = init.
 * Replaces  static int TVInpaintFista::forward(float* d_dx, float* d_dy, float* d_c, float* d_b, float* d_i,
 * float* d_solution, int ic, int ih, int iw, int its, int id)   (cudaTV/cudaCode/TVInpaintFista.h:71-72,
 * TVInpaintFista.cu:1463-1559), extended by a leading batch dimension n and an explicit stream.
 * Stores the iterate history that cnl_tv_backward(id) consumes in the slot `id` (0..9) of the current device.
 * Inputs are not modified.
 */
int cnl_tv_forward(const float* wx, const float* wy, const float* c, const float* b, const float* init,
                   float* out, int n, int ch, int h, int w, int its, int id, void* stream);

/*
 * Hand-derived reverse sweep.  Replaces  static int TVInpaintFista::backward(float* d_dx, float* d_dy, float* d_c,
 * float* d_b, float* d_inGrad, float* d_outGradX, float* d_outGradY, float* d_outGradC, float* d_outGradB,
 * float* d_outGradI, int ic, int ih, int iw, int its, int id)   (cudaTV/cudaCode/TVInpaintFista.h:81-85,
 * TVInpaintFista.cu:1570-1831).  The five outputs are overwritten.  Returned scalings follow the reference:
 * g_c and g_wx/g_wy carry 0.01 x the true gradient, g_b 0.1 x, g_init is the gradient w.r.t. the first primal
 * iterate.  Non-finite entries of grad_out are treated as 0.
 */
int cnl_tv_backward(const float* wx, const float* wy, const float* c, const float* b, const float* grad_out,
                    float* g_wx, float* g_wy, float* g_c, float* g_b, float* g_init,
                    int n, int ch, int h, int w, int its, int id, void* stream);

/*
 * Frees the device memory held by slot `id` on the current device and resets its run counter and running means.
 * Replaces idStruct::free_buf (cudaTV/cudaCode/TVInpaintFista.h:23-37).  Synchronises the device.
 */
int cnl_tv_release(int id);

/*
 * Copies one stored iterate of the last forward(id) into dst (device memory, n*ch*h*w floats):
 *   cnl_tv_read_history   : x^{g+1/2}, the pre-prox iterate of iteration g, 0 <= g < 2*floor(its/2)
 *                           (the reference's d_xk05, cudaTV/cudaCode/TVInpaintFista.cu:1414, :1660)
 *   cnl_tv_read_checkpoint: the momentum variable y at the k-th checkpoint iteration floor(k*sqrt(its)/2)*2
 *                           (the reference's intermediate_y[k], TVInpaintFista.cu:1504, :1543)
 * Used by the parity tests to run the oracle's reverse sweep on exactly the iterates the device produced.
 */
int cnl_tv_read_history(int id, int g, float* dst, void* stream);
int cnl_tv_read_checkpoint(int id, int k, float* dst, void* stream);
int cnl_tv_num_checkpoints(int id);

/* Per-slot options (see CNL_OPT_*).  No reference counterpart beyond its compile-time #defines
 * (cudaTV/cudaCode/TVInpaintFista.cu:22-90). */
int cnl_tv_set_option(int id, int option, int value);

/*
 * Reads and clears the CUDA-event records made under CNL_OPT_TIMING.  out_host (HOST memory, 8 doubles) receives
 * {forward ms (summed over recorded calls), kernel launches timed, recorded forward calls,
 *  reverse ms, launches timed, recorded backward calls, forward iterations the timed launches cover, reverse ditto}.
 * A record brackets the iteration kernels of a sweep: the single-launch sweep alone where it runs (a shorter last time
 * block then follows outside the record), otherwise the whole loop of launches.  Waits for the recorded events.
 * No reference counterpart (the reference has no timing code).
 */
int cnl_tv_get_timing(int id, double* out_host);

/* Number of forward+backward pairs completed on slot `id` (idStruct::run, cudaTV/cudaCode/TVInpaintFista.h:39);
 * negative on error. */
int cnl_tv_run_count(int id);

/* Number of forward passes stored on slot `id` of the current device since the library was loaded (not reset by
 * cnl_tv_release); negative on error.  A slot keeps only its LAST forward pass, like the reference's idStruct
 * (cudaTV/cudaCode/TVInpaintFista.h:18-37, checkpoints freed on re-forward): a caller that remembers this value after
 * its forward call can tell, before calling backward, whether another forward pass has replaced its history. */
int cnl_tv_forward_count(int id);

/* Kernel launches enqueued by this library on the calling thread's process since load (for benchmark accounting). */
unsigned long long cnl_launch_count(void);

/*
 * Gradient of the loss w.r.t. a scalar lambda that multiplies a raw confidence map (c = lambda * c_raw):
 * out[0] = sum_i g_c[i] * c_raw[i], a deterministic reduction in one launch (per-block partial sums in
 * double; the block that finishes last adds them in a fixed order).  This is the one value the
 * data-parallel layer all-reduces.  The reference has no learned scalar; its per-pixel confidence gradient is
 * d_outGradC (cudaTV/cudaCode/TVInpaintFista.cu:1795-1798).
 * `scratch` must hold at least cnl_dot_scratch_floats() floats of device memory.
 */
int cnl_tv_lambda_grad(const float* g_c, const float* c_raw, long long count, float* out, float* scratch,
                       void* stream);
int cnl_dot_scratch_floats(void);

/*
 * Sum of `count` (<= 64) floats over the `world` (<= 16) GPUs of one node through peer memory (NVLink / NVSwitch): the
 * all-reduce of the learned-scalar gradients, which at this size is pure latency.  Every rank stores its values straight
 * into every peer's exchange buffer (value and call number in one 8-byte store) and sums, in rank order, what the peers
 * stored into its own; the result is identical on all ranks.  No counterpart in the reference (it is single-GPU); the
 * plain alternative is an NCCL all-reduce of the same vector.
 *   peer_bufs: HOST array of `world` device pointers; peer_bufs[r] is rank r's exchange buffer as mapped into THIS
 *              process (symmetric / IPC memory), cnl_peer_allreduce_bytes() bytes each, zeroed before the first call;
 *   seq:       call number, 1, 2, 3, ... and the same on every rank for the same call.
 * Every rank must make the same calls in the same order.  Waits are bounded (about a second): a rank whose peers do not
 * answer gets NaN, and cnl_peer_allreduce_status() then returns that call's number (0: none gave up).
 * cnl_tv_lambda_grad_allreduce is cnl_tv_lambda_grad with this exchange appended inside the same kernel: out[0] is the sum
 * over all ranks.
 */
long long cnl_peer_allreduce_bytes(void);
int cnl_peer_allreduce_sum(float* values, int count, void* const* peer_bufs, int rank, int world, unsigned long long seq,
                           void* stream);
int cnl_peer_allreduce_status(void);
int cnl_tv_lambda_grad_allreduce(const float* g_c, const float* c_raw, long long count, float* out, float* scratch,
                                 void* const* peer_bufs, int rank, int world, unsigned long long seq, void* stream);

/*
 * The same reduction for callers that must not allocate device memory (real-time loops, plugins inside an engine
 * that owns all device memory): no scratch argument; the block partials live in a 32 KiB array inside the library
 * that every GPU loading the library holds until exit.  No counterpart in the reference.
 * Limits: count <= cnl_tv_lambda_grad_static_max_count() (16,777,216), otherwise CNL_ERR_BAD_SHAPE.  All calls on a
 * device share the array: calls that overlap on the GPU (different streams) race; calls on one stream are safe.
 * The first call on each device resolves the array's address and should be made outside stream capture.
 * The entry point itself calls no cudaMalloc / cudaFree and no allocating library routine.  One thing it cannot
 * avoid: when the CUDA runtime loads modules lazily, the first cudaGetSymbolAddress or kernel launch on a device
 * loads this library's module, and that one-time load may synchronise and allocate inside the driver.  Callers that
 * must never see that inside their loop make one warm-up call per device at initialisation, outside capture.
 */
int cnl_tv_lambda_grad_static(const float* g_c, const float* c_raw, long long count, float* out, void* stream);
long long cnl_tv_lambda_grad_static_max_count(void);

/*
 * Weighted-median selection over a channel-last weight volume vol [n][h][w][k] whose k weights per pixel sum to 1.
 * Replaces  static int MediMax::forward(float* d_vol, float* d_out_FS, int in, int ih, int iw, int numDisp)  and
 * MediMax::backward(float* d_vol, float* d_inGrad, float* d_outGrad0, int in, int ih, int iw, int numDisp)
 * (cudaMedian/cudaCode/medimax.h:13-14, medimax.cu:142-204).
 *   out   [n][2][h][w]: channel 0 = crossing position c + alpha, channel 1 = weight of the crossing bin; (0, 0) where
 *                       the weights never reach 0.5.
 *   index [n][h][w] (optional, may be null): crossing bin, -1 if none.  No reference counterpart (debug / tests).
 *   grad  [n][2][h][w] upstream gradient; gvol [n][h][w][k] gradient w.r.t. vol (fully overwritten).
 * Unlike the reference, n > 1 is decoded correctly (the reference decodes pixel indices against the 2-channel
 * output, medimax.cu:18-22).  k <= 453: a block stages 128 rows of k floats in shared memory; larger k returns
 * CNL_ERR_BAD_SHAPE (the reference takes any numDisp).
 */
int cnl_median_forward(const float* vol, float* out, int* index, int n, int h, int w, int k, void* stream);
int cnl_median_backward(const float* vol, const float* grad, float* gvol, int n, int h, int w, int k, void* stream);

/*
 * Differentiable quadratic fit around the rounded displaced pixel.  Replaces
 *   static int FlowQuadFitting::forward(float* d_input0, float* d_input1, float* d_dxdy, float* d_outF, int in, int ic, int ih, int iw)
 *   static int FlowQuadFitting::backward(float* d_input0, float* d_input1, float* d_dxdy, float* d_inGrad,
 *                                        float* d_outGradIm0, float* d_outGradIm1, int in, int ic, int ih, int iw)
 * (cudaQuadFit/cudaCode/quadFit.h:24-31, quadFit.cu:303-360).
 *   feat0, feat1 [n][c][h][w]; flow [n][flow_channels][h][w] (only channels 0, 1 = x, y displacement are read; the
 *   reference's Python layer passes three); out [n][3][h][w] = (fx, fy, fitted score), zero where the displaced
 *   location leaves the image; loc (optional, may be null) [n][2][h][w] int = rounded location (x, y), -1 outside.
 *   grad [n][3][h][w]; g_feat0, g_feat1 [n][c][h][w] are overwritten.  g_feat1 is accumulated with fp32 atomics (as in
 *   the reference), so its last bits depend on scheduling.  No gradient w.r.t. flow (quadFit.h:10-12).
 * cnl_quadfit_cost_*: the same fit applied to a given stencil cost5 [n][5][h][w] = (c00, c0+, c+0, c0-, c-0) of a
 * correlation to maximise, without the image-border tests; no reference counterpart as an entry point (it is the
 * fit of quadFit.cu:74-134 and its derivative :245-281).
 */
int cnl_quadfit_forward(const float* feat0, const float* feat1, const float* flow, int flow_channels, float* out,
                        int* loc, int n, int c, int h, int w, void* stream);
int cnl_quadfit_backward(const float* feat0, const float* feat1, const float* flow, int flow_channels,
                         const float* grad, float* g_feat0, float* g_feat1, int n, int c, int h, int w, void* stream);
int cnl_quadfit_cost_forward(const float* cost5, float* out, int n, int h, int w, void* stream);
int cnl_quadfit_cost_backward(const float* cost5, const float* grad, float* g_cost5, int n, int h, int w, void* stream);

/*
 * Unrolled FISTA TGV-inpainting layer (second-order TGV: primary plane u and auxiliary planes v1, v2 per channel).
 * Replaces  static int FistaTGVHuberB2_id::forward(float* d_x, float* d_y, float* d_c, float* d_b, float* d_i, float* d_out,
 * int ic, int ih, int iw, int its, int id)  and  ::backward(float* d_dx, float* d_dy, float* d_c, float* d_b, float* d_inGrad,
 * float* d_outGradX, float* d_outGradY, float* d_outGradC, float* d_outGradB, float* d_outGradI, int ic, int ih, int iw,
 * int its, int id)   (cudaTGV/cudaCode/TGVInpaintFista.h:66-86, TGVInpaintFistaBetas.cu:2475-2618, :2621-3063),
 * extended by a batch dimension and a stream.
 *   dx = [wx, beta_x], dy = [wy, beta_y] : [n][2][h][w];  c [n][1][h][w];  b [n][ch][h][w]
 *   init, out, grad_out, g_init          : [n][3*ch][h][w] ordered u(ch), v1(ch), v2(ch)  (what the reference's kernels
 *                                          index; its binding allocates too few planes, TGVInpaintFista_cuda.cpp:91, :157)
 *   g_dx, g_dy [n][2][h][w]; g_c [n][1][h][w]; g_b [n][ch][h][w]
 * 1/Lipschitz is computed per image from the weights on every call and treated as a constant by the gradient.
 * cnl_tgv_backward synchronises the stream once: like the reference it returns all-zero gradients when grad_out holds
 * a non-finite value or is identically zero (TGVInpaintFistaBetas.cu:2698-2703), and that decision is taken on the host.
 * cnl_tgv_read_state copies stored iterates for the parity tests: kind 0 = pre-prox iterate of iteration idx,
 * kind 1 = checkpointed y number idx (both n*3*ch*h*w floats), kind 2 = the n per-image 1/Lipschitz factors.
 */
int cnl_tgv_forward(const float* dx, const float* dy, const float* c, const float* b, const float* init, float* out,
                    int n, int ch, int h, int w, int its, int id, void* stream);
int cnl_tgv_backward(const float* dx, const float* dy, const float* c, const float* b, const float* grad_out,
                     float* g_dx, float* g_dy, float* g_c, float* g_b, float* g_init,
                     int n, int ch, int h, int w, int its, int id, void* stream);
int cnl_tgv_release(int id);
int cnl_tgv_set_option(int id, int option, int value);
int cnl_tgv_read_state(int id, int kind, int idx, float* dst, void* stream);
int cnl_tgv_num_checkpoints(int id);

/*
 * Learnable weighted-median FILTER: k x k window (k = 3, 5, 7; replicate border), taps sorted by value (stable), the
 * k*k normalised weights (device memory, must sum to 1) permuted alike, then the reference's selection rule
 * (sequential fp32 running sum, first rank with score < 0.5 <= score + p; cudaMedian/cudaCode/medimax.cu:27-40).
 *   flow, out, grad, g_flow [n][c][h][w]; tap [n][c][h][w] int = selected window offset index (row-major, -1: none);
 *   alpha [n][c][h][w] = the rule's interpolation factor (1 - 2 score - p) / (2 p) at the crossing (medimax.cu:33),
 *   which the backward pass needs; tap and alpha may be null in a forward call that no backward call follows;
 *   g_weights [k*k] = the reference's d/dp (medimax.cu:55-98, output gradient in the role of the position gradient)
 *   scattered back through the sort and summed over all pixels in a fixed order; g_flow = pass-through to the selected
 *   tap.  scratch: cnl_wmedian_scratch_bytes(k) bytes of device memory.
 * Only the selection rule and d/dp have a reference counterpart; the window, the sort and the input gradient do not.
 */
int cnl_wmedian_forward(const float* flow, const float* weights, float* out, int* tap, float* alpha, int n, int c, int h,
                        int w, int k, void* stream);
int cnl_wmedian_backward(const float* flow, const float* weights, const int* tap, const float* alpha, const float* grad,
                         float* g_flow, float* g_weights, void* scratch, int n, int c, int h, int w, int k, void* stream);
long long cnl_wmedian_scratch_bytes(int k);

/* Message for the last error on the calling thread ("" if none). */
const char* cnl_last_error(void);

/* Library version string. */
const char* cnl_version(void);

#ifdef __cplusplus
}
#endif
#endif /* CNL_B200_H */
