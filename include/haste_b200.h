/* haste_b200 C ABI: fused RNN layers (LSTM, GRU, IndRNN and their LayerNorm
 * variants) for NVIDIA B200 (sm_100a).
 *
 * Each entry point replaces one `haste::v0::<cell>::{ForwardPass,BackwardPass}<T>::Run`
 * of lmnt-com/haste (file:line cited per function).  Conventions shared by all:
 *
 *   - Every pointer is a DEVICE pointer owned by the caller, including scratch.
 *     Tensors are dense, row-major, rightmost index fastest
 *     (T steps, N batch, C input size, H hidden size), as in lib/haste.h:18-26.
 *   - `dtype` selects the storage type of EVERY tensor of the call:
 *     HASTE_B200_F32 (float), HASTE_B200_BF16 (__nv_bfloat16; all arithmetic,
 *     carries and accumulators stay fp32) or, for the GRU entry points and
 *     haste_b200_gemm, HASTE_B200_F16 (__half, same rule).
 *   - `h`/`c` are [T+1,N,H]; slot 0 holds the initial state and is filled by the
 *     caller.  Gate order: i,g,f,o (LSTM), z,r,g (GRU).
 *   - Outputs documented as "accumulated" are added to and must be zeroed by the
 *     caller (dW, dR, db*, du, dgamma*, dbeta*, dh, dc); `dx` is assigned.
 *   - `zoneout_mask` may be NULL: zoneout is applied only if zoneout_prob != 0
 *     and the mask is non-NULL.
 *   - Backward entry points take `transposed_inputs`: non-zero means x, W and R
 *     are passed pre-transposed exactly as the reference wants them
 *     (x_t [C,T,N], W_t [G*H,C], R_t [G*H,H]); zero means they are passed in their
 *     forward layout (x [T,N,C], W [C,G*H], R [H,G*H]) and no copy is made.
 *   - `stream` is a cudaStream_t (NULL = default stream).  All work is issued on
 *     it, in order; nothing blocks the host.
 *   - Return value: HASTE_B200_OK or an error code; haste_b200_last_error()
 *     returns a thread-local message.  No exceptions cross this boundary.
 */
#ifndef HASTE_B200_H_
#define HASTE_B200_H_

#ifdef __cplusplus
extern "C" {
#endif

enum {
  HASTE_B200_OK = 0,
  HASTE_B200_ERR_INVALID = 1,     /* bad shape, NULL pointer, unknown dtype */
  HASTE_B200_ERR_CUDA = 2,        /* a CUDA runtime call failed */
  HASTE_B200_ERR_TIMEOUT = 3,     /* a bounded in-kernel wait ran out */
  HASTE_B200_ERR_UNSUPPORTED = 4  /* shape outside what a kernel supports */
};

/* HASTE_B200_F16 (__half storage, fp32-grade arithmetic on exact bf16 (hi, lo) splits of the
 * stored values): GRU entry points and haste_b200_gemm only - the one reduced-precision type
 * the reference ships (lib/gru_forward_gpu.cu.cc:373). */
enum { HASTE_B200_F32 = 0, HASTE_B200_BF16 = 1, HASTE_B200_F16 = 2,
       /* LayerNormLSTM entry points only.  Tensors the caller exchanges with the layer are
        * __nv_bfloat16 exactly as with HASTE_B200_BF16 (x, W, R, b, gamma*, beta_h, h, c,
        * zoneout_mask, dh_new, dc_new and every gradient), but everything the forward pass
        * leaves for the backward pass is FLOAT: act_Wx, act_Wx_norm, act_Rh, act_c_norm,
        * tmp_Rh and the three caches must be float buffers of the documented shapes, and h and
        * c are carried in fp32 from step to step (only the returned copies are rounded).
        * Three LayerNorms per step amplify the rounding of a bf16-stored x.W, LN(x.W) or
        * running h to 2e-2 .. 1e-1 of the result; this mode stays within 2e-2 of fp32
        * arithmetic on the same bf16 inputs.  It runs the fp32 kernels on converted operands,
        * i.e. at fp32 speed with bf16 interface traffic. */
       HASTE_B200_BF16_WIDE = 3 };

const char* haste_b200_last_error(void);
const char* haste_b200_version(void);

/* Selects the implementation of the recurrence / contractions for subsequent
 * calls of the calling process (debug and test knob; 0 = automatic). */
enum {
  HASTE_B200_PATH_AUTO = 0,
  HASTE_B200_PATH_STEPWISE = 1,   /* one launch sequence per time step */
  HASTE_B200_PATH_PERSISTENT = 2, /* one persistent kernel per layer pass */
  HASTE_B200_PATH_NO_TENSOR_CORE = 3 /* automatic, but without the tcgen05 recurrence */
};
int haste_b200_set_recurrence_path(int path);
/* Limits the number of SMs one persistent recurrence launch of the calling process occupies
 * (0 = the whole GPU, the default).  With half the GPU per launch the two directions of a
 * bidirectional layer, issued on two streams, are co-resident and run concurrently.  Honoured by
 * the tensor-core GRU recurrence; no reference counterpart. */
int haste_b200_set_sm_budget(int sms);
enum { HASTE_B200_GEMM_AUTO = 0, HASTE_B200_GEMM_SIMT = 1, HASTE_B200_GEMM_TCGEN05 = 2,
       HASTE_B200_GEMM_TCGEN05_SINGLE = 3 /* tensor cores, never the CTA-pair kernel */ };
int haste_b200_set_gemm_path(int path);
/* Number of kernels this library has launched in the calling process. */
long long haste_b200_launch_count(void);
/* Device-side timing by phase (CUDA events on each call's stream).  After
 * haste_b200_profile_enable(1), haste_b200_profile_read fills ms[0..n) with the
 * milliseconds spent since the previous read in: 0 input projection, 1 forward
 * recurrence, 2 backward recurrence, 3 weight-gradient contractions, 4 input-gradient
 * contraction, 5 everything else.  Reading synchronises with the recorded work. */
/* Waits for the work queued on `stream` and reports whether any kernel of this library
 * abandoned a bounded wait since the last check (HASTE_B200_ERR_TIMEOUT) - the
 * asynchronous entry points cannot report that themselves. */
int haste_b200_sync_check(void* stream);
int haste_b200_profile_enable(int on);
/* Measurement aid, no reference counterpart: runs `steps` steps of the forward recurrence's
 * inter-CTA hand-off alone (publish tagged words, wait for all of them, CTA barrier; no
 * contraction, no gate math, no activation traffic) with the tiling a recurrence of batch N
 * and H hidden units uses, waits for it, and returns the device time per step in
 * microseconds.  N*H must fit one CTA per SM (16 rows x 16 units per CTA). */
int haste_b200_probe_exchange_latency(int N, int H, int steps, float* us_per_step, void* stream);
int haste_b200_profile_read(float* ms, int n);

/* ---- LSTM -------------------------------------------------------------- */
/* Replaces lstm::ForwardPass<T>::Run  (lib/haste/lstm.h:118-129,
 * lib/lstm_forward_gpu.cu.cc:313-366).
 *   W [C,4H]  R [H,4H]  b [4H]  x [T,N,C]  h,c [T+1,N,H]
 *   v [T,N,4H] receives the gate activations when training (may be NULL otherwise)
 *   tmp_Rh [N,4H] scratch  zoneout_mask [T,N,H] or NULL */
int haste_b200_lstm_forward(int dtype, int training, int T, int N, int C, int H,
                            const void* W, const void* R, const void* b, const void* x,
                            void* h, void* c, void* v, void* tmp_Rh,
                            float zoneout_prob, const void* zoneout_mask, void* stream);

/* Replaces lstm::BackwardPass<T>::Run  (lib/haste/lstm.h:248-265,
 * lib/lstm_backward_gpu.cu.cc:319-405).
 *   dh_new, dc_new [T+1,N,H] (slot 0 is never read)  dx [T,N,C] assigned
 *   dW [C,4H] dR [H,4H] db [4H] dh,dc [N,H] accumulated;  v is overwritten. */
int haste_b200_lstm_backward(int dtype, int transposed_inputs, int T, int N, int C, int H,
                             const void* W, const void* R, const void* b, const void* x,
                             const void* h, const void* c, const void* dh_new,
                             const void* dc_new, void* dx, void* dW, void* dR, void* db,
                             void* dh, void* dc, void* v, const void* zoneout_mask,
                             void* stream);

/* ---- GRU --------------------------------------------------------------- */
/* Replaces gru::ForwardPass<T>::Run  (lib/haste/gru.h:86-98,
 * lib/gru_forward_gpu.cu.cc:310-371).
 *   W [C,3H] R [H,3H] bx,br [3H]  v [T,N,4H] = [z,r,g,Rh_g+br_g] when training
 *   tmp_Wx [T,N,3H], tmp_Rh [N,3H] scratch */
int haste_b200_gru_forward(int dtype, int training, int T, int N, int C, int H,
                           const void* W, const void* R, const void* bx, const void* br,
                           const void* x, void* h, void* v, void* tmp_Wx, void* tmp_Rh,
                           float zoneout_prob, const void* zoneout_mask, void* stream);

/* Replaces gru::BackwardPass<T>::Run  (lib/haste/gru.h:191-209,
 * lib/gru_backward_gpu.cu.cc:322-409).  dp,dq [T,N,3H] scratch (written). */
int haste_b200_gru_backward(int dtype, int transposed_inputs, int T, int N, int C, int H,
                            const void* W, const void* R, const void* bx, const void* br,
                            const void* x, const void* h, const void* v, const void* dh_new,
                            void* dx, void* dW, void* dR, void* dbx, void* dbr, void* dh,
                            void* dp, void* dq, const void* zoneout_mask, void* stream);

/* ---- single-step forms (the reference's Iterate, for autoregressive use) -- */
/* One time step with the state in separate [N,H] buffers; same arithmetic as T == 1 of the
 * sequence entry points, no scratch beyond the arguments.  x [N,C]; v, tmp_* sized for one step.
 * Replaces lstm::ForwardPass<T>::Iterate (lib/haste/lstm.h:73-86,
 * lib/lstm_forward_gpu.cu.cc:141-208). */
int haste_b200_lstm_forward_iterate(int dtype, int training, int N, int C, int H,
                                    const void* W, const void* R, const void* b, const void* x,
                                    const void* h, const void* c, void* h_out, void* c_out,
                                    void* v, void* tmp_Rh, float zoneout_prob,
                                    const void* zoneout_mask, void* stream);
/* Replaces lstm::BackwardPass<T>::Iterate (lib/haste/lstm.h:201-219,
 * lib/lstm_backward_gpu.cu.cc:144-243).  h, c: state before the step; c_new: cell state the
 * step produced; dh_new, dc_new [N,H]: gradient arriving at the step's outputs; dh, dc [N,H]
 * in/out carries; dW, dR, db accumulate; dx [N,C] assigned; v [N,4H] is overwritten.
 * With transposed_inputs, x is [C,N] and W, R are [4H,C], [4H,H]. */
int haste_b200_lstm_backward_iterate(int dtype, int transposed_inputs, int N, int C, int H,
                                     const void* W, const void* R, const void* b, const void* x,
                                     const void* h, const void* c, const void* c_new,
                                     const void* dh_new, const void* dc_new, void* dx, void* dW,
                                     void* dR, void* db, void* dh, void* dc, void* v,
                                     const void* zoneout_mask, void* stream);
/* Replaces gru::ForwardPass<T>::Iterate (lib/haste/gru.h:72-84,
 * lib/gru_forward_gpu.cu.cc:160-212).  v [N,4H] (may be null when not training),
 * tmp_Wx, tmp_Rh [N,3H]. */
int haste_b200_gru_forward_iterate(int dtype, int training, int N, int C, int H, const void* W,
                                   const void* R, const void* bx, const void* br, const void* x,
                                   const void* h, void* h_out, void* v, void* tmp_Wx,
                                   void* tmp_Rh, float zoneout_prob, const void* zoneout_mask,
                                   void* stream);
/* Replaces gru::BackwardPass<T>::Iterate (lib/haste/gru.h:172-189,
 * lib/gru_backward_gpu.cu.cc:168-250).  dp, dq [N,3H] scratch (written). */
int haste_b200_gru_backward_iterate(int dtype, int transposed_inputs, int N, int C, int H,
                                    const void* W, const void* R, const void* bx, const void* br,
                                    const void* x, const void* h, const void* v,
                                    const void* dh_new, void* dx, void* dW, void* dR, void* dbx,
                                    void* dbr, void* dh, void* dp, void* dq,
                                    const void* zoneout_mask, void* stream);

/* ---- IndRNN ------------------------------------------------------------ */
/* Replaces indrnn::ForwardPass<T>::Run  (lib/haste/indrnn.h:38-47,
 * lib/indrnn_forward_gpu.cu.cc:126-210).  W [C,H] u,b [H] workspace [T,N,H]. */
int haste_b200_indrnn_forward(int dtype, int training, int T, int N, int C, int H,
                              const void* W, const void* u, const void* b, const void* x,
                              void* h, void* workspace, float zoneout_prob,
                              const void* zoneout_mask, void* stream);

/* Replaces indrnn::BackwardPass<T>::Run  (lib/haste/indrnn.h:66-80,
 * lib/indrnn_backward_gpu.cu.cc:134-207).  dW [C,H] is ASSIGNED (the reference
 * uses beta=0 here); du, db [H], dh [N,H] accumulated. */
int haste_b200_indrnn_backward(int dtype, int transposed_inputs, int T, int N, int C, int H,
                               const void* W, const void* u, const void* b, const void* x,
                               const void* h, const void* dh_new, void* dx, void* dW,
                               void* du, void* db, void* dh, void* workspace,
                               const void* zoneout_mask, void* stream);

/* ---- LayerNorm --------------------------------------------------------- */
/* Replaces layer_norm::ForwardPass<T>::Run/RunPartial  (lib/haste/layer_norm.h:30-49,
 * lib/layer_norm_forward_gpu.cu.cc:22-150).  Row LayerNorm over `width` with
 * biased variance and eps 1e-5; beta may be NULL; cache [rows,2] = (mean, invstd). */
int haste_b200_layer_norm_forward(int dtype, int rows, int width, const void* gamma,
                                  const void* beta, const void* x, void* y, void* cache,
                                  void* stream);

/* Replaces layer_norm::BackwardPass<T>::Run/RunPartial  (lib/haste/layer_norm.h:63-79,
 * lib/layer_norm_backward_gpu.cu.cc:23-165).  dx may alias dy.  dgamma [width]
 * (and dbeta if non-NULL) accumulated. */
int haste_b200_layer_norm_backward(int dtype, int rows, int width, const void* gamma,
                                   const void* x, const void* dy, void* dx, void* dgamma,
                                   void* dbeta, const void* cache, void* stream);

/* No counterpart in the reference.  The same computation as
 * haste_b200_layer_norm_backward, for callers that cannot let the library allocate: a
 * process whose own arena already owns all device memory, code inside a stream-capture
 * region, or a latency-critical loop that must not hit cudaMalloc's device-wide
 * synchronisation.  The reduction scratch lives in a fixed 2 MiB array inside the library
 * image (held by every GPU that loads the library until the process exits) instead of the
 * grow-only pool, so this call never allocates or frees.
 *   - width must be <= 4096; larger widths return HASTE_B200_ERR_UNSUPPORTED with a message.
 *   - The first call on each device looks up the array's device address (the device of the
 *     pointers must be current); make that first call before starting any stream capture.
 *   - All calls on a device share the one array.  Nothing in it needs to start at zero (each
 *     call overwrites what it later reads), but two calls that overlap on the GPU - different
 *     streams, no ordering between them - race on it and give wrong gradients. */
int haste_b200_layer_norm_backward_noalloc(int dtype, int rows, int width, const void* gamma,
                                           const void* x, const void* dy, void* dx,
                                           void* dgamma, void* dbeta, const void* cache,
                                           void* stream);

/* ---- LayerNormLSTM ----------------------------------------------------- */
/* Replaces layer_norm_lstm::ForwardPass<T>::Run  (lib/haste/layer_norm_lstm.h:75-92,
 * lib/layer_norm_lstm_forward_gpu.cu.cc:276-340).
 *   gamma_Wx, gamma_Rh [4H] (the two rows of the module's [2,4H] gamma: the first
 *   normalises x.W, the second h.R)  gamma_h, beta_h [H]
 *   act_Wx, act_Wx_norm, act_Rh [T,N,4H]  act_c_norm [T,N,H]
 *   cache_Wx, cache_Rh, cache_c [T,N,2]  tmp_Rh [N,4H] */
int haste_b200_layer_norm_lstm_forward(
    int dtype, int training, int T, int N, int C, int H, const void* W, const void* R,
    const void* b, const void* gamma_Wx, const void* gamma_Rh, const void* gamma_h,
    const void* beta_h, const void* x,
    void* h, void* c, void* act_Wx, void* act_Wx_norm, void* cache_Wx, void* act_Rh,
    void* cache_Rh, void* act_c_norm, void* cache_c, void* tmp_Rh, float zoneout_prob,
    const void* zoneout_mask, void* stream);

/* Replaces layer_norm_lstm::BackwardPass<T>::Run  (lib/haste/layer_norm_lstm.h:160-183,
 * lib/layer_norm_lstm_backward_gpu.cu.cc:255-352).  dgamma_Wx, dgamma_Rh [4H], dgamma_h,
 * dbeta_h [H] accumulated; act_Wx, act_Wx_norm, act_Rh, act_c_norm are overwritten. */
int haste_b200_layer_norm_lstm_backward(
    int dtype, int transposed_inputs, int T, int N, int C, int H, const void* W, const void* R,
    const void* b, const void* gamma_Wx, const void* gamma_Rh, const void* gamma_h,
    const void* beta_h, const void* x,
    const void* h, const void* c, const void* dh_new, const void* dc_new, void* dx, void* dW,
    void* dR, void* db, void* dgamma_Wx, void* dgamma_Rh, void* dgamma_h, void* dbeta_h, void* dh,
    void* dc,
    void* act_Wx, void* act_Wx_norm, const void* cache_Wx, void* act_Rh, const void* cache_Rh,
    void* act_c_norm, const void* cache_c, const void* zoneout_mask, void* stream);

/* ---- LayerNormGRU ------------------------------------------------------ */
/* Replaces layer_norm_gru::ForwardPass<T>::Run  (lib/haste/layer_norm_gru.h:72-88,
 * lib/layer_norm_gru_forward_gpu.cu.cc:243-305).  gamma_Wx, gamma_Rh [3H];
 * act_Wx, tmp_Wx_norm [T,N,3H]; act_Rh [T,N,3H]; tmp_Rh_norm [N,3H]. */
int haste_b200_layer_norm_gru_forward(
    int dtype, int training, int T, int N, int C, int H, const void* W, const void* R,
    const void* bx, const void* br, const void* gamma_Wx, const void* gamma_Rh, const void* x,
    void* h, void* v, void* act_Wx, void* cache_Wx, void* tmp_Wx_norm, void* act_Rh, void* cache_Rh,
    void* tmp_Rh_norm, float zoneout_prob, const void* zoneout_mask, void* stream);

/* Replaces layer_norm_gru::BackwardPass<T>::Run  (lib/haste/layer_norm_gru.h:164-184,
 * lib/layer_norm_gru_backward_gpu.cu.cc:246-310).  dgamma_Wx, dgamma_Rh [3H] accumulated;
 * act_Rh is overwritten (it receives the gradient of h.R). */
int haste_b200_layer_norm_gru_backward(
    int dtype, int transposed_inputs, int T, int N, int C, int H, const void* W, const void* R,
    const void* bx, const void* br, const void* gamma_Wx, const void* gamma_Rh, const void* x,
    const void* h, const void* v, const void* dh_new, void* dx, void* dW, void* dR, void* dbx,
    void* dbr, void* dgamma_Wx, void* dgamma_Rh, void* dh, void* dp, void* dq, const void* act_Wx, const void* cache_Wx,
    void* act_Rh, const void* cache_Rh, const void* zoneout_mask, void* stream);

/* ---- LayerNormIndRNN --------------------------------------------------- */
/* Replaces layer_norm_indrnn::ForwardPass<T>::Run  (lib/haste/layer_norm_indrnn.h:38-49,
 * lib/layer_norm_indrnn_forward_gpu.cu.cc:128-213).  gamma [H] (row 0 of the
 * module's [2,H] parameter); act_Wx, workspace [T,N,H]. */
int haste_b200_layer_norm_indrnn_forward(
    int dtype, int training, int T, int N, int C, int H, const void* W, const void* u,
    const void* b, const void* gamma, const void* x, void* h, void* workspace, void* act_Wx,
    void* cache_Wx, float zoneout_prob, const void* zoneout_mask, void* stream);

/* Replaces layer_norm_indrnn::BackwardPass<T>::Run  (lib/haste/layer_norm_indrnn.h:68-83,
 * lib/layer_norm_indrnn_backward_gpu.cu.cc:136-209).  dW assigned. */
int haste_b200_layer_norm_indrnn_backward(
    int dtype, int transposed_inputs, int T, int N, int C, int H, const void* W, const void* u,
    const void* b, const void* gamma, const void* x, const void* h, const void* dh_new,
    void* dx, void* dW, void* du, void* db, void* dgamma, void* dh, void* workspace,
    const void* act_Wx, const void* cache_Wx, const void* zoneout_mask, void* stream);

/* ---- Dense contraction (exposed for tests and benchmarks) --------------- */
/* C[m,n] (+)= sum_k A(m,k) B(k,n);  A(m,k) at a[m*a_rs + k*a_cs],
 * B(k,n) at b[k*b_rs + n*b_cs], C row-major with leading dimension ldc.
 * This is the library's replacement for the cuBLAS calls of lib/blas.h:48-61. */
int haste_b200_gemm(int dtype, int M, int N, int K, const void* a, long long a_rs,
                    long long a_cs, const void* b, long long b_rs, long long b_cs, void* c,
                    long long ldc, int accumulate, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HASTE_B200_H_ */
