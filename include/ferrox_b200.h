/* ferrox_b200 — C ABI of the B200 (sm_100a) implementation of Ferrox's training hot path.
 *
 * This is the boundary a Ferrox build binds instead of its PTX launcher: every entry point
 * below replaces the body of one method of `CudaOps<T>` (src/backend/cuda/ops.rs) together
 * with the `KernelManager::launch_*` wrapper (src/backend/cuda/kernels.rs) and the kernel it
 * used to start (kernels/*.cu).  The citation on each declaration names that method.
 *
 * Conventions (all taken from how the reference drives its kernels):
 *  - Buffers are raw device pointers to contiguous row-major data (NCHW for images, KCRS for
 *    filters); the library never allocates, frees or resizes tensor memory — outputs and
 *    scratch come from the caller's pool (src/backend/cuda/ops.rs:121-133).  The only device
 *    memory it owns is an 8 KB status / counter block per handle, allocated by fxb_create.
 *  - Outputs are written in full: a recycled pool buffer may hold stale data and may be
 *    longer than requested (src/backend/cuda/context.rs:72).
 *  - Every call is asynchronous on the caller's stream (the reference's "compute" stream,
 *    src/backend/cuda/context.rs:40-44); no hidden synchronisation, no default-stream use.
 *  - Return value: FXB_OK or an FXB_ERR_* code; fxb_last_error() gives the message that the
 *    Rust shim turns into `Err(String)`.  Nothing aborts, nothing traps on the device.
 *  - `_f32` entry points contract on the tcgen05 tensor cores (3xTF32 by default, see
 *    fxb_set_math_mode); `_f64` entry points use the f64 tensor instruction (DMMA).
 *  - A handle belongs to one device and one caller thread at a time.
 */
#ifndef FERROX_B200_H
#define FERROX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FXB_OK 0
#define FXB_ERR_INVALID_ARGUMENT 1
#define FXB_ERR_UNSUPPORTED 2
#define FXB_ERR_LAUNCH_FAILED 3
#define FXB_ERR_DEVICE_TIMEOUT 4
#define FXB_ERR_CUDA 5
#define FXB_ERR_WORKSPACE 6

#define FXB_ACT_NONE 0
#define FXB_ACT_RELU 1
#define FXB_ACT_SIGMOID 2
#define FXB_ACT_TANH 3

#define FXB_MATH_3XTF32 0 /* default: hi/lo split, three MMAs per product, f32-grade accuracy */
#define FXB_MATH_TF32 1   /* one MMA per product, ~1e-3 relative accuracy */

typedef struct fxb_context* fxb_handle_t;
typedef void* fxb_stream_t; /* a cudaStream_t / CUstream */

/* conv2d geometry: input [N,C,H,W], filter [K,C,R,S], output [N,K,OH,OW] with
 * OH = (H + 2*pad_h - R) / stride_h + 1 (src/backend/cuda/ops.rs:1250-1251). */
typedef struct fxb_conv2d_desc {
    int64_t N, C, H, W;
    int64_t K, R, S;
    int64_t stride_h, stride_w;
    int64_t pad_h, pad_w;
} fxb_conv2d_desc;

/* ---- context (replaces CudaContextManager::from_device_id + KernelManager::new,
 *      src/backend/cuda/context.rs:35-59, src/backend/cuda/kernels.rs:223-262) ---- */
int fxb_create(int device, fxb_handle_t* out);
int fxb_destroy(fxb_handle_t h);
const char* fxb_last_error(fxb_handle_t h); /* h may be NULL: last error of this thread */
const char* fxb_status_string(int status);
int fxb_set_math_mode(fxb_handle_t h, int mode);
/* f32 convolutions (forward and input gradient) have three operand paths with identical results.
 * FXB_PATH_AUTO (default): with a large enough workspace the operands are pre-split into it and
 * copied into the tensor-core tiles by the tensor-map engine (cp.async.bulk.tensor); shapes that
 * tensor maps cannot describe use 16-byte cp.async copies instead.  FXB_PATH_CP_ASYNC skips the
 * tensor-map engine.  FXB_PATH_GATHER always gathers and splits inside the kernel (no workspace use). */
#define FXB_PATH_AUTO 0
#define FXB_PATH_GATHER 1
#define FXB_PATH_CP_ASYNC 2
int fxb_set_operand_path(fxb_handle_t h, int path);
/* The tensor-map f32 convolution kernels keep a running sum in TMEM for `stages` K stages of 32 values (1, 2 or 4)
 * before the drain warps add it into their f32 registers with round-to-nearest adds.  The tensor core's own
 * accumulation truncates, so fewer drains trade a little accuracy (still far inside the f32 tolerance) for fewer
 * TMEM reads.  Default 4 (measured on conv 64->128 at batch 1024: kernel 13 % faster than with 1, maximum error
 * against an f64 evaluation 3e-6 instead of 2e-6 at an output rms of 1.4). */
int fxb_set_accumulate_stages(fxb_handle_t h, int stages);
/* 0 (default) reproduces the reference's Sigmoid::gradient, dY*s*(s-1)
 * (src/ops/unary.rs:270-273); 1 selects the derivative dY*s*(1-s). */
int fxb_set_sigmoid_grad_mode(fxb_handle_t h, int math_mode);
/* Synchronises `stream` and reports whether any kernel gave up on a bounded device-side
 * wait since the last call (FXB_ERR_DEVICE_TIMEOUT) — the counterpart of the launch error
 * string formatted at src/backend/cuda/kernels.rs:33. */
int fxb_check_device_status(fxb_handle_t h, fxb_stream_t stream);
/* Self-test of that convention (no reference counterpart): launches one warp that waits, for at most
 * `limit_cycles` SM cycles (1..1e8), on a barrier nobody arrives on.  The wait gives up, the kernel
 * returns normally, and the next fxb_check_device_status reports FXB_ERR_DEVICE_TIMEOUT with tag 99
 * and clears it; the handle stays usable.  Nothing faults, traps or spins without a bound. */
int fxb_selftest_bounded_wait(fxb_handle_t h, int64_t limit_cycles, fxb_stream_t stream);
int fxb_version(void);
/* Number of kernels this handle has launched so far (for launch accounting in benchmarks). */
uint64_t fxb_launch_count(fxb_handle_t h);

/* ---- matmul: CudaOps::matmul (src/backend/cuda/ops.rs:841-889), kernel `matmul`/`matmul_f64`
 *      (kernels/matmul.cu:20-105).  C[M,N] = A[M,K] . B[K,N]. ---- */
int fxb_matmul_f32(fxb_handle_t h, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                   fxb_stream_t stream);
int fxb_matmul_f64(fxb_handle_t h, const double* A, const double* B, double* C, int64_t M, int64_t N, int64_t K,
                   fxb_stream_t stream);

/* General form with transposed views instead of the clone+transpose+materialize of
 * MatMul::gradient (src/ops/matrix.rs:45-52; src/backend/storage/cuda.rs:826-857):
 * C[M,N] = act(op(A) . op(B) + bias[N]);  op(A) is A[M,K] (ld = lda) or, with trans_a, the
 * transpose of A[K,M].  workspace may be NULL (no split-K, and no tensor-map engine: with a workspace of
 * fxb_gemm_workspace_bytes, large f32 products pre-split both operands into it (which also absorbs the
 * transposes) and run on the kernel of the convolutions, tiles fed by the copy engine). */
int fxb_gemm_f32(fxb_handle_t h, int trans_a, int trans_b, int64_t M, int64_t N, int64_t K, const float* A,
                 int64_t lda, const float* B, int64_t ldb, float* C, int64_t ldc, const float* bias, int act,
                 void* workspace, size_t workspace_bytes, fxb_stream_t stream);
int fxb_gemm_f64(fxb_handle_t h, int trans_a, int trans_b, int64_t M, int64_t N, int64_t K, const double* A,
                 int64_t lda, const double* B, int64_t ldb, double* C, int64_t ldc, const double* bias, int act,
                 void* workspace, size_t workspace_bytes, fxb_stream_t stream);
size_t fxb_gemm_workspace_bytes(fxb_handle_t h, int64_t M, int64_t N, int64_t K, size_t elem_size);

/* ---- fused linear layer.  Forward replaces Transpose + MatMul + BroadcastTo + Add + activation
 *      (src/nn/layers/linear.rs:183-279): Y[B,out] = act(X[B,in] . W[out,in]^T + bias).
 *      Backward replaces activation gradient + Add::gradient + MatMul::gradient +
 *      Transpose::gradient (src/ops/unary.rs:254-375, src/ops/basic.rs:95-115,
 *      src/ops/matrix.rs:30-55): dZ = dY * act'(.), dX = dZ . W, dW = dZ^T . X, db = sum_rows dZ.
 *      `Y` is the layer output (any activation; for relu Y>0 <=> pre-activation>0); NULL when
 *      act == FXB_ACT_NONE.  dX, db may be NULL. ---- */
int fxb_linear_fwd_f32(fxb_handle_t h, const float* X, const float* W, const float* bias, float* Y, int64_t B,
                       int64_t in_features, int64_t out_features, int act, fxb_stream_t stream);
int fxb_linear_fwd_f64(fxb_handle_t h, const double* X, const double* W, const double* bias, double* Y, int64_t B,
                       int64_t in_features, int64_t out_features, int act, fxb_stream_t stream);
/* The same with a workspace (fxb_linear_fwd_workspace_bytes; 0 when none is of use): large f32 layers then
 * run on the tensor-map engine (operands pre-split into the workspace, tiles fed by the copy engine). */
int fxb_linear_fwd_ws_f32(fxb_handle_t h, const float* X, const float* W, const float* bias, float* Y, int64_t B,
                          int64_t in_features, int64_t out_features, int act, void* workspace, size_t workspace_bytes,
                          fxb_stream_t stream);
int fxb_linear_fwd_ws_f64(fxb_handle_t h, const double* X, const double* W, const double* bias, double* Y, int64_t B,
                          int64_t in_features, int64_t out_features, int act, void* workspace, size_t workspace_bytes,
                          fxb_stream_t stream);
size_t fxb_linear_fwd_workspace_bytes(fxb_handle_t h, int64_t B, int64_t in_features, int64_t out_features,
                                      size_t elem_size);
int fxb_linear_bwd_f32(fxb_handle_t h, const float* X, const float* W, const float* Y, const float* dY, float* dX,
                       float* dW, float* db, int64_t B, int64_t in_features, int64_t out_features, int act,
                       void* workspace, size_t workspace_bytes, fxb_stream_t stream);
int fxb_linear_bwd_f64(fxb_handle_t h, const double* X, const double* W, const double* Y, const double* dY,
                       double* dX, double* dW, double* db, int64_t B, int64_t in_features, int64_t out_features,
                       int act, void* workspace, size_t workspace_bytes, fxb_stream_t stream);
size_t fxb_linear_bwd_workspace_bytes(fxb_handle_t h, int64_t B, int64_t in_features, int64_t out_features,
                                      size_t elem_size);

/* ---- conv2d forward: CudaOps::conv2d_forward (src/backend/cuda/ops.rs:1202-1298), kernel
 *      `conv2d_forward[_f64]` (kernels/convolutions.cu:10-136).  The fused form also covers the
 *      bias broadcast + Add (src/nn/layers/utils.rs:6-42, conv2d.rs:203-208) and the activation.
 *      bias may be NULL. ---- */
int fxb_conv2d_forward_f32(fxb_handle_t h, const float* X, const float* W, float* Y, const fxb_conv2d_desc* d,
                           void* workspace, size_t workspace_bytes, fxb_stream_t stream);
int fxb_conv2d_forward_f64(fxb_handle_t h, const double* X, const double* W, double* Y, const fxb_conv2d_desc* d,
                           void* workspace, size_t workspace_bytes, fxb_stream_t stream);
int fxb_conv2d_bias_act_fwd_f32(fxb_handle_t h, const float* X, const float* W, const float* bias, float* Y,
                                const fxb_conv2d_desc* d, int act, void* workspace, size_t workspace_bytes,
                                fxb_stream_t stream);
int fxb_conv2d_bias_act_fwd_f64(fxb_handle_t h, const double* X, const double* W, const double* bias, double* Y,
                                const fxb_conv2d_desc* d, int act, void* workspace, size_t workspace_bytes,
                                fxb_stream_t stream);
/* Workspace of the f32 forward / input-gradient kernels (0 for f64).  With a 256-byte aligned workspace of
 * at least this size the image and the filter are first rewritten once into TF32 hi / lo arrays with
 * 4 channels per pixel contiguous (one plane per stride class), and the contraction kernel's operand
 * tiles are filled by the tensor-map copy engine (cp.async.bulk.tensor), or by 16-byte cp.async copies
 * for shapes a tensor map cannot describe; with workspace == NULL (or too small) the operands are
 * gathered and split on the fly inside the kernel.  All ways give the same values. */
size_t fxb_conv2d_fprop_workspace_bytes(fxb_handle_t h, const fxb_conv2d_desc* d, size_t elem_size);
/* Runs only the operand pre-pass of fxb_conv2d_forward_f32 (image and filter rewritten as TF32 hi / lo
 * arrays in the workspace) and stops before the contraction kernel, so that the two parts can be timed
 * separately.  No reference counterpart.  FXB_ERR_UNSUPPORTED for shapes whose forward pass has no
 * pre-pass (C*R*S <= 32, or shapes the tensor-map engine cannot describe). */
int fxb_conv2d_fprop_prepass_f32(fxb_handle_t h, const float* X, const float* W, const fxb_conv2d_desc* d,
                                 void* workspace, size_t workspace_bytes, fxb_stream_t stream);
/* The other half: only the contraction kernel of fxb_conv2d_bias_act_fwd_f32, reading the operands that
 * fxb_conv2d_fprop_prepass_f32 left in `workspace` for the same descriptor (so the kernel can be timed
 * on its own).  No reference counterpart.  Same FXB_ERR_UNSUPPORTED cases as the pre-pass. */
int fxb_conv2d_fprop_main_f32(fxb_handle_t h, const float* bias, float* Y, const fxb_conv2d_desc* d, int act,
                              void* workspace, size_t workspace_bytes, fxb_stream_t stream);
size_t fxb_conv2d_dgrad_workspace_bytes(fxb_handle_t h, const fxb_conv2d_desc* d, size_t elem_size);

/* ---- conv2d input gradient: CudaOps::deconv2d (src/backend/cuda/ops.rs:1458-1539), kernel
 *      `deconv2d[_f64]` (kernels/convolutions.cu:360-438).  dX[N,C,H,W] from dY[N,K,OH,OW] and
 *      W[K,C,R,S]; every dX element is written exactly once.  The fused form multiplies dY by
 *      act'(Y) on the fly (Y = the conv layer's activated output). ---- */
int fxb_deconv2d_f32(fxb_handle_t h, const float* dY, const float* W, float* dX, const fxb_conv2d_desc* d,
                     void* workspace, size_t workspace_bytes, fxb_stream_t stream);
int fxb_deconv2d_f64(fxb_handle_t h, const double* dY, const double* W, double* dX, const fxb_conv2d_desc* d,
                     void* workspace, size_t workspace_bytes, fxb_stream_t stream);
int fxb_conv2d_dgrad_act_f32(fxb_handle_t h, const float* dY, const float* Y, const float* W, float* dX,
                             const fxb_conv2d_desc* d, int act, void* workspace, size_t workspace_bytes,
                             fxb_stream_t stream);
int fxb_conv2d_dgrad_act_f64(fxb_handle_t h, const double* dY, const double* Y, const double* W, double* dX,
                             const fxb_conv2d_desc* d, int act, void* workspace, size_t workspace_bytes,
                             fxb_stream_t stream);

/* ---- conv2d filter gradient: CudaOps::cross_correlation2d (src/backend/cuda/ops.rs:1544-1622),
 *      kernel `cross_correlation2d[_f64]` (kernels/convolutions.cu:279-355).  dW[K,C,R,S] from
 *      X and dY.  The fused form also applies act'(Y) to dY and returns the bias gradient
 *      db[K] = sum over N,OH,OW of dZ (the three successive axis sums of
 *      src/backend/cuda/ops.rs:2225-2281) from the same pass.  The reduction over N*OH*OW is
 *      split across CTAs; the partial sums live in `workspace` and are added in a fixed order
 *      (deterministic).  workspace may be NULL: then no split is used. ---- */
int fxb_cross_correlation2d_f32(fxb_handle_t h, const float* X, const float* dY, float* dW,
                                const fxb_conv2d_desc* d, void* workspace, size_t workspace_bytes,
                                fxb_stream_t stream);
int fxb_cross_correlation2d_f64(fxb_handle_t h, const double* X, const double* dY, double* dW,
                                const fxb_conv2d_desc* d, void* workspace, size_t workspace_bytes,
                                fxb_stream_t stream);
int fxb_conv2d_wgrad_bias_act_f32(fxb_handle_t h, const float* X, const float* dY, const float* Y, float* dW,
                                  float* db, const fxb_conv2d_desc* d, int act, void* workspace,
                                  size_t workspace_bytes, fxb_stream_t stream);
int fxb_conv2d_wgrad_bias_act_f64(fxb_handle_t h, const double* X, const double* dY, const double* Y, double* dW,
                                  double* db, const fxb_conv2d_desc* d, int act, void* workspace,
                                  size_t workspace_bytes, fxb_stream_t stream);
size_t fxb_conv2d_wgrad_workspace_bytes(fxb_handle_t h, const fxb_conv2d_desc* d, size_t elem_size);

/* ---- whole backward of a conv layer: Conv2dOp::gradient (src/ops/batched.rs:194-217) together with the
 *      activation and bias gradients around it, i.e. fxb_conv2d_wgrad_bias_act + fxb_conv2d_dgrad_act with
 *      ONE operand pass over dY (dZ = dY * act'(Y) is formed, split and laid out for both kernels at once,
 *      and the bias gradient falls out of the same pass).  Same results as the two separate calls.
 *      dX and db may be NULL.  `packed_input` (f32 only, may be NULL): the layer input already packed for
 *      the filter-gradient kernel by fxb_conv2d_bias_act_fwd_packing_f32 for the same descriptor; without
 *      it X is packed here.  Workspace: fxb_conv2d_backward_workspace_bytes. ---- */
int fxb_conv2d_backward_f32(fxb_handle_t h, const float* X, const float* dY, const float* Y, const float* W, float* dX,
                            float* dW, float* db, const fxb_conv2d_desc* d, int act, void* workspace,
                            size_t workspace_bytes, const void* packed_input, fxb_stream_t stream);
int fxb_conv2d_backward_f64(fxb_handle_t h, const double* X, const double* dY, const double* Y, const double* W,
                            double* dX, double* dW, double* db, const fxb_conv2d_desc* d, int act, void* workspace,
                            size_t workspace_bytes, const void* packed_input, fxb_stream_t stream);
size_t fxb_conv2d_backward_workspace_bytes(fxb_handle_t h, const fxb_conv2d_desc* d, size_t elem_size);
/* fxb_conv2d_bias_act_fwd_f32 whose operand pass over X also writes the packed input that the filter
 * gradient of the same layer reads (so that the backward pass need not read X again): `packed_input` must
 * hold fxb_conv2d_packed_input_bytes (256-byte aligned; 0 = this shape has no packed form) and stays valid
 * until the backward call.  *packed_written (may be NULL) tells whether it was written; when it was not,
 * pass NULL as packed_input to fxb_conv2d_backward_f32.  Y is identical to the plain forward call's. */
int fxb_conv2d_bias_act_fwd_packing_f32(fxb_handle_t h, const float* X, const float* W, const float* bias, float* Y,
                                        const fxb_conv2d_desc* d, int act, void* workspace, size_t workspace_bytes,
                                        void* packed_input, size_t packed_bytes, int* packed_written, fxb_stream_t stream);
size_t fxb_conv2d_packed_input_bytes(fxb_handle_t h, const fxb_conv2d_desc* d, size_t elem_size);
/* The same call for consecutive convolution layers (conv -> activation -> conv, src/nn/layers/conv2d.rs:197-213
 * applied twice): the f32 tensor-map kernel reads its input as hi/lo "class slabs" that an operand pass over X
 * normally writes into the workspace.  Here the producing layer writes them instead, from the registers of its
 * epilogue: with `next` (the descriptor of the layer that consumes Y) and `output_slabs` (a buffer of
 * fxb_conv2d_input_slab_bytes(next), 256-byte aligned, ZEROED ONCE by the caller: the cells of the padding ring
 * are never written) the call also leaves act(conv + bias) there; *output_slabs_written tells whether it did
 * (split-K and fallback paths do not).  The consuming layer then passes that buffer as `input_slabs` (NULL
 * otherwise) and skips its operand pass; X must still be the tensor the slabs were made from.  Y, and every
 * result computed from the slabs, are bit-identical to the unchained calls. */
int fxb_conv2d_bias_act_fwd_chain_f32(fxb_handle_t h, const float* X, const float* W, const float* bias, float* Y,
                                      const fxb_conv2d_desc* d, int act, void* workspace, size_t workspace_bytes,
                                      void* packed_input, size_t packed_bytes, int* packed_written,
                                      const void* input_slabs, const fxb_conv2d_desc* next, void* output_slabs,
                                      size_t output_slab_bytes, int* output_slabs_written, fxb_stream_t stream);
size_t fxb_conv2d_input_slab_bytes(fxb_handle_t h, const fxb_conv2d_desc* d, size_t elem_size);

/* ---- activations: CudaOps::relu/sigmoid/tanh (src/backend/cuda/ops.rs:539-558, :620-628),
 *      kernels/activations.cu:10-48.  Backward replaces the mask/mul chains of
 *      src/ops/unary.rs:254-375: dX = dY * act'(aux), aux = op input for relu, op output for
 *      sigmoid and tanh. ---- */
int fxb_act_fwd_f32(fxb_handle_t h, const float* x, float* y, int64_t n, int act, fxb_stream_t stream);
int fxb_act_fwd_f64(fxb_handle_t h, const double* x, double* y, int64_t n, int act, fxb_stream_t stream);
int fxb_act_bwd_f32(fxb_handle_t h, const float* dy, const float* aux, float* dx, int64_t n, int act,
                    fxb_stream_t stream);
int fxb_act_bwd_f64(fxb_handle_t h, const double* dy, const double* aux, double* dx, int64_t n, int act,
                    fxb_stream_t stream);

/* ---- elementwise: CudaOps::add / mul (src/backend/cuda/ops.rs:217, :244; kernels/elementwise.cu:8-38),
 *      greater_scalar (ops.rs:1052; kernels/comparison.cu:66-76), and out = alpha*x + beta*y used
 *      for gradient accumulation (src/graph/mod.rs:681-698) and gradient averaging. ---- */
int fxb_add_f32(fxb_handle_t h, const float* a, const float* b, float* out, int64_t n, fxb_stream_t stream);
int fxb_add_f64(fxb_handle_t h, const double* a, const double* b, double* out, int64_t n, fxb_stream_t stream);
int fxb_mul_f32(fxb_handle_t h, const float* a, const float* b, float* out, int64_t n, fxb_stream_t stream);
int fxb_mul_f64(fxb_handle_t h, const double* a, const double* b, double* out, int64_t n, fxb_stream_t stream);
int fxb_axpby_f32(fxb_handle_t h, float alpha, const float* x, float beta, const float* y, float* out, int64_t n,
                  fxb_stream_t stream);
int fxb_axpby_f64(fxb_handle_t h, double alpha, const double* x, double beta, const double* y, double* out,
                  int64_t n, fxb_stream_t stream);
int fxb_greater_scalar_f32(fxb_handle_t h, const float* x, float s, float* out, int64_t n, fxb_stream_t stream);
int fxb_greater_scalar_f64(fxb_handle_t h, const double* x, double s, double* out, int64_t n, fxb_stream_t stream);
/* Bias add as its own op (broadcast + Add): y[n,k,p] += bias[k]; plane = OH*OW (1 for linear). */
int fxb_bias_add_f32(fxb_handle_t h, float* y, const float* bias, int64_t outer, int64_t channels, int64_t plane,
                     fxb_stream_t stream);
int fxb_bias_add_f64(fxb_handle_t h, double* y, const double* bias, int64_t outer, int64_t channels, int64_t plane,
                     fxb_stream_t stream);

/* ---- reductions: CudaOps::sum_axes / sum_all (src/backend/cuda/ops.rs:653-697, :2171-2284),
 *      kernels `reduce_sum_axes`, `reduce_sum_all` (kernels/reduction.cu:9-84).  `axes` lists the
 *      reduced axes (any order); the output holds the kept axes in order (keep_dims only
 *      changes the shape on the caller's side).  Up to 8-D inputs; two-stage and deterministic
 *      (more than two separate runs of reduced axes take a second round through the workspace).
 *      The partial sums of stage one live in `workspace`. ---- */
int fxb_sum_axes_f32(fxb_handle_t h, const float* x, const int64_t* shape, int ndim, const int* axes, int naxes,
                     float* out, void* workspace, size_t workspace_bytes, fxb_stream_t stream);
int fxb_sum_axes_f64(fxb_handle_t h, const double* x, const int64_t* shape, int ndim, const int* axes, int naxes,
                     double* out, void* workspace, size_t workspace_bytes, fxb_stream_t stream);
size_t fxb_sum_axes_workspace_bytes(fxb_handle_t h, const int64_t* shape, int ndim, const int* axes, int naxes,
                                    size_t elem_size);
/* No counterpart in the reference.  fxb_sum_axes_f32 for callers that cannot allocate a workspace
 * at the moment they need the sum: code running while the memory pool's mutex is held (a Drop
 * handler, the pool's eviction path) and out-of-memory handlers that still want a loss or
 * gradient-norm value after the pool refused a request; cudaMalloc is no way out there (it
 * synchronises the device and may fail for the same reason).  The stage-one partial sums live in a
 * 512 KiB device array that is part of the library image (held by every GPU that loads the library
 * until exit); nothing is allocated or freed.  Reductions whose partial sums exceed 512 KiB return
 * FXB_ERR_WORKSPACE.  fxb_create resolves the array's device address (cudaGetSymbolAddress with the
 * handle's device current), so a call here never reaches the module loader; create the handle before
 * any stream capture.  All calls on a device share the array: calls that overlap on the GPU race;
 * nothing needs clearing between calls.  Results are bit-identical to fxb_sum_axes_f32. */
int fxb_sum_axes_static_scratch_f32(fxb_handle_t h, const float* x, const int64_t* shape, int ndim, const int* axes,
                                    int naxes, float* out, fxb_stream_t stream);
int fxb_sum_all_f32(fxb_handle_t h, const float* x, int64_t n, float* out, void* workspace, size_t workspace_bytes,
                    fxb_stream_t stream);
int fxb_sum_all_f64(fxb_handle_t h, const double* x, int64_t n, double* out, void* workspace,
                    size_t workspace_bytes, fxb_stream_t stream);

/* ---- layout: CudaOps::materialize (src/backend/cuda/ops.rs:175-214), kernel `materialize[_f64]`
 *      (kernels/materialize.cu:25-46): out (contiguous, `shape`) = the view of `in` with element
 *      strides `strides` (0 = a broadcast dimension).  Shape and strides travel in the launch
 *      parameters (the reference copies both arrays to the device on every call).  Up to 8-D,
 *      fewer than 2^31 elements.  Pure data movement: bit-exact. ---- */
int fxb_materialize_f32(fxb_handle_t h, const float* in, float* out, const int64_t* shape, const int64_t* strides,
                        int ndim, fxb_stream_t stream);
int fxb_materialize_f64(fxb_handle_t h, const double* in, double* out, const int64_t* shape, const int64_t* strides,
                        int ndim, fxb_stream_t stream);
/* Transpose as its own op: Tensor::transpose + materialize (src/ops/matrix.rs:69-110,
 * src/backend/storage/cuda.rs:826-857).  `in` is contiguous with `shape`; out[i0..] = in permuted so
 * that output axis i is input axis axes[i]; axes == NULL reverses all axes (the matrix transpose). */
int fxb_transpose_f32(fxb_handle_t h, const float* in, float* out, const int64_t* shape, int ndim, const int* axes,
                      fxb_stream_t stream);
int fxb_transpose_f64(fxb_handle_t h, const double* in, double* out, const int64_t* shape, int ndim, const int* axes,
                      fxb_stream_t stream);
/* broadcast_to + materialize (src/backend/storage/cuda.rs:795-803, src/ops/reshape.rs:26-41): shapes are
 * aligned at the last axis; an input extent must equal the target's or be 1. */
int fxb_broadcast_to_f32(fxb_handle_t h, const float* in, const int64_t* in_shape, int in_ndim, float* out,
                         const int64_t* out_shape, int out_ndim, fxb_stream_t stream);
int fxb_broadcast_to_f64(fxb_handle_t h, const double* in, const int64_t* in_shape, int in_ndim, double* out,
                         const int64_t* out_shape, int out_ndim, fxb_stream_t stream);

/* ---- batch normalisation: BatchNorm::forward (src/nn/layers/norm.rs:214-331) and the gradients its
 *      graph ops chain (Mean, Sub, Mul, Sqrt, Div, BroadcastTo: src/ops/reduction.rs:156-196,
 *      src/ops/basic.rs:187-263, src/ops/unary.rs:123-143), fused.  x is [N, C, P] with P = H*W
 *      (P = 1 for a [N, F] input).  Training: batch_mean / batch_var (biased, as the reference
 *      computes it) are outputs and the running statistics, when given, are updated in place with
 *      running = (1 - momentum) * running + momentum * batch (norm.rs:126-163).  Inference
 *      (training == 0): the running statistics normalise, no workspace is needed.
 *      y = act(((x - mean) / sqrt(var + eps)) * gamma + beta); gamma / beta may be NULL (1 / 0).
 *      Backward: dZ = dY * act'(Y); dbeta = sum dZ, dgamma = sum dZ * xhat,
 *      dX = (gamma / std) * (dZ - dbeta / M - xhat * dgamma / M); dX may be NULL. ---- */
int fxb_batch_norm_fwd_f32(fxb_handle_t h, const float* x, const float* gamma, const float* beta, float* y,
                           float* batch_mean, float* batch_var, float* running_mean, float* running_var, int64_t N,
                           int64_t C, int64_t P, double eps, double momentum, int training, int act, void* workspace,
                           size_t workspace_bytes, fxb_stream_t stream);
int fxb_batch_norm_fwd_f64(fxb_handle_t h, const double* x, const double* gamma, const double* beta, double* y,
                           double* batch_mean, double* batch_var, double* running_mean, double* running_var, int64_t N,
                           int64_t C, int64_t P, double eps, double momentum, int training, int act, void* workspace,
                           size_t workspace_bytes, fxb_stream_t stream);
int fxb_batch_norm_bwd_f32(fxb_handle_t h, const float* x, const float* dy, const float* y, const float* gamma,
                           const float* batch_mean, const float* batch_var, float* dx, float* dgamma, float* dbeta,
                           int64_t N, int64_t C, int64_t P, double eps, int act, void* workspace, size_t workspace_bytes,
                           fxb_stream_t stream);
int fxb_batch_norm_bwd_f64(fxb_handle_t h, const double* x, const double* dy, const double* y, const double* gamma,
                           const double* batch_mean, const double* batch_var, double* dx, double* dgamma, double* dbeta,
                           int64_t N, int64_t C, int64_t P, double eps, int act, void* workspace, size_t workspace_bytes,
                           fxb_stream_t stream);
size_t fxb_batch_norm_workspace_bytes(fxb_handle_t h, int64_t N, int64_t C, int64_t P, size_t elem_size);

/* ---- global average pooling: GlobalAvgPool2d::forward = Mean over axes [2, 3]
 *      (src/nn/layers/pooling.rs:604-619) and Mean::gradient (src/ops/reduction.rs:170-196):
 *      y[N, C] = sum over H*W * (1 / (H*W));  dx[n, c, :, :] = dy[n, c] * (1 / (H*W)). ---- */
int fxb_global_avg_pool_fwd_f32(fxb_handle_t h, const float* x, float* y, int64_t N, int64_t C, int64_t H, int64_t W,
                                fxb_stream_t stream);
int fxb_global_avg_pool_fwd_f64(fxb_handle_t h, const double* x, double* y, int64_t N, int64_t C, int64_t H, int64_t W,
                                fxb_stream_t stream);
int fxb_global_avg_pool_bwd_f32(fxb_handle_t h, const float* dy, float* dx, int64_t N, int64_t C, int64_t H, int64_t W,
                                fxb_stream_t stream);
int fxb_global_avg_pool_bwd_f64(fxb_handle_t h, const double* dy, double* dx, int64_t N, int64_t C, int64_t H, int64_t W,
                                fxb_stream_t stream);

/* ---- loss and optimizers (the callers right after / before the path inside a train step).
 *      Softmax cross-entropy with mean reduction, forward and gradient in one kernel:
 *      CCELoss::forward (src/nn/losses/classification.rs:191-257) and the operator gradients it
 *      chains (src/ops/batched.rs:106-131, src/ops/comparison.rs:270-289).  targets are one-hot
 *      (or soft) [B,C].  loss_out: one element on the device.  dlogits may be NULL.
 *      grad_scale multiplies dlogits (1 for a single device; used for sharded batches). ---- */
int fxb_softmax_ce_f32(fxb_handle_t h, const float* logits, const float* targets, float* loss_out, float* dlogits,
                       int64_t B, int64_t C, float grad_scale, fxb_stream_t stream);
int fxb_softmax_ce_f64(fxb_handle_t h, const double* logits, const double* targets, double* loss_out,
                       double* dlogits, int64_t B, int64_t C, double grad_scale, fxb_stream_t stream);
/* SGD::step (src/nn/optim/sgd.rs:117-245).  mom may be NULL when momentum == 0.
 * grad_scale multiplies g first (1/world_size after a gradient all-reduce). */
int fxb_sgd_step_f32(fxb_handle_t h, float* p, const float* g, float* mom, int64_t n, float lr, float momentum,
                     float weight_decay, int nesterov, float grad_scale, fxb_stream_t stream);
int fxb_sgd_step_f64(fxb_handle_t h, double* p, const double* g, double* mom, int64_t n, double lr,
                     double momentum, double weight_decay, int nesterov, double grad_scale, fxb_stream_t stream);
/* Adam::step (src/nn/optim/adam.rs:110-126, :136-210, :230-358); step is the 1-based count. */
int fxb_adam_step_f32(fxb_handle_t h, float* p, const float* g, float* m, float* v, int64_t n, float lr,
                      float beta1, float beta2, float eps, float weight_decay, int64_t step, float grad_scale,
                      fxb_stream_t stream);
int fxb_adam_step_f64(fxb_handle_t h, double* p, const double* g, double* m, double* v, int64_t n, double lr,
                      double beta1, double beta2, double eps, double weight_decay, int64_t step,
                      double grad_scale, fxb_stream_t stream);

/* The same update with the step count kept in device memory (*step_dev = steps done so far; the update
 * uses *step_dev + 1 and the call advances the counter), so that a train step captured once in a CUDA
 * graph can be replayed: kernel arguments are frozen at capture, the bias corrections are not. */
int fxb_adam_step_devcount_f32(fxb_handle_t h, float* p, const float* g, float* m, float* v, int64_t n, float lr,
                               float beta1, float beta2, float eps, float weight_decay, int64_t* step_dev,
                               float grad_scale, fxb_stream_t stream);
int fxb_adam_step_devcount_f64(fxb_handle_t h, double* p, const double* g, double* m, double* v, int64_t n, double lr,
                               double beta1, double beta2, double eps, double weight_decay, int64_t* step_dev,
                               double grad_scale, fxb_stream_t stream);

/* ---- sequential conv/linear network train step: the host-side sequence that Ferrox's layers,
 *      graph and loss issue for one step (examples/common/training.rs:33-81;
 *      src/nn/layers/conv2d.rs:168-214, linear.rs:183-279; src/graph/mod.rs:700-783), expressed
 *      with the fused entry points above.  All memory is the caller's: parameters and gradients
 *      are two flat buffers (per layer: weight then bias, layers in order, so the gradients of
 *      the last layers form a contiguous tail that can be all-reduced while the first layers
 *      are still in backward), activations and scratch live in one arena. ---- */
#define FXB_LAYER_CONV 0
#define FXB_LAYER_FLATTEN 1
#define FXB_LAYER_LINEAR 2

typedef struct fxb_layer_desc {
    int32_t kind;          /* FXB_LAYER_* */
    int32_t act;           /* FXB_ACT_* applied to the layer output */
    int64_t out_channels;  /* conv: K; linear: out_features */
    int64_t kernel;        /* conv: R = S */
    int64_t stride, pad;   /* conv */
} fxb_layer_desc;

typedef struct fxb_net* fxb_net_t;

/* elem_size 4 (f32) or 8 (f64); input is [batch, in_c, in_h, in_w] (in_h = in_w = 1 and
 * in_c = features for a plain MLP); the last layer must produce [batch, classes]. */
int fxb_net_create(fxb_handle_t h, size_t elem_size, const fxb_layer_desc* layers, int nlayers, int64_t batch,
                   int64_t in_c, int64_t in_h, int64_t in_w, fxb_net_t* out);
int fxb_net_destroy(fxb_net_t net);
int64_t fxb_net_param_count(fxb_net_t net);                 /* elements in the flat parameter buffer */
int fxb_net_param_layers(fxb_net_t net);                    /* number of layers that own parameters */
/* Offsets (in elements) of parameter layer i inside the flat buffer: weight, bias, end. */
int fxb_net_param_offsets(fxb_net_t net, int i, int64_t* weight_off, int64_t* bias_off, int64_t* end_off);
size_t fxb_net_arena_bytes(fxb_net_t net);
int64_t fxb_net_num_classes(fxb_net_t net);
int fxb_net_bind(fxb_net_t net, void* params, void* grads, void* arena, size_t arena_bytes);
/* Forward pass; logits_out (optional) receives the device pointer of the [batch, classes] logits. */
int fxb_net_forward(fxb_net_t net, const void* x, void** logits_out, fxb_stream_t stream);
/* Softmax cross-entropy (mean over this batch) on the logits of the last forward: writes the
 * loss to loss_out (device, one element) and seeds the backward pass.  grad_scale multiplies
 * the seed (1/world_size when the global mean is taken over several shards). */
int fxb_net_loss(fxb_net_t net, const void* targets_onehot, void* loss_out, double grad_scale, fxb_stream_t stream);
/* Backward for parameter layers [first, last] (inclusive, indices as in fxb_net_param_offsets),
 * which must be called from the last layer towards the first, e.g. (nl-1 .. 2) then (1 .. 0). */
int fxb_net_backward_range(fxb_net_t net, const void* x, int last, int first, fxb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* FERROX_B200_H */
