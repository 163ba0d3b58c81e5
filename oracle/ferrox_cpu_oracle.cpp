// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// Single-threaded C++ restatement of the reference (RaulMoldes/ferrox) CPU storage path for
// the conv2d / linear training hot path.  It exists to check the CUDA library and to be the
// timed CPU baseline; nothing in the shipped library links, loads or calls it.
//
// The reference's contractions go through ndarray 0.16.1 `ArrayBase::dot`, which calls
// matrixmultiply 0.3.10 (Cargo.lock:163-174); neither crate is vendored in the reference, so
// the GEMM here is a plain register-blocked triple loop that the compiler vectorises (any f32
// summation order is inside the parity tolerance; a hand-tuned SIMD micro-kernel like
// matrixmultiply's is still somewhat faster).  Everything else follows the reference line by line; each function cites
// the file:line it restates (paths relative to the reference repository root).
//
// Parity pinning: checked against the reference's own known-answer tests (tests/golden/),
// which pin forward values only.  Gradient values of matmul/conv/activations are NOT pinned
// by any reference test ("parity unpinned" for those); they are cross-checked against an
// independent f64 autograd in the test-suite instead.
//
// Conv-gradient modes: the reference's deconv2d_impl / cross_correlation2d_impl reinterpret
// NCHW grad_output as [OC, B*H*W] without a transpose, which is only right at batch 1.
//   mode 0 ("literal")    : the reference code verbatim for any batch.
//   mode 1 ("per-sample") : the same algorithm applied to each sample alone, dX concatenated
//                           and dW summed in sample order; this equals the true gradient and
//                           the reference's CUDA kernels and is the parity contract.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#include <algorithm>

namespace {

// ---------------------------------------------------------------------------------------
// C[M,N] = A[M,K] . B[K,N], all row-major contiguous.
// Call sites restated: src/backend/storage/cpu.rs:967-1002 (matmul, `a.dot(&b)` at :999),
// src/backend/storage/extensions/convolutions.rs:256, :296, :332.
template <typename T>
void gemm_nn(const T* A, const T* B, T* C, int64_t M, int64_t N, int64_t K) {
    // Register-blocked: a 4 x 32 block of C is accumulated over one k-panel in local variables (the
    // compiler keeps them in vector registers), so every loaded B value feeds four rows.  Per output
    // element the products are added in ascending k inside a panel and the panels in ascending order.
    std::fill(C, C + M * N, T(0));
    constexpr int64_t KB = 256, MR = 4, NR = 32;
    for (int64_t k0 = 0; k0 < K; k0 += KB) {
        const int64_t k1 = std::min(K, k0 + KB);
        int64_t i = 0;
        for (; i + MR <= M; i += MR) {
            int64_t j = 0;
            for (; j + NR <= N; j += NR) {
                T acc[MR][NR];
                for (int64_t r = 0; r < MR; ++r)
                    for (int64_t c = 0; c < NR; ++c) acc[r][c] = T(0);
                for (int64_t k = k0; k < k1; ++k) {
                    const T* b = B + k * N + j;
                    const T a0 = A[(i + 0) * K + k], a1 = A[(i + 1) * K + k], a2 = A[(i + 2) * K + k], a3 = A[(i + 3) * K + k];
                    for (int64_t c = 0; c < NR; ++c) {
                        const T bv = b[c];
                        acc[0][c] += a0 * bv;
                        acc[1][c] += a1 * bv;
                        acc[2][c] += a2 * bv;
                        acc[3][c] += a3 * bv;
                    }
                }
                for (int64_t r = 0; r < MR; ++r)
                    for (int64_t c = 0; c < NR; ++c) C[(i + r) * N + j + c] += acc[r][c];
            }
            for (; j < N; ++j)
                for (int64_t r = 0; r < MR; ++r) {
                    T s = T(0);
                    for (int64_t k = k0; k < k1; ++k) s += A[(i + r) * K + k] * B[k * N + j];
                    C[(i + r) * N + j] += s;
                }
        }
        for (; i < M; ++i) {
            T* c = C + i * N;
            for (int64_t k = k0; k < k1; ++k) {
                const T a = A[i * K + k];
                const T* b = B + k * N;
                for (int64_t j = 0; j < N; ++j) c[j] += a * b[j];
            }
        }
    }
}

// Materialised transpose: the reference transposes by permuting axes and copying
// (`permuted_axes().to_owned()`, src/backend/storage/cpu.rs:543-562).
template <typename T>
void transpose2d(const T* A, T* At, int64_t R, int64_t Cc) {
    for (int64_t i = 0; i < R; ++i)
        for (int64_t j = 0; j < Cc; ++j) At[j * R + i] = A[i * Cc + j];
}

// ---------------------------------------------------------------------------------------
// im2col — src/backend/storage/extensions/convolutions.rs:10-75.
// col is [C*kh*kw, B*oh*ow]; zero where the tap falls in the padding (:50-54).
template <typename T>
void im2col(const T* x, int64_t B, int64_t C, int64_t H, int64_t W, int64_t kh, int64_t kw,
            int64_t sh, int64_t sw, int64_t ph, int64_t pw, T* col) {
    const int64_t oh = (H + 2 * ph - kh) / sh + 1;
    const int64_t ow = (W + 2 * pw - kw) / sw + 1;
    const int64_t colw = B * oh * ow;
    std::fill(col, col + C * kh * kw * colw, T(0));
    for (int64_t b = 0; b < B; ++b)
        for (int64_t c = 0; c < C; ++c)
            for (int64_t ky = 0; ky < kh; ++ky)
                for (int64_t kx = 0; kx < kw; ++kx) {
                    const int64_t row = c * kh * kw + ky * kw + kx;
                    for (int64_t oy = 0; oy < oh; ++oy)
                        for (int64_t ox = 0; ox < ow; ++ox) {
                            const int64_t iy = oy * sh + ky, ix = ox * sw + kx;
                            if (iy >= ph && iy < H + ph && ix >= pw && ix < W + pw) {
                                const int64_t ay = iy - ph, ax = ix - pw;
                                col[row * colw + b * oh * ow + oy * ow + ox] =
                                    x[b * C * H * W + c * H * W + ay * W + ax];
                            }
                        }
                }
}

// conv2d forward — convolutions.rs:218-265: im2col, filter as [OC, C*kh*kw], dot, then
// transpose_conv_output (:156-185) from [OC, B*oh*ow] to [B, OC, oh, ow].  No bias.
template <typename T>
void conv2d_fwd(const T* x, const T* w, T* y, int64_t B, int64_t C, int64_t H, int64_t W,
                int64_t OC, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph,
                int64_t pw) {
    const int64_t oh = (H + 2 * ph - kh) / sh + 1;
    const int64_t ow = (W + 2 * pw - kw) / sw + 1;
    const int64_t colh = C * kh * kw, colw = B * oh * ow;
    std::vector<T> col(colh * colw), col2(colh * colw), out2d(OC * colw);
    im2col(x, B, C, H, W, kh, kw, sh, sw, ph, pw, col.data());
    std::memcpy(col2.data(), col.data(), sizeof(T) * col.size());  // safe_reshape_to_2d copy (:188-195)
    gemm_nn(w, col2.data(), out2d.data(), OC, colw, colh);
    for (int64_t oc = 0; oc < OC; ++oc)
        for (int64_t b = 0; b < B; ++b)
            for (int64_t p = 0; p < oh * ow; ++p)
                y[b * OC * oh * ow + oc * oh * ow + p] = out2d[oc * colw + b * oh * ow + p];
}

// col2im — convolutions.rs:79-153.  The flat index (:122-127) treats the column matrix as
// [B, C, kh, kw, col_h, col_w]; accumulation into a padded image, then the centre is cropped.
template <typename T>
void col2im(const T* colflat, int64_t colsize, T* out, int64_t B, int64_t C, int64_t H, int64_t W,
            int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw) {
    const int64_t PH = H + 2 * ph, PW = W + 2 * pw;
    const int64_t ch = (PH - kh) / sh + 1, cw = (PW - kw) / sw + 1;
    std::vector<T> pad(B * C * PH * PW, T(0));
    for (int64_t b = 0; b < B; ++b)
        for (int64_t c = 0; c < C; ++c)
            for (int64_t ky = 0; ky < kh; ++ky)
                for (int64_t kx = 0; kx < kw; ++kx)
                    for (int64_t cy = 0; cy < ch; ++cy)
                        for (int64_t cx = 0; cx < cw; ++cx) {
                            const int64_t iy = cy * sh + ky, ix = cx * sw + kx;
                            const int64_t idx = b * (C * kh * kw * ch * cw) + c * (kh * kw * ch * cw) +
                                                ky * (kw * ch * cw) + kx * (ch * cw) + cy * cw + cx;
                            if (idx < colsize) pad[((b * C + c) * PH + iy) * PW + ix] += colflat[idx];
                        }
    for (int64_t b = 0; b < B; ++b)
        for (int64_t c = 0; c < C; ++c)
            for (int64_t h = 0; h < H; ++h)
                for (int64_t ww = 0; ww < W; ++ww)
                    out[((b * C + c) * H + h) * W + ww] = pad[((b * C + c) * PH + h + ph) * PW + ww + pw];
}

// deconv2d (dX) literal — convolutions.rs:268-307: grad reinterpreted as [OC, B*gh*gw]
// (:292-293), col = filter_2d^T . grad_2d (:296), col2im.
template <typename T>
void deconv2d_literal(const T* dy, const T* w, T* dx, int64_t B, int64_t C, int64_t H, int64_t W,
                      int64_t OC, int64_t kh, int64_t kw, int64_t gh, int64_t gw, int64_t sh,
                      int64_t sw, int64_t ph, int64_t pw) {
    const int64_t ckk = C * kh * kw, n = B * gh * gw;
    std::vector<T> wt(ckk * OC), col(ckk * n);
    transpose2d(w, wt.data(), OC, ckk);
    gemm_nn(wt.data(), dy, col.data(), ckk, n, OC);
    col2im(col.data(), ckk * n, dx, B, C, H, W, kh, kw, sh, sw, ph, pw);
}

// cross_correlation2d (dW) literal — convolutions.rs:310-338: im2col of the input with the
// filter's spatial size, grad reinterpreted as [OC, B*gh*gw] (:323-326), grad_2d . col^T (:332).
template <typename T>
void xcorr2d_literal(const T* x, const T* dy, T* dw, int64_t B, int64_t C, int64_t H, int64_t W,
                     int64_t OC, int64_t kh, int64_t kw, int64_t gh, int64_t gw, int64_t sh,
                     int64_t sw, int64_t ph, int64_t pw) {
    const int64_t oh = (H + 2 * ph - kh) / sh + 1, ow = (W + 2 * pw - kw) / sw + 1;
    const int64_t ckk = C * kh * kw, n = B * oh * ow;
    (void)gh; (void)gw;
    std::vector<T> col(ckk * n), colt(n * ckk);
    im2col(x, B, C, H, W, kh, kw, sh, sw, ph, pw, col.data());
    transpose2d(col.data(), colt.data(), ckk, n);
    gemm_nn(dy, colt.data(), dw, OC, ckk, n);
}

template <typename T>
void deconv2d(const T* dy, const T* w, T* dx, int64_t B, int64_t C, int64_t H, int64_t W, int64_t OC,
              int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int mode) {
    const int64_t gh = (H + 2 * ph - kh) / sh + 1, gw = (W + 2 * pw - kw) / sw + 1;
    if (mode == 0) {
        deconv2d_literal(dy, w, dx, B, C, H, W, OC, kh, kw, gh, gw, sh, sw, ph, pw);
        return;
    }
    for (int64_t b = 0; b < B; ++b)
        deconv2d_literal(dy + b * OC * gh * gw, w, dx + b * C * H * W, 1, C, H, W, OC, kh, kw, gh, gw,
                         sh, sw, ph, pw);
}

template <typename T>
void xcorr2d(const T* x, const T* dy, T* dw, int64_t B, int64_t C, int64_t H, int64_t W, int64_t OC,
             int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int mode) {
    const int64_t gh = (H + 2 * ph - kh) / sh + 1, gw = (W + 2 * pw - kw) / sw + 1;
    if (mode == 0) {
        xcorr2d_literal(x, dy, dw, B, C, H, W, OC, kh, kw, gh, gw, sh, sw, ph, pw);
        return;
    }
    const int64_t wn = OC * C * kh * kw;
    std::vector<T> part(wn);
    std::fill(dw, dw + wn, T(0));
    for (int64_t b = 0; b < B; ++b) {
        xcorr2d_literal(x + b * C * H * W, dy + b * OC * gh * gw, part.data(), 1, C, H, W, OC, kh, kw,
                        gh, gw, sh, sw, ph, pw);
        for (int64_t i = 0; i < wn; ++i) dw[i] += part[i];
    }
}

// ---------------------------------------------------------------------------------------
// Activations.  relu: cpu.rs:1070-1082 (strict >).  sigmoid: cpu.rs:1004-1016.
// tanh: cpu.rs:1102-1150 (clamped at |x|>20, exp(-2x)/exp(2x) forms).
template <typename T> T relu1(T x) { return x > T(0) ? x : T(0); }
template <typename T> T sigmoid1(T x) { return T(1) / (T(1) + std::exp(-x)); }
template <typename T> T tanh1(T x) {
    if (x > T(20)) return T(1);
    if (x < T(-20)) return T(-1);
    if (x >= T(0)) {
        const T e = std::exp(-x * T(2));
        const T den = T(1) + e;
        return den == T(0) ? T(1) : (T(1) - e) / den;
    }
    const T e = std::exp(x * T(2));
    const T den = e + T(1);
    return den == T(0) ? T(-1) : (e - T(1)) / den;
}

// act codes shared with the CUDA library: 0 none, 1 relu, 2 sigmoid, 3 tanh.
template <typename T>
void act_fwd(const T* x, T* y, int64_t n, int act) {
    for (int64_t i = 0; i < n; ++i)
        y[i] = act == 1 ? relu1(x[i]) : act == 2 ? sigmoid1(x[i]) : act == 3 ? tanh1(x[i]) : x[i];
}

// Backward rules of the autograd operators.
//  relu   : mask = greater_scalar(input, 0) (cpu.rs:876-885); dY*mask   — src/ops/unary.rs:358-375
//  sigmoid: (out - 1) then out*(out-1) then dY*that                     — src/ops/unary.rs:254-276
//           (this is the reference's literal rule: s*(s-1), the negative of the derivative;
//            sigmoid_math=1 gives s*(1-s) instead)
//  tanh   : -((out*out) - 1) then dY*that                               — src/ops/unary.rs:306-328
// `aux` is the op INPUT for relu and the cached op OUTPUT for sigmoid/tanh.
template <typename T>
void act_bwd(const T* dy, const T* aux, T* dx, int64_t n, int act, int sigmoid_math) {
    for (int64_t i = 0; i < n; ++i) {
        const T a = aux[i];
        if (act == 1) dx[i] = dy[i] * (a > T(0) ? T(1) : T(0));
        else if (act == 2) dx[i] = sigmoid_math ? dy[i] * (a * (T(1) - a)) : dy[i] * (a * (a - T(1)));
        else if (act == 3) dx[i] = dy[i] * (-(a * a - T(1)));
        else dx[i] = dy[i];
    }
}

// ---------------------------------------------------------------------------------------
// sum over axes — cpu.rs:60-130 + :1183-1191: axes sorted descending, deduplicated, then one
// `sum_axis` per axis on the running result.  shape has ndim entries; reduce[i] != 0 marks
// axis i as reduced.  Output is the kept axes in order (keep_dims only changes the shape).
template <typename T>
void sum_axes(const T* x, const int64_t* shape, int ndim, const int* reduce, T* out) {
    std::vector<int64_t> shp(shape, shape + ndim);
    int64_t total = 1;
    for (int i = 0; i < ndim; ++i) total *= shp[i];
    std::vector<T> cur(x, x + total);
    for (int ax = ndim - 1; ax >= 0; --ax) {
        if (!reduce[ax]) continue;
        int64_t outer = 1, inner = 1;
        for (int i = 0; i < ax; ++i) outer *= shp[i];
        for (int i = ax + 1; i < (int)shp.size(); ++i) inner *= shp[i];
        const int64_t len = shp[ax];
        std::vector<T> nxt(outer * inner, T(0));
        for (int64_t o = 0; o < outer; ++o)
            for (int64_t r = 0; r < len; ++r) {
                const T* src = cur.data() + (o * len + r) * inner;
                T* dst = nxt.data() + o * inner;
                for (int64_t i = 0; i < inner; ++i) dst[i] += src[i];
            }
        shp[ax] = 1;
        cur.swap(nxt);
    }
    int64_t n = 1;
    for (auto s : shp) n *= s;
    std::memcpy(out, cur.data(), sizeof(T) * n);
}

// ---------------------------------------------------------------------------------------
// Layers as the reference composes them.
// Linear forward — src/nn/layers/linear.rs:183-279: Transpose(W[out,in]) materialised,
// MatMul(x, Wt), bias broadcast to [B,out] then Add.
template <typename T>
void linear_fwd(const T* x, const T* w, const T* bias, T* y, int64_t B, int64_t in, int64_t out) {
    std::vector<T> wt(in * out);
    transpose2d(w, wt.data(), out, in);
    gemm_nn(x, wt.data(), y, B, out, in);
    if (bias)
        for (int64_t i = 0; i < B; ++i)
            for (int64_t j = 0; j < out; ++j) y[i * out + j] += bias[j];
}

// Linear backward — MatMul::gradient src/ops/matrix.rs:30-55 (dA = dC.B^T, dB = A^T.dC with
// materialised transposes), Transpose::gradient (:88-110) brings dWt back to [out,in],
// bias: Add::gradient -> reduce_gradient_for_broadcasting -> sum(axes=[0])
// (src/ops/basic.rs:10-53, :95-115; src/ops/reshape.rs:82-99).
template <typename T>
void linear_bwd(const T* x, const T* w, const T* dz, T* dx, T* dw, T* db, int64_t B, int64_t in,
                int64_t out) {
    if (dx) gemm_nn(dz, w, dx, B, in, out);  // dZ . (Wt)^T = dZ . W
    if (dw) {
        std::vector<T> xt(in * B), dwt(in * out);
        transpose2d(x, xt.data(), B, in);
        gemm_nn(xt.data(), dz, dwt.data(), in, out, B);  // dWt = x^T . dZ
        transpose2d(dwt.data(), dw, in, out);
    }
    if (db) {
        const int64_t shape[2] = {B, out};
        const int red[2] = {1, 0};
        sum_axes(dz, shape, 2, red, db);
    }
}

// Conv bias add — src/nn/layers/utils.rs:6-42 + conv2d.rs:203-208: bias [K] reshaped to
// [1,K,1,1], broadcast to the activation shape, added.
template <typename T>
void conv_bias_add(T* y, const T* bias, int64_t B, int64_t K, int64_t P) {
    for (int64_t b = 0; b < B; ++b)
        for (int64_t k = 0; k < K; ++k)
            for (int64_t p = 0; p < P; ++p) y[(b * K + k) * P + p] += bias[k];
}

// ---------------------------------------------------------------------------------------
// Softmax cross-entropy with mean reduction — src/nn/losses/classification.rs:191-257:
// softmax(axis 1) (cpu.rs:1034-1068) -> clamp [1e-8, 1-1e-8] (cpu.rs:792-805) -> log ->
// * targets -> sum axis 1 keep_dims -> neg -> mean.  Backward composed from the operator rules:
// Mean (src/ops/reduction.rs:156-196), Neg, Sum (broadcast back), Mul (dL * targets for the
// log branch), Log (grad / input, src/ops/unary.rs:76-101), Clamp mask on the softmax output
// (src/ops/comparison.rs:270-289), Softmax batch gradient (src/ops/batched.rs:106-131).
// Returns the loss; dlogits may be null.
template <typename T>
T softmax_ce(const T* logits, const T* targets, T* dlogits, int64_t B, int64_t Cn) {
    const T eps = T(1e-8), one_m = T(1.0 - 1e-8);
    std::vector<T> p(Cn), pc(Cn), g(Cn);
    const T scale = T(1.0 / double(B));
    T total = T(0);
    for (int64_t i = 0; i < B; ++i) {
        const T* z = logits + i * Cn;
        T mx = std::numeric_limits<T>::lowest();
        for (int64_t j = 0; j < Cn; ++j) if (z[j] > mx) mx = z[j];
        T s = T(0);
        for (int64_t j = 0; j < Cn; ++j) { p[j] = std::exp(z[j] - mx); s += p[j]; }
        T row = T(0);
        for (int64_t j = 0; j < Cn; ++j) {
            p[j] = p[j] / s;
            pc[j] = p[j] < eps ? eps : (p[j] > one_m ? one_m : p[j]);
            row += targets[i * Cn + j] * std::log(pc[j]);
        }
        total += -row;
        if (dlogits) {
            // d(loss)/d(per-sample) = 1/B; Neg -> -1/B; Sum/broadcast; Mul by targets;
            // Log: / clamped p; Clamp: mask (p >= eps)&(p <= 1-eps); Softmax: p*(g - sum(g*p)).
            T dot = T(0);
            for (int64_t j = 0; j < Cn; ++j) {
                T gj = (-scale) * targets[i * Cn + j];
                gj = gj / pc[j];
                const T mask = (p[j] >= eps ? T(1) : T(0)) * (p[j] <= one_m ? T(1) : T(0));
                g[j] = gj * mask;
                dot += g[j] * p[j];
            }
            for (int64_t j = 0; j < Cn; ++j) dlogits[i * Cn + j] = p[j] * (g[j] - dot);
        }
    }
    return total * scale;  // mean = sum * (1/len) (cpu.rs:1193-1221)
}

// ---------------------------------------------------------------------------------------
// SGD step — src/nn/optim/sgd.rs:117-245 (weight decay folded into the gradient, optional
// momentum / nesterov buffers, p - lr*update).
template <typename T>
void sgd_step(T* p, const T* g, T* mom, int64_t n, T lr, T momentum, T wd, int nesterov) {
    for (int64_t i = 0; i < n; ++i) {
        T eg = wd == T(0) ? g[i] : g[i] + p[i] * wd;
        if (momentum != T(0)) {
            mom[i] = mom[i] * momentum + eg;
            const T upd = nesterov ? mom[i] * momentum + eg : mom[i];
            p[i] = p[i] - upd * lr;
        } else {
            p[i] = p[i] - eg * lr;
        }
    }
}

// Adam step — src/nn/optim/adam.rs:110-126 (bias corrections 1 - max(beta^t, 1e-8)),
// :136-210 (moment updates), :230-282 (update = m/bc1 / (sqrt(v/bc2)+eps) * lr, decoupled
// weight decay), :288-358.  `step` is the 1-based step count after the increment at :289.
template <typename T>
void adam_step(T* p, const T* g, T* m, T* v, int64_t n, T lr, T b1, T b2, T eps, T wd, int64_t step) {
    const T b1p = std::max(T(std::pow(b1, T(step))), T(1e-8));
    const T b2p = std::max(T(std::pow(b2, T(step))), T(1e-8));
    const T bc1 = T(1) - b1p, bc2 = T(1) - b2p;
    const T omb1 = T(1) - b1, omb2 = T(1) - b2;
    for (int64_t i = 0; i < n; ++i) {
        m[i] = m[i] * b1 + g[i] * omb1;
        v[i] = v[i] * b2 + (g[i] * g[i]) * omb2;
        const T den = std::sqrt(v[i] / bc2) + eps;
        const T upd = ((m[i] / bc1) / den) * lr;
        if (wd != T(0)) p[i] = (p[i] - upd) - p[i] * (wd * lr);
        else p[i] = p[i] - upd;
    }
}

}  // namespace

#define ORC_EXPORT(SUF, T)                                                                          \
    extern "C" {                                                                                    \
    void orc_matmul_##SUF(const T* A, const T* B, T* C, int64_t M, int64_t N, int64_t K) {          \
        gemm_nn<T>(A, B, C, M, N, K);                                                               \
    }                                                                                               \
    void orc_transpose2d_##SUF(const T* A, T* At, int64_t R, int64_t Cc) { transpose2d<T>(A, At, R, Cc); } \
    void orc_conv2d_fwd_##SUF(const T* x, const T* w, T* y, int64_t B, int64_t C, int64_t H,        \
                              int64_t W, int64_t OC, int64_t kh, int64_t kw, int64_t sh, int64_t sw, \
                              int64_t ph, int64_t pw) {                                             \
        conv2d_fwd<T>(x, w, y, B, C, H, W, OC, kh, kw, sh, sw, ph, pw);                             \
    }                                                                                               \
    void orc_deconv2d_##SUF(const T* dy, const T* w, T* dx, int64_t B, int64_t C, int64_t H,        \
                            int64_t W, int64_t OC, int64_t kh, int64_t kw, int64_t sh, int64_t sw,  \
                            int64_t ph, int64_t pw, int mode) {                                     \
        deconv2d<T>(dy, w, dx, B, C, H, W, OC, kh, kw, sh, sw, ph, pw, mode);                       \
    }                                                                                               \
    void orc_cross_correlation2d_##SUF(const T* x, const T* dy, T* dw, int64_t B, int64_t C,        \
                                       int64_t H, int64_t W, int64_t OC, int64_t kh, int64_t kw,    \
                                       int64_t sh, int64_t sw, int64_t ph, int64_t pw, int mode) {  \
        xcorr2d<T>(x, dy, dw, B, C, H, W, OC, kh, kw, sh, sw, ph, pw, mode);                        \
    }                                                                                               \
    void orc_act_fwd_##SUF(const T* x, T* y, int64_t n, int act) { act_fwd<T>(x, y, n, act); }      \
    void orc_act_bwd_##SUF(const T* dy, const T* aux, T* dx, int64_t n, int act, int sigmoid_math) { \
        act_bwd<T>(dy, aux, dx, n, act, sigmoid_math);                                              \
    }                                                                                               \
    void orc_sum_axes_##SUF(const T* x, const int64_t* shape, int ndim, const int* reduce, T* out) { \
        sum_axes<T>(x, shape, ndim, reduce, out);                                                   \
    }                                                                                               \
    void orc_linear_fwd_##SUF(const T* x, const T* w, const T* b, T* y, int64_t B, int64_t in,      \
                              int64_t out) {                                                        \
        linear_fwd<T>(x, w, b, y, B, in, out);                                                      \
    }                                                                                               \
    void orc_linear_bwd_##SUF(const T* x, const T* w, const T* dz, T* dx, T* dw, T* db, int64_t B,  \
                              int64_t in, int64_t out) {                                            \
        linear_bwd<T>(x, w, dz, dx, dw, db, B, in, out);                                            \
    }                                                                                               \
    void orc_conv_bias_add_##SUF(T* y, const T* bias, int64_t B, int64_t K, int64_t P) {            \
        conv_bias_add<T>(y, bias, B, K, P);                                                         \
    }                                                                                               \
    T orc_softmax_ce_##SUF(const T* logits, const T* targets, T* dlogits, int64_t B, int64_t Cn) {  \
        return softmax_ce<T>(logits, targets, dlogits, B, Cn);                                      \
    }                                                                                               \
    void orc_sgd_step_##SUF(T* p, const T* g, T* mom, int64_t n, T lr, T momentum, T wd, int nest) { \
        sgd_step<T>(p, g, mom, n, lr, momentum, wd, nest);                                          \
    }                                                                                               \
    void orc_adam_step_##SUF(T* p, const T* g, T* m, T* v, int64_t n, T lr, T b1, T b2, T eps,      \
                             T wd, int64_t step) {                                                  \
        adam_step<T>(p, g, m, v, n, lr, b1, b2, eps, wd, step);                                     \
    }                                                                                               \
    }

ORC_EXPORT(f32, float)
ORC_EXPORT(f64, double)
