// Batch normalisation (training and inference forward, backward) and global average pooling:
// the layers of Ferrox's shipped CNN classifier that sit between the convolutions
// (src/nn/layers/norm.rs:214-331, src/nn/layers/pooling.rs:535-619).  The reference expresses them
// as a dozen graph ops (means, broadcasts, sub, mul, sqrt, div ...), each a full pass over the
// activation; here the statistics are two-stage deterministic channel reductions and the
// normalisation is one streaming pass, all HBM-bound.
//
// Tensors are [N, C, P] (P = H*W, or 1 for a [N, F] input); statistics are per channel c over the
// M = N*P other elements, computed like the reference: mean = sum * (1/M), variance =
// sum((x - mean)^2) * (1/M) (biased), std = sqrt(var + eps), y = ((x - mean) / std) * gamma + beta.
#include "fxb_common.cuh"

#include <algorithm>

namespace fxb {

template <typename T> struct NVec;
template <> struct NVec<float> { static constexpr int N = 4; };
template <> struct NVec<double> { static constexpr int N = 2; };

template <typename T> __device__ __forceinline__ T norm_sqrt(T x);
template <> __device__ __forceinline__ float norm_sqrt<float>(float x) { return sqrtf(x); }
template <> __device__ __forceinline__ double norm_sqrt<double>(double x) { return sqrt(x); }

struct NormGeom {
    int64_t N, C, P;
    int parts;
    FastDiv dP;   // by P (or P / V on the vector path)
};

enum : int { BN_SUM = 0, BN_SQDEV = 1, BN_GRADS = 2 };

// Stage one of a channel reduction.  Grid (C, parts): CTA (c, p) walks part p of channel c's N*P
// elements (runs of P contiguous values, one per image) and writes one or two partial sums.
//   BN_SUM    s0 = sum x
//   BN_SQDEV  s0 = sum (x - mean[c])^2
//   BN_GRADS  s0 = sum dz, s1 = sum dz * ((x - mean[c]) / std[c]),  dz = dy * act'(y)
template <typename T, int MODE, int V>
__global__ void __launch_bounds__(256) bn_channel_reduce_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                                const T* __restrict__ yact, const T* __restrict__ mean,
                                                                const T* __restrict__ var, T eps, T* __restrict__ part,
                                                                NormGeom g, int act, int sig_math) {
    __shared__ T red[2][8];
    const int c = blockIdx.x, p = blockIdx.y;
    const uint32_t units = (uint32_t)(g.N * g.P / V);  // vectors (or elements) of this channel
    const uint32_t len = (units + g.parts - 1) / g.parts;
    const uint32_t u0 = (uint32_t)p * len;
    const uint32_t u1 = u0 + len < units ? u0 + len : units;
    T mu = T(0), sd = T(1);
    if (MODE != BN_SUM) mu = __ldg(mean + c);
    if (MODE == BN_GRADS) sd = norm_sqrt<T>(__ldg(var + c) + eps);
    T s0 = T(0), s1 = T(0);
    for (uint32_t u = u0 + threadIdx.x; u < u1; u += 256) {
        uint32_t n, iv;
        g.dP.divmod(u, n, iv);
        const int64_t off = ((int64_t)n * g.C + c) * g.P + (int64_t)iv * V;
        __align__(16) T xv[V], dv[V], yv[V];
        if (V == 1) {
            xv[0] = __ldg(x + off);
            if (MODE == BN_GRADS) { dv[0] = __ldg(dy + off); if (yact) yv[0] = __ldg(yact + off); }
        } else {
            *reinterpret_cast<uint4*>(xv) = __ldg(reinterpret_cast<const uint4*>(x + off));
            if (MODE == BN_GRADS) {
                *reinterpret_cast<uint4*>(dv) = __ldg(reinterpret_cast<const uint4*>(dy + off));
                if (yact) *reinterpret_cast<uint4*>(yv) = __ldg(reinterpret_cast<const uint4*>(yact + off));
            }
        }
#pragma unroll
        for (int e = 0; e < V; ++e) {
            if (MODE == BN_SUM) {
                s0 += xv[e];
            } else if (MODE == BN_SQDEV) {
                const T d = xv[e] - mu;
                s0 += d * d;
            } else {
                T dz = dv[e];
                if (yact) dz *= act_grad_factor<T>(yv[e], act, sig_math);
                s0 += dz;
                s1 += dz * ((xv[e] - mu) / sd);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s0 += __shfl_xor_sync(0xffffffffu, s0, o);
        if (MODE == BN_GRADS) s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { red[0][warp] = s0; red[1][warp] = s1; }
    __syncthreads();
    if (threadIdx.x == 0) {
        T a = T(0), b = T(0);
        for (int w = 0; w < 8; ++w) { a += red[0][w]; b += red[1][w]; }
        part[((int64_t)p * 2 + 0) * g.C + c] = a;
        if (MODE == BN_GRADS) part[((int64_t)p * 2 + 1) * g.C + c] = b;
    }
}

// The same stage one for P == 1 (a [N, F] input): the channel is the contiguous index, so a CTA takes 32
// consecutive channels x 8 row lanes (coalesced rows) and adds the eight lanes in lane order.
template <typename T, int MODE>
__global__ void __launch_bounds__(256) bn_column_reduce_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                               const T* __restrict__ yact, const T* __restrict__ mean,
                                                               const T* __restrict__ var, T eps, T* __restrict__ part,
                                                               NormGeom g, int act, int sig_math) {
    __shared__ T red[2][8][33];
    const int cl = threadIdx.x & 31, rl = threadIdx.x >> 5;
    const int64_t c = (int64_t)blockIdx.x * 32 + cl;
    const int p = blockIdx.y;
    const uint32_t rows = (uint32_t)g.N;
    const uint32_t len = (rows + g.parts - 1) / g.parts;
    const uint32_t r0 = (uint32_t)p * len;
    const uint32_t r1 = r0 + len < rows ? r0 + len : rows;
    T s0 = T(0), s1 = T(0);
    if (c < g.C) {
        T mu = T(0), sd = T(1);
        if (MODE != BN_SUM) mu = __ldg(mean + c);
        if (MODE == BN_GRADS) sd = norm_sqrt<T>(__ldg(var + c) + eps);
        for (uint32_t r = r0 + rl; r < r1; r += 8) {
            const int64_t off = (int64_t)r * g.C + c;
            const T xv = __ldg(x + off);
            if (MODE == BN_SUM) {
                s0 += xv;
            } else if (MODE == BN_SQDEV) {
                const T d = xv - mu;
                s0 += d * d;
            } else {
                T dz = __ldg(dy + off);
                if (yact) dz *= act_grad_factor<T>(__ldg(yact + off), act, sig_math);
                s0 += dz;
                s1 += dz * ((xv - mu) / sd);
            }
        }
    }
    red[0][rl][cl] = s0;
    red[1][rl][cl] = s1;
    __syncthreads();
    if (rl == 0 && c < g.C) {
        T a = T(0), b = T(0);
        for (int w = 0; w < 8; ++w) { a += red[0][w][cl]; b += red[1][w][cl]; }
        part[((int64_t)p * 2 + 0) * g.C + c] = a;
        if (MODE == BN_GRADS) part[((int64_t)p * 2 + 1) * g.C + c] = b;
    }
}

// Stage two: adds the partial sums in part order and derives the per-channel result.
//   BN_SUM    out0 = mean;   running_mean <- (1 - momentum) * running_mean + momentum * mean
//   BN_SQDEV  out0 = variance; running_var likewise
//   BN_GRADS  out0 = dbeta = sum dz,  out1 = dgamma = sum dz * xhat
template <typename T, int MODE>
__global__ void __launch_bounds__(256) bn_channel_finish_kernel(const T* __restrict__ part, T* __restrict__ out0,
                                                                T* __restrict__ out1, T* __restrict__ running, int C,
                                                                int parts, T inv_m, T momentum, T one_minus_momentum) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    T a = T(0), b = T(0);
    for (int p = 0; p < parts; ++p) {
        a += part[((int64_t)p * 2 + 0) * C + c];
        if (MODE == BN_GRADS) b += part[((int64_t)p * 2 + 1) * C + c];
    }
    if (MODE == BN_GRADS) {
        out0[c] = a;
        if (out1) out1[c] = b;
    } else {
        const T v = a * inv_m;
        out0[c] = v;
        if (running) running[c] = running[c] * one_minus_momentum + v * momentum;
    }
}

// y = act(((x - mean) / sqrt(var + eps)) * gamma + beta), one vector of V elements per thread step.
template <typename T, int V>
__global__ void __launch_bounds__(256) bn_apply_kernel(const T* __restrict__ x, const T* __restrict__ mean,
                                                       const T* __restrict__ var, const T* __restrict__ gamma,
                                                       const T* __restrict__ beta, T eps, T* __restrict__ y, int64_t nunits,
                                                       FastDiv dP, FastDiv dC, int act) {
    for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < nunits; u += (int64_t)gridDim.x * blockDim.x) {
        uint32_t q, iv, n, c;
        dP.divmod((uint32_t)u, q, iv);
        dC.divmod(q, n, c);
        const T mu = __ldg(mean + c), sd = norm_sqrt<T>(__ldg(var + c) + eps);
        const T ga = gamma ? __ldg(gamma + c) : T(1), be = beta ? __ldg(beta + c) : T(0);
        __align__(16) T xv[V], r[V];
        if (V == 1) xv[0] = __ldg(x + u);
        else *reinterpret_cast<uint4*>(xv) = __ldg(reinterpret_cast<const uint4*>(x + u * V));
#pragma unroll
        for (int e = 0; e < V; ++e) r[e] = act_apply<T>(((xv[e] - mu) / sd) * ga + be, act);
        if (V == 1) y[u] = r[0];
        else *reinterpret_cast<uint4*>(y + u * V) = *reinterpret_cast<const uint4*>(r);
    }
}

// dx = (gamma / std) * (dz - dbeta / M - xhat * dgamma / M),  dz = dy * act'(y), xhat = (x - mean) / std.
template <typename T, int V>
__global__ void __launch_bounds__(256) bn_backward_apply_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                                const T* __restrict__ yact, const T* __restrict__ mean,
                                                                const T* __restrict__ var, const T* __restrict__ gamma,
                                                                const T* __restrict__ dbeta, const T* __restrict__ dgamma,
                                                                T eps, T inv_m, T* __restrict__ dx, int64_t nunits, FastDiv dP,
                                                                FastDiv dC, int act, int sig_math) {
    for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < nunits; u += (int64_t)gridDim.x * blockDim.x) {
        uint32_t q, iv, n, c;
        dP.divmod((uint32_t)u, q, iv);
        dC.divmod(q, n, c);
        const T mu = __ldg(mean + c), sd = norm_sqrt<T>(__ldg(var + c) + eps);
        const T ga = gamma ? __ldg(gamma + c) : T(1);
        const T mb = __ldg(dbeta + c) * inv_m, mg = __ldg(dgamma + c) * inv_m;
        __align__(16) T xv[V], dv[V], yv[V], r[V];
        if (V == 1) {
            xv[0] = __ldg(x + u);
            dv[0] = __ldg(dy + u);
            if (yact) yv[0] = __ldg(yact + u);
        } else {
            *reinterpret_cast<uint4*>(xv) = __ldg(reinterpret_cast<const uint4*>(x + u * V));
            *reinterpret_cast<uint4*>(dv) = __ldg(reinterpret_cast<const uint4*>(dy + u * V));
            if (yact) *reinterpret_cast<uint4*>(yv) = __ldg(reinterpret_cast<const uint4*>(yact + u * V));
        }
#pragma unroll
        for (int e = 0; e < V; ++e) {
            T dz = dv[e];
            if (yact) dz *= act_grad_factor<T>(yv[e], act, sig_math);
            const T xhat = (xv[e] - mu) / sd;
            r[e] = (ga / sd) * ((dz - mb) - xhat * mg);
        }
        if (V == 1) dx[u] = r[0];
        else *reinterpret_cast<uint4*>(dx + u * V) = *reinterpret_cast<const uint4*>(r);
    }
}

// Global average pooling: y[n, c] = sum over the P values of the plane * (1/P); one warp per plane.
template <typename T, int V>
__global__ void __launch_bounds__(256) gap_forward_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t planes, int P,
                                                          T inv_p) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t pl = warp0; pl < planes; pl += nwarps) {
        const T* src = x + pl * P;
        T a0 = T(0), a1 = T(0);
        if (V == 1) {
            int i = lane;
            for (; i + 32 < P; i += 64) { a0 += __ldg(src + i); a1 += __ldg(src + i + 32); }
            if (i < P) a0 += __ldg(src + i);
        } else {
            for (int i = lane; i < P / V; i += 32) {
                __align__(16) T v[V];
                *reinterpret_cast<uint4*>(v) = __ldg(reinterpret_cast<const uint4*>(src + (int64_t)i * V));
#pragma unroll
                for (int e = 0; e < V; e += 2) { a0 += v[e]; a1 += v[e + 1]; }
            }
        }
        T s = a0 + a1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) y[pl] = s * inv_p;
    }
}

// dx[n, c, :] = dy[n, c] * (1/P)
template <typename T, int V>
__global__ void __launch_bounds__(256) gap_backward_kernel(const T* __restrict__ dy, T* __restrict__ dx, int64_t nunits,
                                                           FastDiv dP, T inv_p) {
    for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < nunits; u += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t pl = dP.div((uint32_t)u);
        const T v = __ldg(dy + pl) * inv_p;
        if (V == 1) {
            dx[u] = v;
        } else {
            __align__(16) T r[V];
#pragma unroll
            for (int e = 0; e < V; ++e) r[e] = v;
            *reinterpret_cast<uint4*>(dx + u * V) = *reinterpret_cast<const uint4*>(r);
        }
    }
}

// ------------------------------------------------------------------------------------------ host side
static int bn_parts(const Context* c, int64_t C, int64_t per_channel) {
    // aim for four CTAs per SM; every part keeps at least 4096 elements so that its reduction is amortised
    int64_t parts = ((int64_t)c->sm_count * 4 + C - 1) / C;
    parts = std::min<int64_t>(parts, std::max<int64_t>(1, per_channel / 4096));
    return (int)std::max<int64_t>(1, std::min<int64_t>(parts, 1024));
}
static size_t bn_ws_bytes(const Context* c, int64_t N, int64_t C, int64_t P, size_t elem) {
    return (size_t)bn_parts(c, C, N * P) * 2 * (size_t)C * elem;
}
static int stream_grid(const Context* c, int64_t units) {
    return (int)std::max<int64_t>(1, std::min<int64_t>((units + 255) / 256, (int64_t)c->sm_count * 16));
}

template <typename T>
static int bn_check(Context* c, int64_t N, int64_t C, int64_t P, const void* ws, size_t ws_bytes) {
    FXB_CHECK_ARG(c, N > 0 && C > 0 && P > 0, "BatchNorm requires at least 2D input [batch_size, features] with positive sizes");
    FXB_CHECK_ARG(c, N * C * P < ((int64_t)1 << 31) && C <= 65535 * 32, "BatchNorm tensor has more than 2^31-1 elements");
    if (ws == nullptr || ws_bytes < bn_ws_bytes(c, N, C, P, sizeof(T)))
        return fail(c, FXB_ERR_WORKSPACE, "BatchNorm: workspace smaller than fxb_batch_norm_workspace_bytes");
    return FXB_OK;
}

template <typename T, int MODE>
static int bn_reduce(Context* c, const T* x, const T* dy, const T* yact, const T* mean, const T* var, T eps, T* part,
                     int64_t N, int64_t C, int64_t P, bool vec, int act, cudaStream_t st) {
    NormGeom g;
    g.N = N; g.C = C; g.P = P;
    g.parts = bn_parts(c, C, N * P);
    dim3 grid((unsigned)C, (unsigned)g.parts);
    constexpr int V = NVec<T>::N;
    if (P == 1) {
        dim3 cgrid((unsigned)((C + 31) / 32), (unsigned)g.parts);
        bn_column_reduce_kernel<T, MODE><<<cgrid, 256, 0, st>>>(x, dy, yact, mean, var, eps, part, g, act, c->sigmoid_grad_math);
        return launch_status(c, "bn_column_reduce_kernel");
    }
    if (vec) {
        g.dP.init((uint32_t)(P / V));
        bn_channel_reduce_kernel<T, MODE, V><<<grid, 256, 0, st>>>(x, dy, yact, mean, var, eps, part, g, act, c->sigmoid_grad_math);
    } else {
        g.dP.init((uint32_t)P);
        bn_channel_reduce_kernel<T, MODE, 1><<<grid, 256, 0, st>>>(x, dy, yact, mean, var, eps, part, g, act, c->sigmoid_grad_math);
    }
    return launch_status(c, "bn_channel_reduce_kernel");
}

template <typename T>
static bool bn_vec_ok(int64_t P, std::initializer_list<const void*> ptrs) {
    if (P % NVec<T>::N != 0) return false;
    for (const void* p : ptrs)
        if (p != nullptr && (reinterpret_cast<uintptr_t>(p) & 15) != 0) return false;
    return true;
}

template <typename T>
static int bn_forward_impl(Context* c, const T* x, const T* gamma, const T* beta, T* y, T* batch_mean, T* batch_var,
                           T* running_mean, T* running_var, int64_t N, int64_t C, int64_t P, double eps, double momentum,
                           int training, int act, void* ws, size_t ws_bytes, cudaStream_t st) {
    FXB_CHECK_ARG(c, act >= FXB_ACT_NONE && act <= FXB_ACT_TANH, "Unknown activation code");
    FXB_CHECK_ARG(c, x && y, "BatchNorm got a null buffer");
    const bool vec = bn_vec_ok<T>(P, {x, y});
    constexpr int V = NVec<T>::N;
    const T* mean = running_mean;
    const T* var = running_var;
    if (training) {
        int rc = bn_check<T>(c, N, C, P, ws, ws_bytes);
        if (rc) return rc;
        FXB_CHECK_ARG(c, batch_mean && batch_var, "BatchNorm training forward needs batch_mean and batch_var outputs");
        T* part = static_cast<T*>(ws);
        const int parts = bn_parts(c, C, N * P);
        const T inv_m = (T)(1.0 / (double)(N * P));
        const T mom = (T)momentum, omm = (T)(1.0 - momentum);
        const int fb = (int)((C + 255) / 256);
        rc = bn_reduce<T, BN_SUM>(c, x, nullptr, nullptr, nullptr, nullptr, T(0), part, N, C, P, vec, 0, st);
        if (rc) return rc;
        bn_channel_finish_kernel<T, BN_SUM><<<fb, 256, 0, st>>>(part, batch_mean, nullptr, running_mean, (int)C, parts, inv_m, mom, omm);
        rc = launch_status(c, "bn_channel_finish_kernel");
        if (rc) return rc;
        rc = bn_reduce<T, BN_SQDEV>(c, x, nullptr, nullptr, batch_mean, nullptr, T(0), part, N, C, P, vec, 0, st);
        if (rc) return rc;
        bn_channel_finish_kernel<T, BN_SQDEV><<<fb, 256, 0, st>>>(part, batch_var, nullptr, running_var, (int)C, parts, inv_m, mom, omm);
        rc = launch_status(c, "bn_channel_finish_kernel");
        if (rc) return rc;
        mean = batch_mean;
        var = batch_var;
    } else {
        FXB_CHECK_ARG(c, N > 0 && C > 0 && P > 0 && N * C * P < ((int64_t)1 << 31), "BatchNorm: bad shape");
        FXB_CHECK_ARG(c, running_mean && running_var, "BatchNorm inference forward needs the running statistics");
    }
    const int64_t units = N * C * P / (vec ? V : 1);
    if (vec)
        bn_apply_kernel<T, V><<<stream_grid(c, units), 256, 0, st>>>(x, mean, var, gamma, beta, (T)eps, y, units, FastDiv((uint32_t)(P / V)),
                                                                     FastDiv((uint32_t)C), act);
    else
        bn_apply_kernel<T, 1><<<stream_grid(c, units), 256, 0, st>>>(x, mean, var, gamma, beta, (T)eps, y, units, FastDiv((uint32_t)P),
                                                                     FastDiv((uint32_t)C), act);
    return launch_status(c, "bn_apply_kernel");
}

template <typename T>
static int bn_backward_impl(Context* c, const T* x, const T* dy, const T* yact, const T* gamma, const T* batch_mean,
                            const T* batch_var, T* dx, T* dgamma, T* dbeta, int64_t N, int64_t C, int64_t P, double eps,
                            int act, void* ws, size_t ws_bytes, cudaStream_t st) {
    int rc = bn_check<T>(c, N, C, P, ws, ws_bytes);
    if (rc) return rc;
    FXB_CHECK_ARG(c, x && dy && batch_mean && batch_var && dgamma && dbeta, "BatchNorm backward got a null buffer");
    FXB_CHECK_ARG(c, act == FXB_ACT_NONE || yact != nullptr, "Fused activation backward needs the layer output");
    const T* ya = act == FXB_ACT_NONE ? nullptr : yact;
    const bool vec = bn_vec_ok<T>(P, {x, dy, ya, dx});
    constexpr int V = NVec<T>::N;
    T* part = static_cast<T*>(ws);
    const int parts = bn_parts(c, C, N * P);
    rc = bn_reduce<T, BN_GRADS>(c, x, dy, ya, batch_mean, batch_var, (T)eps, part, N, C, P, vec, act, st);
    if (rc) return rc;
    bn_channel_finish_kernel<T, BN_GRADS><<<(int)((C + 255) / 256), 256, 0, st>>>(part, dbeta, dgamma, nullptr, (int)C, parts, T(0), T(0), T(0));
    rc = launch_status(c, "bn_channel_finish_kernel");
    if (rc || dx == nullptr) return rc;
    const T inv_m = (T)(1.0 / (double)(N * P));
    const int64_t units = N * C * P / (vec ? V : 1);
    if (vec)
        bn_backward_apply_kernel<T, V><<<stream_grid(c, units), 256, 0, st>>>(x, dy, ya, batch_mean, batch_var, gamma, dbeta, dgamma, (T)eps,
                                                                              inv_m, dx, units, FastDiv((uint32_t)(P / V)),
                                                                              FastDiv((uint32_t)C), act, c->sigmoid_grad_math);
    else
        bn_backward_apply_kernel<T, 1><<<stream_grid(c, units), 256, 0, st>>>(x, dy, ya, batch_mean, batch_var, gamma, dbeta, dgamma, (T)eps,
                                                                              inv_m, dx, units, FastDiv((uint32_t)P), FastDiv((uint32_t)C),
                                                                              act, c->sigmoid_grad_math);
    return launch_status(c, "bn_backward_apply_kernel");
}

template <typename T>
static int gap_forward_impl(Context* c, const T* x, T* y, int64_t N, int64_t C, int64_t H, int64_t W, cudaStream_t st) {
    FXB_CHECK_ARG(c, N >= 0 && C > 0 && H > 0 && W > 0, "GlobalAvgPool2d requires 4D input [batch, channels, height, width]");
    const int64_t planes = N * C, P = H * W;
    if (planes == 0) return FXB_OK;
    FXB_CHECK_ARG(c, x && y, "GlobalAvgPool2d got a null buffer");
    FXB_CHECK_ARG(c, P < ((int64_t)1 << 31), "GlobalAvgPool2d plane has more than 2^31-1 elements");
    constexpr int V = NVec<T>::N;
    const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((planes + 7) / 8, (int64_t)c->sm_count * 16));
    const T inv_p = (T)(1.0 / (double)P);
    if (P % V == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0)
        gap_forward_kernel<T, V><<<blocks, 256, 0, st>>>(x, y, planes, (int)P, inv_p);
    else
        gap_forward_kernel<T, 1><<<blocks, 256, 0, st>>>(x, y, planes, (int)P, inv_p);
    return launch_status(c, "gap_forward_kernel");
}

template <typename T>
static int gap_backward_impl(Context* c, const T* dy, T* dx, int64_t N, int64_t C, int64_t H, int64_t W, cudaStream_t st) {
    FXB_CHECK_ARG(c, N >= 0 && C > 0 && H > 0 && W > 0, "GlobalAvgPool2d requires 4D input [batch, channels, height, width]");
    const int64_t planes = N * C, P = H * W, total = planes * P;
    if (total == 0) return FXB_OK;
    FXB_CHECK_ARG(c, dy && dx, "GlobalAvgPool2d got a null buffer");
    FXB_CHECK_ARG(c, total < ((int64_t)1 << 31), "GlobalAvgPool2d tensor has more than 2^31-1 elements");
    constexpr int V = NVec<T>::N;
    const T inv_p = (T)(1.0 / (double)P);
    if (P % V == 0 && (reinterpret_cast<uintptr_t>(dx) & 15) == 0)
        gap_backward_kernel<T, V><<<stream_grid(c, total / V), 256, 0, st>>>(dy, dx, total / V, FastDiv((uint32_t)(P / V)), inv_p);
    else
        gap_backward_kernel<T, 1><<<stream_grid(c, total), 256, 0, st>>>(dy, dx, total, FastDiv((uint32_t)P), inv_p);
    return launch_status(c, "gap_backward_kernel");
}

}  // namespace fxb

using namespace fxb;
#define CTX(h) reinterpret_cast<fxb::Context*>(h)
#define ST(s) static_cast<cudaStream_t>(s)
#define NEED_HANDLE(h) \
    if ((h) == nullptr) return fxb::fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null ferrox_b200 handle")

#define FXB_NORM_API(SUF, T)                                                                                            \
    extern "C" int fxb_batch_norm_fwd_##SUF(fxb_handle_t h, const T* x, const T* gamma, const T* beta, T* y,            \
                                            T* batch_mean, T* batch_var, T* running_mean, T* running_var, int64_t N,    \
                                            int64_t C, int64_t P, double eps, double momentum, int training, int act,   \
                                            void* ws, size_t wsb, fxb_stream_t s) {                                     \
        NEED_HANDLE(h);                                                                                                 \
        return bn_forward_impl<T>(CTX(h), x, gamma, beta, y, batch_mean, batch_var, running_mean, running_var, N, C, P, \
                                  eps, momentum, training, act, ws, wsb, ST(s));                                        \
    }                                                                                                                   \
    extern "C" int fxb_batch_norm_bwd_##SUF(fxb_handle_t h, const T* x, const T* dy, const T* y, const T* gamma,        \
                                            const T* batch_mean, const T* batch_var, T* dx, T* dgamma, T* dbeta,        \
                                            int64_t N, int64_t C, int64_t P, double eps, int act, void* ws, size_t wsb, \
                                            fxb_stream_t s) {                                                           \
        NEED_HANDLE(h);                                                                                                 \
        return bn_backward_impl<T>(CTX(h), x, dy, y, gamma, batch_mean, batch_var, dx, dgamma, dbeta, N, C, P, eps,     \
                                   act, ws, wsb, ST(s));                                                                \
    }                                                                                                                   \
    extern "C" int fxb_global_avg_pool_fwd_##SUF(fxb_handle_t h, const T* x, T* y, int64_t N, int64_t C, int64_t H,     \
                                                 int64_t W, fxb_stream_t s) {                                           \
        NEED_HANDLE(h);                                                                                                 \
        return gap_forward_impl<T>(CTX(h), x, y, N, C, H, W, ST(s));                                                    \
    }                                                                                                                   \
    extern "C" int fxb_global_avg_pool_bwd_##SUF(fxb_handle_t h, const T* dy, T* dx, int64_t N, int64_t C, int64_t H,   \
                                                 int64_t W, fxb_stream_t s) {                                           \
        NEED_HANDLE(h);                                                                                                 \
        return gap_backward_impl<T>(CTX(h), dy, dx, N, C, H, W, ST(s));                                                 \
    }

FXB_NORM_API(f32, float)
FXB_NORM_API(f64, double)

extern "C" size_t fxb_batch_norm_workspace_bytes(fxb_handle_t h, int64_t N, int64_t C, int64_t P, size_t elem) {
    if (!h || N <= 0 || C <= 0 || P <= 0) return 0;
    return bn_ws_bytes(CTX(h), N, C, P, elem);
}
