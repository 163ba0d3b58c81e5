// CUDA-core kernels for the two shapes of the hot path that do not fill a tensor-core tile:
//   * "skinny" linear layers (at most 16 output features: the classifier head), forward and backward;
//   * convolutions with at most 32 values of C*R*S (the first layer of a CNN on RGB input),
//     forward and filter gradient.
// They are bound by memory traffic, not arithmetic, so plain FMAs in the operand type (f32 or f64)
// are used; accumulation order is fixed, results do not depend on scheduling.
#pragma once
#include "fxb_operands.cuh"

namespace fxb {

constexpr int SKINNY_MAXO = 16;

// Y[b][o] = act(sum_i X[b][i] * W[o][i] + bias[o]); one block of 256 threads per R rows: every thread takes the
// columns i = t, t + 256, ..., loads the `out` weights of a column once and uses them for the R rows (the
// weights are what the blocks re-read from L2: R = 4 quarters that traffic); the partial sums are added by
// warp shuffles and then over the eight warps in warp order.  The result does not depend on R.
template <typename T, int R>
__global__ void __launch_bounds__(256) skinny_linear_fwd_kernel(const T* __restrict__ X, const T* __restrict__ W,
                                                                const T* __restrict__ bias, T* __restrict__ Y, int B, int in,
                                                                int out, int act) {
    __shared__ T red[R][8][SKINNY_MAXO];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b0 = blockIdx.x * R;
    T acc[R][SKINNY_MAXO];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int o = 0; o < SKINNY_MAXO; ++o) acc[r][o] = T(0);
#pragma unroll 2
    for (int i = threadIdx.x; i < in; i += 256) {
        T xv[R];
#pragma unroll
        for (int r = 0; r < R; ++r) xv[r] = b0 + r < B ? __ldg(X + (int64_t)(b0 + r) * in + i) : T(0);
#pragma unroll
        for (int o = 0; o < SKINNY_MAXO; ++o)
            if (o < out) {
                const T wv = __ldg(W + (int64_t)o * in + i);
#pragma unroll
                for (int r = 0; r < R; ++r) acc[r][o] += xv[r] * wv;
            }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int o = 0; o < SKINNY_MAXO; ++o) {
            T v = acc[r][o];
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            if (lane == 0) red[r][warp][o] = v;
        }
    __syncthreads();
    for (int e = threadIdx.x; e < R * out; e += 256) {
        const int r = e / out, o = e - r * out;
        if (b0 + r < B) {
            const T v = ((red[r][0][o] + red[r][1][o]) + (red[r][2][o] + red[r][3][o])) +
                        ((red[r][4][o] + red[r][5][o]) + (red[r][6][o] + red[r][7][o]));
            Y[(int64_t)(b0 + r) * out + o] = act_apply<T>(v + (bias ? __ldg(bias + o) : T(0)), act);
        }
    }
}

// dX[b][i] = sum_o dZ[b][o] * W[o][i], dZ = dY * act'(Y); grid (ceil(B / rows), ceil(in/256)): a block keeps the
// `out` weights of its 256 columns in registers and walks over `rows` (<= SKINNY_DX_ROWS) batch rows, so the
// weights are read once per block instead of once per row.
constexpr int SKINNY_DX_ROWS = 32;
template <typename T>
__global__ void __launch_bounds__(256) skinny_linear_dx_kernel(const T* __restrict__ dY, const T* __restrict__ Yact,
                                                               const T* __restrict__ W, T* __restrict__ dX, int B, int in, int out,
                                                               int act, int sig_math, int rows) {
    __shared__ T dz[SKINNY_DX_ROWS * SKINNY_MAXO];
    const int b0 = blockIdx.x * rows;
    const int nr = min(rows, B - b0);
    for (int e = threadIdx.x; e < nr * out; e += 256) {
        T v = __ldg(dY + (int64_t)b0 * out + e);
        if (Yact) v *= act_grad_factor<T>(__ldg(Yact + (int64_t)b0 * out + e), act, sig_math);
        dz[e] = v;
    }
    __syncthreads();
    const int i = blockIdx.y * blockDim.x + threadIdx.x;
    if (i >= in) return;
    T w[SKINNY_MAXO];
#pragma unroll
    for (int o = 0; o < SKINNY_MAXO; ++o) w[o] = o < out ? __ldg(W + (int64_t)o * in + i) : T(0);
    for (int r = 0; r < nr; ++r) {
        T acc = T(0);
#pragma unroll
        for (int o = 0; o < SKINNY_MAXO; ++o)
            if (o < out) acc += dz[r * out + o] * w[o];
        dX[(int64_t)(b0 + r) * in + i] = acc;
    }
}

// Partial dW / db over one chunk of `rows_per_chunk` (<= SKINNY_ROWS) batch rows: part[chunk][o][i] = sum_b dZ[b][o] * X[b][i],
// dbpart[chunk][o] = sum_b dZ[b][o]; grid (ceil(in/256), chunks).  The chunks are added in order afterwards.
constexpr int SKINNY_ROWS = 128;
template <typename T>
__global__ void __launch_bounds__(256) skinny_linear_dw_kernel(const T* __restrict__ X, const T* __restrict__ dY,
                                                               const T* __restrict__ Yact, T* __restrict__ part,
                                                               T* __restrict__ dbpart, int B, int in, int out, int act,
                                                               int sig_math, int rows_per_chunk) {
    __shared__ T dz[SKINNY_ROWS * SKINNY_MAXO];
    const int b0 = blockIdx.y * rows_per_chunk;
    const int rows = min(rows_per_chunk, B - b0);
    for (int e = threadIdx.x; e < rows * out; e += blockDim.x) {
        T v = __ldg(dY + (int64_t)b0 * out + e);
        if (Yact) v *= act_grad_factor<T>(__ldg(Yact + (int64_t)b0 * out + e), act, sig_math);
        dz[e] = v;
    }
    __syncthreads();
    if (blockIdx.x == 0 && dbpart != nullptr && threadIdx.x < out) {
        T s = T(0);
        for (int r = 0; r < rows; ++r) s += dz[r * out + threadIdx.x];
        dbpart[(int64_t)blockIdx.y * out + threadIdx.x] = s;
    }
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= in) return;
    T acc[SKINNY_MAXO];
#pragma unroll
    for (int o = 0; o < SKINNY_MAXO; ++o) acc[o] = T(0);
    const T* xp = X + (int64_t)b0 * in + i;
    int r = 0;
    for (; r + 8 <= rows; r += 8) {  // eight row loads in flight, then the FMAs in row order
        T xv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) xv[u] = __ldg(xp + (int64_t)(r + u) * in);
#pragma unroll
        for (int u = 0; u < 8; ++u)
#pragma unroll
            for (int o = 0; o < SKINNY_MAXO; ++o)
                if (o < out) acc[o] += dz[(r + u) * out + o] * xv[u];
    }
    for (; r < rows; ++r) {
        const T xv = __ldg(xp + (int64_t)r * in);
#pragma unroll
        for (int o = 0; o < SKINNY_MAXO; ++o)
            if (o < out) acc[o] += dz[r * out + o] * xv;
    }
#pragma unroll
    for (int o = 0; o < SKINNY_MAXO; ++o)
        if (o < out) part[((int64_t)blockIdx.y * out + o) * in + i] = acc[o];
}

// ------------------------------------------------------------------------------------------
// Convolutions with C*R*S <= 32.
constexpr int SMALLC_K = 32;  // padded length of one im2col row

// Column k of an im2col row -> offset of (c, r, s) inside one image and the window displacement (r, s).
struct SmallcTap { int off, r, s, valid; };
__device__ __forceinline__ SmallcTap smallc_tap(const ConvGeom& g, int k) {
    SmallcTap t;
    const int c = k / g.RS, rs = k - c * g.RS;
    t.r = rs / g.S;
    t.s = rs - t.r * g.S;
    t.off = (c * g.H + t.r) * g.W + t.s;
    t.valid = k < g.CRS ? 1 : 0;
    return t;
}

// Y[n][o][p] = act(bias[o] + sum_k W[o][k] * im2col(p)[k]); one thread per output pixel, filter and the
// column table in shared memory.
template <typename T, bool EMIT>
__global__ void __launch_bounds__(256) smallc_conv_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                              const T* __restrict__ bias, T* __restrict__ y, ConvGeom g,
                                                              int64_t npix, int act, SlabEmit em) {
    extern __shared__ __align__(16) unsigned char smallc_smem[];
    __shared__ SmallcTap taps[SMALLC_K];
    T* ws = reinterpret_cast<T*>(smallc_smem);  // [K][SMALLC_K], zero padded
    for (int e = threadIdx.x; e < g.K * SMALLC_K; e += blockDim.x) {
        const int o = e / SMALLC_K, k = e - o * SMALLC_K;
        ws[e] = k < g.CRS ? __ldg(w + (int64_t)o * g.CRS + k) : T(0);
    }
    if (threadIdx.x < SMALLC_K) taps[threadIdx.x] = smallc_tap(g, threadIdx.x);
    __syncthreads();
    const int64_t pix = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (pix >= npix) return;
    uint32_t n, p, oy, ox;
    g.dP.divmod((uint32_t)pix, n, p);
    g.dOW.divmod(p, oy, ox);
    const int y0 = (int)oy * g.sh - g.ph, x0 = (int)ox * g.sw - g.pw;
    const T* xn = x + (int64_t)n * g.C * g.HW + (int64_t)y0 * g.W + x0;
    T v[SMALLC_K];
#pragma unroll
    for (int k = 0; k < SMALLC_K; ++k) {
        const SmallcTap t = taps[k];
        const bool in = t.valid && (unsigned)(y0 + t.r) < (unsigned)g.H && (unsigned)(x0 + t.s) < (unsigned)g.W;
        v[k] = in ? __ldg(xn + t.off) : T(0);
    }
    T* yo = y + (int64_t)n * g.K * g.P + p;
    if constexpr (!EMIT) {
        for (int o = 0; o < g.K; ++o) {
            const T* wr = ws + o * SMALLC_K;
            T a0 = T(0), a1 = T(0);
#pragma unroll
            for (int k = 0; k < SMALLC_K; k += 2) {
                a0 += wr[k] * v[k];
                a1 += wr[k + 1] * v[k + 1];
            }
            yo[(int64_t)o * g.P] = act_apply<T>((a0 + a1) + (bias ? __ldg(bias + o) : T(0)), act);
        }
    } else {
        // the same values also as the next convolution's class slabs: four consecutive channels per 16-byte chunk
        const int64_t eoff = slab_cell_offset(em, (int)n, (int)oy, (int)ox);
        for (int o4 = 0; o4 < g.K; o4 += 4) {
            float r[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int o = o4 + j;
                r[j] = 0.f;
                if (o < g.K) {
                    const T* wr = ws + o * SMALLC_K;
                    T a0 = T(0), a1 = T(0);
#pragma unroll
                    for (int k = 0; k < SMALLC_K; k += 2) {
                        a0 += wr[k] * v[k];
                        a1 += wr[k + 1] * v[k + 1];
                    }
                    const T t = act_apply<T>((a0 + a1) + (bias ? __ldg(bias + o) : T(0)), act);
                    yo[(int64_t)o * g.P] = t;
                    r[j] = (float)t;
                }
            }
            store_split4(em.hi, em.lo, eoff + (int64_t)(o4 >> 2) * em.plane_stride, r[0], r[1], r[2], r[3]);
        }
    }
}

// Filter gradient, K <= 64: block = 256 threads = 64 output channels x 4 groups of 8 im2col columns.
// Each block walks over tiles of 32 output pixels (grid-stride), staging dZ[32][64] and the im2col rows
// [32][32] in shared memory, and writes its partial sums part[block][o][32] and dbpart[block][o].
template <typename T>
__global__ void __launch_bounds__(256) smallc_conv_wgrad_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                                const T* __restrict__ yact, T* __restrict__ part,
                                                                T* __restrict__ dbpart, ConvGeom g, int64_t npix, int act,
                                                                int sig_math) {
    __shared__ T dz_s[32][65];
    __shared__ T in_s[32][SMALLC_K];
    const int o = threadIdx.x & 63, kg = threadIdx.x >> 6;
    T acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = T(0);
    T dbs = T(0);
    const int64_t ntiles = (npix + 31) / 32;
    // Staging roles, fixed per thread: dZ element (channel (tid>>5) + 8j, pixel tid&31);
    // im2col element (pixel (tid>>5) + 8j, column tid&31).
    const int lane_e = threadIdx.x & 31, row_e = threadIdx.x >> 5;
    const SmallcTap tap = smallc_tap(g, lane_e);
    // Software pipeline: the global loads of tile t+1 are issued into registers before the FMAs of tile t,
    // so their latency overlaps the arithmetic; the activation factor is applied when they are stored.
    T rdy[8], rya[8], rx[4];
    auto fetch = [&](int64_t tile) {
        const int64_t pix0 = tile * 32;
        const int64_t pix = pix0 + lane_e;
        const bool pin = pix < npix;
        uint32_t n = 0, p = 0;
        if (pin) g.dP.divmod((uint32_t)pix, n, p);
        const int64_t base = (int64_t)n * g.K * g.P + p;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int oc = row_e + 8 * j;
            rdy[j] = T(0);
            rya[j] = T(0);
            if (pin && oc < g.K) {
                const int64_t src = base + (int64_t)oc * g.P;
                rdy[j] = __ldg(dy + src);
                if (yact) rya[j] = __ldg(yact + src);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t pixj = pix0 + row_e + 8 * j;
            T v = T(0);
            if (tap.valid && pixj < npix) {
                uint32_t n2, p2, oy, ox;
                g.dP.divmod((uint32_t)pixj, n2, p2);
                g.dOW.divmod(p2, oy, ox);
                const int y0 = (int)oy * g.sh - g.ph, x0 = (int)ox * g.sw - g.pw;
                if ((unsigned)(y0 + tap.r) < (unsigned)g.H && (unsigned)(x0 + tap.s) < (unsigned)g.W)
                    v = __ldg(x + (int64_t)n2 * g.C * g.HW + (int64_t)y0 * g.W + x0 + tap.off);
            }
            rx[j] = v;
        }
    };
    if ((int64_t)blockIdx.x < ntiles) fetch(blockIdx.x);
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            T v = rdy[j];
            if (yact) v *= act_grad_factor<T>(rya[j], act, sig_math);
            dz_s[lane_e][row_e + 8 * j] = v;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) in_s[row_e + 8 * j][lane_e] = rx[j];
        __syncthreads();
        if (tile + gridDim.x < ntiles) fetch(tile + gridDim.x);
#pragma unroll 4
        for (int px = 0; px < 32; ++px) {
            const T d = dz_s[px][o];
            if (kg == 0) dbs += d;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += d * in_s[px][kg * 8 + j];
        }
        __syncthreads();
    }
    T* pr = part + ((int64_t)blockIdx.x * 64 + o) * SMALLC_K + kg * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) pr[j] = acc[j];
    if (kg == 0 && dbpart != nullptr) dbpart[(int64_t)blockIdx.x * 64 + o] = dbs;
}

// The same filter gradient for f32 with a 4 x 8 register tile per thread: block = 4 pixel sub-streams x
// (16 groups of 4 output channels x 4 groups of 8 im2col columns).  Per pixel a thread reads its four dZ values
// and eight im2col values with three 16-byte shared-memory loads and issues 32 FMAs, so the kernel is bound by
// the FMA pipe instead of by shared-memory bandwidth.  Same partial-sum layout as the generic kernel
// (part[block][64][32], dbpart[block][64]); the four sub-streams are added in order at the end.
__global__ void __launch_bounds__(256) smallc_conv_wgrad_f32_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                                                                    const float* __restrict__ yact, float* __restrict__ part,
                                                                    float* __restrict__ dbpart, ConvGeom g, int64_t npix, int act,
                                                                    int sig_math) {
    // dz_s [32][68] and in_s [32][32] during the main loop; the sub-stream partials [4][64][33] at the end
    __shared__ __align__(16) float smem_f[4 * 64 * 33];
    float (*dz_s)[68] = reinterpret_cast<float (*)[68]>(smem_f);
    float (*in_s)[SMALLC_K] = reinterpret_cast<float (*)[SMALLC_K]>(smem_f + 32 * 68);
    const int sub = threadIdx.x >> 6, w64 = threadIdx.x & 63;
    const int og = w64 & 15, kg = w64 >> 4;
    float acc[4][8];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[a][j] = 0.f;
    float dbs[4] = {0.f, 0.f, 0.f, 0.f};
    const int64_t ntiles = (npix + 31) / 32;
    // staging roles: dZ values (pixel tid&31, channels 8*(tid>>5) .. +7); im2col values (pixel (tid>>5) + 8j, column tid&31)
    const int lane_e = threadIdx.x & 31, row_e = threadIdx.x >> 5;
    const SmallcTap tap = smallc_tap(g, lane_e);
    float rdy[8], rya[8], rx[4];
    auto fetch = [&](int64_t tile) {
        const int64_t pix0 = tile * 32;
        const int64_t pix = pix0 + lane_e;
        const bool pin = pix < npix;
        uint32_t n = 0, p = 0;
        if (pin) g.dP.divmod((uint32_t)pix, n, p);
        const int64_t base = (int64_t)n * g.K * g.P + p;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int oc = row_e * 8 + j;
            rdy[j] = 0.f;
            rya[j] = 0.f;
            if (pin && oc < g.K) {
                const int64_t src = base + (int64_t)oc * g.P;
                rdy[j] = __ldg(dy + src);
                if (yact) rya[j] = __ldg(yact + src);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t pixj = pix0 + row_e + 8 * j;
            float v = 0.f;
            if (tap.valid && pixj < npix) {
                uint32_t n2, p2, oy, ox;
                g.dP.divmod((uint32_t)pixj, n2, p2);
                g.dOW.divmod(p2, oy, ox);
                const int y0 = (int)oy * g.sh - g.ph, x0 = (int)ox * g.sw - g.pw;
                if ((unsigned)(y0 + tap.r) < (unsigned)g.H && (unsigned)(x0 + tap.s) < (unsigned)g.W)
                    v = __ldg(x + (int64_t)n2 * g.C * g.HW + (int64_t)y0 * g.W + x0 + tap.off);
            }
            rx[j] = v;
        }
    };
    if ((int64_t)blockIdx.x < ntiles) fetch(blockIdx.x);
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[j] = rdy[j];
            if (yact) v[j] *= act_grad_factor<float>(rya[j], act, sig_math);
        }
        *reinterpret_cast<float4*>(&dz_s[lane_e][row_e * 8]) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(&dz_s[lane_e][row_e * 8 + 4]) = make_float4(v[4], v[5], v[6], v[7]);
#pragma unroll
        for (int j = 0; j < 4; ++j) in_s[row_e + 8 * j][lane_e] = rx[j];
        __syncthreads();
        if (tile + gridDim.x < ntiles) fetch(tile + gridDim.x);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int px = sub * 8 + q;
            const float4 d = *reinterpret_cast<const float4*>(&dz_s[px][og * 4]);
            const float4 c0 = *reinterpret_cast<const float4*>(&in_s[px][kg * 8]);
            const float4 c1 = *reinterpret_cast<const float4*>(&in_s[px][kg * 8 + 4]);
            const float dd[4] = {d.x, d.y, d.z, d.w};
            const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                if (kg == 0) dbs[a] += dd[a];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[a][j] += dd[a] * cc[j];
            }
        }
        __syncthreads();
    }
    // add the four pixel sub-streams in order
    float (*red)[64][33] = reinterpret_cast<float (*)[64][33]>(smem_f);
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int j = 0; j < 8; ++j) red[sub][og * 4 + a][kg * 8 + j] = acc[a][j];
    __syncthreads();
    for (int e = threadIdx.x; e < 64 * SMALLC_K; e += 256) {
        const int o = e >> 5, k = e & 31;
        part[((int64_t)blockIdx.x * 64 + o) * SMALLC_K + k] = (red[0][o][k] + red[1][o][k]) + (red[2][o][k] + red[3][o][k]);
    }
    if (dbpart != nullptr) {
        __syncthreads();
        if (kg == 0) {
#pragma unroll
            for (int a = 0; a < 4; ++a) red[sub][og * 4 + a][0] = dbs[a];
        }
        __syncthreads();
        if (threadIdx.x < 64)
            dbpart[(int64_t)blockIdx.x * 64 + threadIdx.x] =
                (red[0][threadIdx.x][0] + red[1][threadIdx.x][0]) + (red[2][threadIdx.x][0] + red[3][threadIdx.x][0]);
    }
}

// dW[o][k] = sum over blocks of part[b][o][k] (k < CRS), eight interleaved running sums combined as a fixed tree.
template <typename T>
__global__ void __launch_bounds__(256) smallc_wgrad_finish_kernel(const T* __restrict__ part, T* __restrict__ dw, int K, int CRS,
                                                                  int rows) {
    __shared__ T red[8][32];
    const int el = threadIdx.x & 31, bl = threadIdx.x >> 5;
    const int e = blockIdx.x * 32 + el;  // index into [64][SMALLC_K]
    T a0 = T(0), a1 = T(0), a2 = T(0), a3 = T(0);
    int b = bl;
    for (; b + 24 < rows; b += 32) {  // four independent loads in flight
        a0 += __ldg(part + (int64_t)b * 64 * SMALLC_K + e);
        a1 += __ldg(part + (int64_t)(b + 8) * 64 * SMALLC_K + e);
        a2 += __ldg(part + (int64_t)(b + 16) * 64 * SMALLC_K + e);
        a3 += __ldg(part + (int64_t)(b + 24) * 64 * SMALLC_K + e);
    }
    for (; b < rows; b += 8) a0 += __ldg(part + (int64_t)b * 64 * SMALLC_K + e);
    red[bl][el] = (a0 + a1) + (a2 + a3);
    __syncthreads();
    const int o = e / SMALLC_K, k = e - o * SMALLC_K;
    if (bl == 0 && o < K && k < CRS)
        dw[(int64_t)o * CRS + k] =
            ((red[0][el] + red[1][el]) + (red[2][el] + red[3][el])) + ((red[4][el] + red[5][el]) + (red[6][el] + red[7][el]));
}

}  // namespace fxb
